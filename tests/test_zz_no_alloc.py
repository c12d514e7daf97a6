"""The allocation-free H128-rotated prefill linear (mixfp4_gemm_h128_static) against the
workspace-taking entry point it mirrors (mixfp4_gemm with rotation_block = 128).

Some hosts cannot allocate device memory around a call -- a server whose memory arena was
sized once at start-up, a plugin inside someone else's allocator -- so this entry point
keeps its staging buffer inside the library.  Both entry points run the same kernels, so
their outputs must agree (checked with the 1e-3 relative Frobenius bound the other GEMM
tests use, and in fact bit for bit); the second call, on different data, shows that
nothing left in the shared buffer by the first call leaks into the next result.
This file is named to be collected last."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import _native as nat
from mixfp4_b200 import synth

pytestmark = pytest.mark.gpu


def _both(x, packed, out_dtype=torch.float32):
    lib = nat.lib()
    m, k = x.shape
    n = packed.n
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = (packed.codes.data_ptr(), packed.scales.data_ptr(), packed.fmt.data_ptr(), packed.global_scale.data_ptr())
    y_static = torch.empty((m, n), dtype=out_dtype, device="cuda")
    rc = lib.mixfp4_gemm_h128_static(x.data_ptr(), m, x.stride(0), *args, n, k, packed.layout_code, None,
                                     y_static.data_ptr(), nat.DTYPE_CODE[out_dtype], n, status.data_ptr(), stream)
    assert rc == 0, lib.mixfp4_status_string(rc)
    nbytes = lib.mixfp4_gemm_workspace_bytes(m, n, k)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    y_ws = torch.empty((m, n), dtype=out_dtype, device="cuda")
    rc = lib.mixfp4_gemm(x.data_ptr(), m, x.stride(0), *args, n, k, packed.layout_code, None, 128, y_ws.data_ptr(),
                         nat.DTYPE_CODE[out_dtype], n, ws.data_ptr(), nbytes, status.data_ptr(), 0, stream)
    assert rc == 0, lib.mixfp4_status_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return y_static, y_ws


def test_static_scratch_variant_matches_workspace_variant_twice():
    w = synth.student_t_weight(384, 1024, 31)
    packed, _, _ = mx.quantize_packed(mx.apply_transform(w.cuda(), "H128"), rotation="H128")
    for call, (m, seed) in enumerate(((256, 41), (130, 42))):      # two calls in a row, new data and shape
        x = synth.activations(m, 1024, seed, outlier_fraction=0.01).cuda()
        y_static, y_ws = _both(x, packed)
        a, b = y_static.cpu().numpy(), y_ws.cpu().numpy()
        assert oracle.relative_l2(a, b) <= 1e-3, f"call {call}"
        assert np.array_equal(a, b), f"call {call}"
        assert np.isfinite(a).all()


def test_static_scratch_variant_rejects_oversize_requests():
    lib = nat.lib()
    cap = lib.mixfp4_gemm_h128_static_max_bytes()
    assert cap == 8 << 20
    one = 256                       # never dereferenced: the size check comes first
    too_big_m = cap // (4096 * 2) + 1
    rc = lib.mixfp4_gemm_h128_static(one, too_big_m, 4096, one, one, one, one, 128, 4096, 0, None, one, nat.F32, 128,
                                     None, None)
    assert rc == -10
    assert b"capacity" in lib.mixfp4_status_string(rc)
