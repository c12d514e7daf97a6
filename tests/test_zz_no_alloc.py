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


def _oracle_rotated_linear(x: torch.Tensor, w_rotated: torch.Tensor) -> np.ndarray:
    """fp32 matmul of bf16(FWHT_fp32(x)) with the reference's dequantized (rotated) weight."""
    ref = oracle.quantize(w_rotated.float().cpu().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    xr = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.fwht(x.float().cpu().numpy(), 128)))
    return oracle.linear(xr, wq)


@pytest.mark.parametrize("m,n,k", [(256, 384, 1024), (32, 512, 4096)])
def test_static_scratch_variant_matches_the_oracle(m, n, k):
    """Against the oracle itself, not only against the sibling entry point.  The second shape is one
    the GEMM runs with K split over several CTAs per tile: the fp32 partial sums then sit in the
    library's array behind the rotated activations."""
    lib = nat.lib()
    w = synth.student_t_weight(n, k, 7 + m)
    wr = mx.apply_transform(w.cuda(), "H128")
    packed, _, _ = mx.quantize_packed(wr, rotation="H128")
    if (m, n, k) == (32, 512, 4096):
        # the split-K plan asks for more than the staging area: partial sums are in use
        assert lib.mixfp4_gemm_workspace_bytes(m, n, k) > m * k * 2 + 256 + 256
    for call in range(2):
        x = synth.activations(m, k, 50 + call, outlier_fraction=0.01).cuda()
        y_static, y_ws = _both(x, packed)
        ystar = _oracle_rotated_linear(x, wr)
        assert oracle.relative_l2(y_static.cpu().numpy(), ystar) <= 1e-3, f"call {call}"
        assert torch.equal(y_static, y_ws)


def test_static_scratch_variant_checks_every_argument_before_it_enqueues_anything():
    lib = nat.lib()
    w = synth.student_t_weight(128, 256, 3)
    packed, _, _ = mx.quantize_packed(mx.apply_transform(w.cuda(), "H128"), rotation="H128")
    x = synth.activations(64, 256, 4).cuda()
    good, _ = _both(x, packed)
    y = torch.full((64, 128), 7.0, device="cuda")
    args = [x.data_ptr(), 64, 256, packed.codes.data_ptr(), packed.scales.data_ptr(), packed.fmt.data_ptr(),
            packed.global_scale.data_ptr(), 128, 256, 0, None, y.data_ptr(), nat.F32, 128, None,
            torch.cuda.current_stream().cuda_stream]
    for pos, bad, want in ((9, 7, -5), (12, nat.F16, -4), (5, None, -1), (3, packed.codes.data_ptr() + 8, -3)):
        call = list(args)
        call[pos] = bad
        assert lib.mixfp4_gemm_h128_static(*call) == want
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())                # nothing ran
    # and the shared array still serves a correct call afterwards
    again, _ = _both(x, packed)
    assert torch.equal(again, good)


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
