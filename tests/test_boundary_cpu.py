"""CPU-only checks of the drop-in boundary: the library loads without a GPU, exports every
symbol the header declares, validates arguments before touching CUDA, and the Python
surface raises the reference's exception types."""

import ctypes
import os
import re

import pytest
import torch

import mixfp4_b200 as mx
from mixfp4_b200 import _native as nat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mixfp4_b200.h")).read()
    declared = set(re.findall(r"MIXFP4_API\s+[\w\s\*]+?\b(mixfp4_\w+)\s*\(", header))
    assert declared == set(nat.EXPORTED)
    handle = nat.lib()
    for name in declared:
        assert getattr(handle, name) is not None
    assert handle.mixfp4_abi_version() == 3
    assert handle.mixfp4_padded_k(70) == 128 and handle.mixfp4_padded_k(4096) == 4096


def test_library_has_no_torch_or_libcuda_dependency():
    import subprocess
    out = subprocess.run(["ldd", os.path.join(ROOT, "mixfp4_b200", "libmixfp4_b200.so")],
                         capture_output=True, text=True).stdout
    assert "libtorch" not in out and "libcuda.so" not in out and "libc10" not in out


def test_c_abi_argument_validation_needs_no_gpu():
    h = nat.lib()
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    assert h.mixfp4_amax(None, nat.BF16, 4, 16, 16, one, None) == -1
    assert h.mixfp4_amax(one, nat.BF16, 0, 16, 16, one, None) == -2
    assert h.mixfp4_amax(one, 7, 4, 16, 16, one, None) == -4
    args = [one, nat.BF16, 4, 64, 64, 0, one, one, one, one, one, None, None, None, None, None, 0, None]
    bad = list(args); bad[0] = None
    assert h.mixfp4_quantize(*bad) == -1
    bad = list(args); bad[4] = 32
    assert h.mixfp4_quantize(*bad) == -2          # ldx < k
    bad = list(args); bad[5] = 9
    assert h.mixfp4_quantize(*bad) == -5          # unknown mode
    bad = list(args); bad[7] = ctypes.c_void_p(20)
    assert h.mixfp4_quantize(*bad) == -3          # codes not 8-byte aligned
    assert h.mixfp4_fwht(one, one, nat.BF16, 4, 64, 64, 64, 48, None, 0, None) == -5
    assert h.mixfp4_gemv(one, 17, 64, one, one, one, one, 8, 64, 0, None, one, nat.F32, 8, 0, None) == -2
    assert h.mixfp4_gemv(one, 1, 64, one, one, one, one, 8, 64, 0, None, one, nat.F16, 8, 0, None) == -4
    assert h.mixfp4_gemv(one, 1, 64, one, one, None, one, 8, 64, 0, None, one, nat.F32, 8, 0, None) == -1   # canonical needs fmt
    assert h.mixfp4_gemv(one, 1, 64, one, one, None, one, 8, 64, 3, None, one, nat.F32, 8, 0, None) == -5   # unknown layout
    seg = (nat.GemvSegment * 1)()
    seg[0].codes = seg[0].scales = seg[0].global_scale = seg[0].y = 16
    seg[0].ldy, seg[0].n = 8, 8
    assert h.mixfp4_gemv_grouped(one, 1, 64, 64, seg, 0, 1, nat.F32, 0, None) == -2     # count out of range
    assert h.mixfp4_gemv_grouped(one, 17, 64, 64, seg, 1, 1, nat.F32, 0, None) == -2    # more than 16 rows of x
    assert h.mixfp4_gemv_grouped(one, 1, 64, 64, None, 1, 1, nat.F32, 0, None) == -1
    assert h.mixfp4_gemv_grouped(one, 1, 64, 64, seg, 1, 0, nat.F32, 0, None) == -5     # grouped launches: kernel or stream layout
    assert h.mixfp4_gemv_grouped(one, 17, 64, 64, seg, 1, 2, nat.F32, 0, None) == -2
    assert h.mixfp4_gemv_grouped(one, 1, 64, 64, seg, 1, 1, nat.F16, 0, None) == -4
    seg[0].ldy = 4
    assert h.mixfp4_gemv_grouped(one, 1, 64, 64, seg, 1, 1, nat.F32, 0, None) == -2     # ldy < n
    assert h.mixfp4_select_regions(one, one, 8, 256, 8, 4, None, None) == -1
    assert h.mixfp4_select_regions(one, one, 8, 256, 8, 3, one, None) == -5      # region width must be 2 or 4 blocks
    assert h.mixfp4_select_regions(one, one, 8, 64, 8, 4, one, None) == -5       # one region along K, several rows
    assert h.mixfp4_select_regions(one, one, 0, 64, 1, 4, one, None) == -2
    bad = list(args); bad[5] = 4
    assert h.mixfp4_quantize(*bad) == -5          # modes are 0..3
    assert h.mixfp4_fake_quantize(one, nat.BF16, 4, 64, 64, 0, one, None, 64, None) == -1
    assert h.mixfp4_fake_quantize(one, nat.BF16, 4, 64, 64, 0, one, one, 32, None) == -2      # ldy < k
    assert h.mixfp4_fake_quantize(one, nat.BF16, 4, 64, 64, 3, one, one, 64, None) == -5      # no format bits to be given
    assert h.mixfp4_fake_quantize(one, nat.BF16, 4, 64, 96, 0, one, one, 64, None) == -2      # in place needs equal strides
    a4 = [one, 64, 64, one, one, one, one, 64, 64, 0, None, 0, 0, one, nat.F32, 64, None, 0, None, 0, None]
    assert h.mixfp4_gemm_a4(*a4) == -7                                                          # workspace is required
    bad = list(a4); bad[11] = 64
    assert h.mixfp4_gemm_a4(*bad) == -5                                                         # rotation 0 or 128
    bad = list(a4); bad[0] = None
    assert h.mixfp4_gemm_a4(*bad) == -1
    assert h.mixfp4_gemm_workspace_bytes(64, 64, 64) >= 64 * 64 * 2 + 4
    assert h.mixfp4_repack(one, one, None, 4, 64, 1, one, one, None, None) == -1
    # stream layout: sizes, argument checks, the x-fits predicate (host arithmetic only)
    assert h.mixfp4_stream_bytes(33, 70) == 3 * 1 * 1152 and h.mixfp4_stream_bytes(4096, 4096) == 256 * 32 * 1152
    assert h.mixfp4_stream_bytes(0, 64) == 0
    assert h.mixfp4_repack_stream(one, one, None, 4, 64, one, None) == -1
    assert h.mixfp4_repack_stream(one, one, one, 4, 0, one, None) == -2
    assert h.mixfp4_repack_from_stream(one, 4, 64, one, one, None, None) == -1
    assert h.mixfp4_gemv(one, 1, 64, one, None, None, one, 8, 64, 2, None, None, nat.F32, 8, 0, None) == -1   # stream: scales and fmt may be NULL, y not
    assert h.mixfp4_gemv(one, 1, 64, one, None, None, one, 8, 64, 1, None, one, nat.F32, 8, 0, None) == -1   # kernel layout needs scales
    assert h.mixfp4_gemv_x_fits(1, 4096, 3) == 1 and h.mixfp4_gemv_x_fits(8, 14336, 1) == 0
    assert h.mixfp4_gemv_x_fits(17, 64, 1) == 0 and h.mixfp4_gemv_x_fits(1, 64, 4) == 0
    assert h.mixfp4_set_wait_limit_ns(0) == -2 and h.mixfp4_set_wait_limit_ns(2_000_000_000) == 0
    assert h.mixfp4_comm_buffer_bytes(2, 100) == 2 * 2 * 100 * 8 and h.mixfp4_comm_buffer_bytes(9, 100) == 0
    assert h.mixfp4_comm_open_local(None, None) == -1
    # the GEMM entry points check every argument before they enqueue anything
    st = [one, 64, 64, one, one, one, one, 64, 64, 0, None, one, nat.F32, 64, None, None]
    bad = list(st); bad[9] = 7
    assert h.mixfp4_gemm_h128_static(*bad) == -5                                                # unknown layout
    bad = list(st); bad[12] = nat.F16
    assert h.mixfp4_gemm_h128_static(*bad) == -4                                                # f32 or bf16 out
    bad = list(st); bad[3] = ctypes.c_void_p(24)
    assert h.mixfp4_gemm_h128_static(*bad) == -3                                                # codes 16-byte aligned
    bad = list(st); bad[5] = None
    assert h.mixfp4_gemm_h128_static(*bad) == -1                                                # canonical needs fmt
    bad = list(st); bad[1] = 1 << 40
    assert h.mixfp4_gemm_h128_static(*bad) == -2                                                # m beyond 2^31
    bad = list(st); bad[1] = 1 << 20; bad[7] = 16; bad[13] = 16
    assert h.mixfp4_gemm_h128_static(*bad) == -10                                               # beyond the built-in array
    bad = list(a4); bad[12] = 3
    assert h.mixfp4_gemm_a4(*bad) == -5                                                         # activation mode 0..2
    bad = list(a4); bad[14] = nat.F16
    assert h.mixfp4_gemm_a4(*bad) == -4
    assert h.mixfp4_decode_table(None, one, None) == -1
    assert h.mixfp4_status_string(-3).decode().startswith("pointer or stride")


def test_reference_error_conventions():
    # project_quant/candidates.py:46-58 and core.py:77-80,105-106; tests/test_quant_core.py:52-53
    x = torch.zeros((9, 70))
    with pytest.raises(ValueError, match="fixes scale_group_size=16"):
        mx.quant_mixfp4_granularity(x, scale_group_size=64)
    with pytest.raises(TypeError, match="floating point"):
        mx.quant_mixfp4_granularity(torch.zeros((4, 16), dtype=torch.int32))
    with pytest.raises(ValueError, match="row dimension"):
        mx.quant_mixfp4_granularity(torch.zeros(16))
    with pytest.raises(ValueError, match=r"\[N,K\]"):
        mx.quant_mixfp4_granularity(torch.zeros((2, 3, 16)))
    with pytest.raises(ValueError, match="operand_role"):
        mx.quant_mixfp4_granularity(x, operand_role="bias")
    with pytest.raises(ValueError, match="unknown selector"):
        mx.quant_mixfp4_granularity(x, selector="best")
    with pytest.raises(ValueError, match="unknown scale_rule"):
        mx.quant_mixfp4_granularity(x, scale_rule="other")
    with pytest.raises(ValueError, match="N8K64"):
        mx.quant_mixfp4_granularity(x, selector="output_aware")
    with pytest.raises(ValueError, match="permutation length"):
        mx.quant_mixfp4_granularity(x, permutation=torch.arange(3))
    with pytest.raises(ValueError, match="invalid for"):
        mx.quant_mixfp4_granularity(x, format_region="n3k7")
    with pytest.raises(ValueError, match="invalid for"):
        mx.quant_mixfp4_granularity(x, format_region="m8k64")            # an activation region on a weight
    with pytest.raises(ValueError, match="invalid for"):
        mx.quant_mixfp4_granularity(x, format_region="m16k16")           # an activation region on a weight
    with pytest.raises(NotImplementedError):
        mx.quant_mixfp4_granularity(x, scale_rule="four_over_six")
    with pytest.raises(ValueError, match="unknown transform"):
        mx.get_transform("H7")


def test_packed_byte_accounting():
    # 4 bits + 8/16 + 1/16 bits per element = 0.5703125 B
    assert mx.packed_nbytes(4096, 4096) == 9_568_256 + 4
    assert mx.packed_nbytes(14336, 4096) == 33_488_896 + 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from mixfp4_b200 import build
    monkeypatch.setattr(nat, "_lib", None)
    monkeypatch.setattr(build, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        nat.lib()


def test_model_walk_helpers_follow_the_reference_rules():
    # project_quant/modeling.py:55-68: heads are skipped, the type is the last name component
    from torch import nn
    from mixfp4_b200 import convert

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.o_proj = nn.Linear(8, 8), nn.Linear(8, 8)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Attn(), Attn()])
            self.score_head = nn.Linear(8, 2)
            self.lm_head = nn.Linear(8, 16)
            self.proj = nn.Linear(8, 8)

    names = [n for n, _ in convert.named_linears(Net())]
    assert names == ["layers.0.q_proj", "layers.0.o_proj", "layers.1.q_proj", "layers.1.o_proj", "proj"]
    assert convert.module_type("layers.1.q_proj") == "q_proj" and convert.module_type("proj") == "other_linear"
    assert convert.layer_index("model.layers.17.mlp.down_proj") == 17 and convert.layer_index("proj") is None
    assert convert.quantize_model_weights(Net(), "fp16") == []          # high-precision modes convert nothing
    with pytest.raises(ValueError, match="packed checkpoint"):
        convert.load_packed(Net(), {"format": "something else", "version": 1, "layers": {}})


def test_activation_modes_follow_the_reference_tables():
    import torch
    from mixfp4_b200 import quant
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    for mode in ("bf16", "fp16", "high_precision"):
        assert quant.fake_quantize_activations(x, mode) is x          # the hook leaves these alone (modeling.py:669)
    with pytest.raises(ValueError):
        quant.fake_quantize_activations(x, "n8k64")                   # a weight region (region.py:42-70)
    with pytest.raises(ValueError):
        quant.fake_quantize_activations(x, "n8k16")                   # a weight region too
    assert quant.region_shape("m8k64", "activation_a") == (8, 4)
    assert quant.region_shape("m16k16", "activation_a") == (16, 1)
    assert quant.region_shape("n8k16", "weight_b") == (8, 1)
    assert quant.region_shape("layer", "weight_b") == quant.region_shape("layer", "activation_a") == (1, 0)
