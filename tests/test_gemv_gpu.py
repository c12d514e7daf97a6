"""GPU parity of the decode-shape dequant-linear (mixfp4_gemv through the C ABI).

Oracle: y* = x.float() @ dequant.float().T with the reference's bf16 dequantized weight
(double accumulation).  Tolerance: relative Frobenius error <= 1e-3 on fp32 outputs (the
bound the task states); bf16 outputs must be within 1 bf16 ulp of bf16(y*)."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3


def oracle_linear(x: torch.Tensor, w: torch.Tensor):
    ref = oracle.quantize(w.float().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    return oracle.linear(x.float().numpy(), wq)


@pytest.mark.parametrize("m", [1, 2, 4, 7, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(256, 512), (50, 70), (33, 131), (128, 1000), (64, 4096), (16, 14336)])
def test_gemv_matches_oracle(m, n, k):
    w = synth.student_t_weight(n, k, seed=n + k)
    x = synth.activations(m, k, seed=m)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed, out_dtype=torch.float32).cpu().numpy()
    ystar = oracle_linear(x, w)
    assert y.shape == (m, n)
    assert oracle.relative_l2(y, ystar) <= TOL


def test_gemv_fp32_accumulation_is_tight():
    # the only deviation from the oracle is fp32 summation order: expect ~1e-6, far below 1e-3
    w, x = synth.config1(0, n=512, k=4096, m=16)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed, out_dtype=torch.float32).cpu().numpy()
    assert oracle.relative_l2(y, oracle_linear(x, w)) <= 2e-6


def test_gemv_bf16_output_within_one_ulp():
    w = synth.student_t_weight(256, 1024, 5)
    x = synth.activations(4, 1024, 6)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed).float().cpu().numpy()           # bf16 out
    ystar = oracle_linear(x, w)
    ulp = np.abs(ystar) * 2.0 ** -7 + 1e-30
    assert np.all(np.abs(y - ystar) <= ulp)


def test_gemv_unaligned_x_and_leading_dims():
    w = synth.student_t_weight(48, 200, 7)
    packed, _, _ = mx.quantize_packed(w.cuda())
    base = synth.activations(6, 260, 8).cuda()
    x = base[:, 3:203]                                   # unaligned rows, K % 8 == 0 but stride 260
    y = mx.mixfp4_linear(x, packed, out_dtype=torch.float32).cpu().numpy()
    assert oracle.relative_l2(y, oracle_linear(x.cpu(), w)) <= TOL
    x3 = synth.activations(6, 200, 9).reshape(2, 3, 200).cuda()
    y3 = mx.mixfp4_linear(x3, packed, out_dtype=torch.float32)
    assert y3.shape == (2, 3, 48)


def test_module_from_linear_with_bias_and_rotation():
    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 96, bias=True).to(torch.bfloat16)
    layer = mx.MixFP4Linear.from_linear(lin, rotation="H128")
    x = synth.activations(3, 256, 10).cuda()
    y = layer(x, out_dtype=torch.float32).cpu().numpy()
    # oracle: rotate both operands the way the layer does, quantize the rotated weight
    wr = oracle.f32_to_bf16_bits(oracle.fwht(lin.weight.detach().float().numpy(), 128, bf16_stages=True))
    wq = oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(oracle.bf16_bits_to_f32(wr)), "bf16"))
    xr = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.fwht(x.float().cpu().numpy(), 128)))
    ystar = oracle.linear(xr, wq) + lin.bias.detach().float().numpy()
    assert oracle.relative_l2(y, ystar) <= TOL


def test_gemv_property_linearity_full_size():
    """Full-size layer (gate/up 14336 x 4096): y(x1 + x2) == y(x1) + y(x2) for inputs whose
    sum is exact in bf16, and a row subset matches the oracle."""
    w = synth.student_t_weight(14336, 4096, 3)
    packed, _, _ = mx.quantize_packed(w.cuda())
    g = torch.Generator().manual_seed(1)
    x1 = torch.randint(-8, 9, (1, 4096), generator=g).to(torch.bfloat16)
    x2 = torch.randint(-8, 9, (1, 4096), generator=g).to(torch.bfloat16)
    f = lambda t: mx.mixfp4_linear(t.cuda(), packed, out_dtype=torch.float32).double().cpu()
    lhs, rhs = f(x1 + x2), f(x1) + f(x2)
    assert float((lhs - rhs).norm() / rhs.norm()) <= 1e-5
    rows = slice(7000, 7064)
    wq = oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(w.float().numpy()), "bf16"))
    ystar = oracle.linear(x1.float().numpy(), wq[rows])
    assert oracle.relative_l2(f(x1)[:, rows].numpy(), ystar) <= TOL
