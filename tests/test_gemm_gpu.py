"""GPU parity of the prefill-shape dequant-linear (mixfp4_gemm, tcgen05) through the C ABI.

Oracle: y* = x.float() @ dequant.float().T with the reference's bf16 dequantized weight
(double accumulation).  Tolerance: relative Frobenius error <= 1e-3 on fp32 outputs; bf16
outputs within one bf16 ulp of y*.  With the H128 rotation the oracle activation is
bf16(FWHT_fp32(x)) (one rounding) and the weight is quantized after the reference's own
bf16 rotation."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import linear as mxl
from mixfp4_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3


def dequant_oracle(w: torch.Tensor) -> np.ndarray:
    return oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(w.float().numpy()), "bf16"))


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64), (128, 128, 128), (128, 128, 512), (256, 256, 1024), (17, 128, 256), (160, 50, 70),
    (300, 200, 131), (129, 257, 1000), (512, 1024, 4096), (384, 128, 14336),
])
def test_gemm_matches_oracle(m, n, k):
    w = synth.student_t_weight(n, k, seed=n + k)
    x = synth.activations(m, k, seed=m, outlier_fraction=0.01)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed, out_dtype=torch.float32)
    assert mxl.gemm_status() == 0
    ystar = oracle.linear(x.float().numpy(), dequant_oracle(w))
    assert y.shape == (m, n)
    assert oracle.relative_l2(y.cpu().numpy(), ystar) <= TOL


@pytest.mark.parametrize("layout", ["canonical", "kernel"])
@pytest.mark.parametrize("m,n,k", [
    (257, 256, 64), (512, 256, 128), (512, 100, 131), (700, 300, 1024), (1024, 1000, 512), (513, 640, 4096),
    (1000, 3600, 192),      # enough tiles for pairs of 128-row CTAs, too few for pairs of 256-row CTAs
    (1024, 14336, 128),     # pairs of 256-row CTAs
])
def test_gemm_cta_pair_shapes(m, n, k, layout):
    # more than 256 tokens: two CTAs share every decoded weight tile; ragged token and weight
    # tiles, an odd number of token tiles (the second CTA of the last pair has no rows), K tails
    w = synth.student_t_weight(n, k, seed=7 * n + k)
    x = synth.activations(m, k, seed=m, outlier_fraction=0.01)
    packed = mx.quantize_packed(w.cuda())[0]
    if layout == "kernel":
        packed = packed.to_kernel_layout().with_decode_table()
    for dt in (torch.float32, torch.bfloat16):
        y = mx.mixfp4_linear(x.cuda(), packed, out_dtype=dt)
        assert mxl.gemm_status() == 0
        ystar = oracle.linear(x.float().numpy(), dequant_oracle(w))
        if dt == torch.float32:
            assert oracle.relative_l2(y.cpu().numpy(), ystar) <= TOL
        else:
            # one bf16 ulp of the exact result, plus fp32 summation noise where the result cancels to ~0
            assert np.all(np.abs(y.float().cpu().numpy() - ystar) <= np.abs(ystar) * 2.0 ** -7 + 2e-6 * np.abs(ystar).max())


def test_gemm_fp32_accumulation_is_tight():
    w, x = synth.config1(0, n=256, k=4096, m=256)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed, out_dtype=torch.float32).cpu().numpy()
    assert oracle.relative_l2(y, oracle.linear(x.float().numpy(), dequant_oracle(w))) <= 5e-6


def test_gemm_bf16_output_within_one_ulp():
    w = synth.student_t_weight(256, 512, 5)
    x = synth.activations(200, 512, 6)
    packed, _, _ = mx.quantize_packed(w.cuda())
    y = mx.mixfp4_linear(x.cuda(), packed).float().cpu().numpy()
    ystar = oracle.linear(x.float().numpy(), dequant_oracle(w))
    assert np.all(np.abs(y - ystar) <= np.abs(ystar) * 2.0 ** -7 + 1e-30)


def test_gemm_agrees_with_gemv_rows():
    """The two kernels decode the same weights: a GEMM row equals the GEMV of that row up to
    fp32 summation order."""
    w = synth.student_t_weight(512, 2048, 11)
    x = synth.activations(130, 2048, 12)
    packed, _, _ = mx.quantize_packed(w.cuda())
    big = mx.mixfp4_linear(x.cuda(), packed, out_dtype=torch.float32)
    small = mx.mixfp4_linear(x[:16].cuda(), packed, out_dtype=torch.float32)
    assert float((big[:16] - small).norm() / small.norm()) <= 1e-5


def test_gemm_unaligned_x_uses_workspace():
    w = synth.student_t_weight(128, 200, 7)
    packed, _, _ = mx.quantize_packed(w.cuda())
    base = synth.activations(150, 260, 8).cuda()
    x = base[:, 3:203]                                   # unaligned start, pitch not 16-byte
    y = mx.mixfp4_linear(x, packed, out_dtype=torch.float32).cpu().numpy()
    ystar = oracle.linear(x.float().cpu().numpy(), dequant_oracle(w))
    assert oracle.relative_l2(y, ystar) <= TOL


@pytest.mark.parametrize("m,n,k", [(256, 384, 1024), (130, 100, 640)])
def test_gemm_with_online_h128_rotation(m, n, k):
    """Config 3: weights rotated offline (the reference's bf16 FWHT), then quantized;
    activations with outlier channels rotated on the fly."""
    w = synth.student_t_weight(n, k, 21)
    x = synth.activations(m, k, 22, outlier_fraction=0.01)
    lin = torch.nn.Linear(k, n, bias=False)
    lin.weight.data = w
    layer = mx.MixFP4Linear.from_linear(lin, rotation="H128")
    y = layer(x.cuda(), out_dtype=torch.float32).cpu().numpy()
    assert mxl.gemm_status() == 0
    wr = oracle.fwht(w.float().numpy(), 128, bf16_stages=True)                    # bf16 values
    wq = oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(wr), "bf16"))
    xr = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.fwht(x.float().numpy(), 128)))
    ystar = oracle.linear(xr, wq)
    assert oracle.relative_l2(y, ystar) <= TOL
    # and the rotation is (nearly) transparent: against the un-rotated product the only
    # difference is quantization error of the rotated vs plain weight, both small
    plain = oracle.linear(x.float().numpy(), w.float().numpy())
    assert oracle.relative_l2(y, plain) <= 0.2


@pytest.mark.parametrize("m,n,k", [(32, 512, 4096), (100, 300, 14336), (128, 1000, 2048), (17, 4096, 4096)])
def test_gemm_split_k_small_m(m, n, k):
    # few output tiles and a long K: several CTAs share a tile along K, fp32 partials are summed
    # in split order; with and without room for the partials (NULL workspace: one CTA per tile)
    from mixfp4_b200 import _native as nat
    w = synth.student_t_weight(n, k, seed=n + k)
    x = synth.activations(m, k, seed=m, outlier_fraction=0.01).cuda()
    packed = mx.quantize_packed(w.cuda())[0].to_kernel_layout().with_decode_table()
    ystar = oracle.linear(x.float().cpu().numpy(), dequant_oracle(w))
    y = mx.mixfp4_linear(x, packed, out_dtype=torch.float32)
    assert mxl.gemm_status() == 0
    assert oracle.relative_l2(y.cpu().numpy(), ystar) <= TOL
    assert torch.equal(y, mx.mixfp4_linear(x, packed, out_dtype=torch.float32))     # deterministic
    if m > 16:
        y2 = torch.empty_like(y)
        st = nat.lib().mixfp4_gemm(x.data_ptr(), m, k, packed.codes.data_ptr(), packed.scales.data_ptr(), None,
                                   packed.global_scale.data_ptr(), n, k, nat.LAYOUT_KERNEL, packed.lut.data_ptr(), 0,
                                   y2.data_ptr(), nat.F32, n, None, 0, None, 0, torch.cuda.current_stream().cuda_stream)
        assert st == 0
        assert oracle.relative_l2(y2.cpu().numpy(), ystar) <= TOL


def test_c_abi_workspace_contract():
    from mixfp4_b200 import _native as nat
    lib = nat.lib()
    assert lib.mixfp4_gemm_workspace_bytes(300, 128, 131) >= 300 * 136 * 2
    w = synth.student_t_weight(128, 256, 1).cuda()
    packed, _, _ = mx.quantize_packed(w)
    x = synth.activations(128, 256, 2).cuda()
    y = torch.empty((128, 128), dtype=torch.float32, device="cuda")
    st = lib.mixfp4_gemm(x.data_ptr(), 128, 256, packed.codes.data_ptr(), packed.scales.data_ptr(),
                         packed.fmt.data_ptr(), packed.global_scale.data_ptr(), 128, 256, 0, None, 128, y.data_ptr(),
                         nat.F32, 128, None, 0, None, 0, torch.cuda.current_stream().cuda_stream)
    assert st == -7        # rotation requested without a workspace


def test_gemm_cta_pairs_with_h128_rotation_started_early():
    """A shape the CTA-pair kernel takes, with the rotation pass in front: the GEMM is launched as a programmatic
    dependent of the rotation kernel (set-up and weight loads under the rotation's tail, x loads after its end).
    Six calls back to back on different activations, no synchronisation between them: every result equals the
    allocation-free entry point's (rotation and GEMM as two ordinary launches) bit for bit, and the oracle's
    within the tolerance."""
    from mixfp4_b200 import _native as nat
    m, n, k = 1024, 7168, 1024
    w = synth.student_t_weight(n, k, 77)
    wr = mx.apply_transform(w.cuda(), "H128")
    packed = mx.quantize_packed(wr, rotation="H128")[0].to_stream_layout()
    lib = nat.lib()
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = lib.mixfp4_gemm_workspace_bytes(m, n, k)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    xs = [synth.activations(m, k, 90 + i, outlier_fraction=0.01).cuda() for i in range(6)]
    ys = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in xs]
    args = (packed.codes.data_ptr(), nat.ptr(packed.scales), nat.ptr(packed.fmt), packed.global_scale.data_ptr(), n, k,
            packed.layout_code, nat.ptr(packed.lut))
    for x, y in zip(xs, ys):
        rc = lib.mixfp4_gemm(x.data_ptr(), m, k, *args, 128, y.data_ptr(), nat.BF16, n, ws.data_ptr(), nbytes,
                             status.data_ptr(), 0, stream)
        assert rc == 0, lib.mixfp4_status_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i, (x, y) in enumerate(zip(xs, ys)):
        y_two = torch.empty_like(y)
        rc = lib.mixfp4_gemm_h128_static(x.data_ptr(), m, k, *args, y_two.data_ptr(), nat.BF16, n, status.data_ptr(), stream)
        assert rc == 0, lib.mixfp4_status_string(rc)
        assert torch.equal(y, y_two), f"call {i}"
    wq = oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(wr.float().cpu().numpy()), "bf16"))
    xr = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.fwht(xs[0].float().cpu().numpy(), 128)))
    y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    rc = lib.mixfp4_gemm(xs[0].data_ptr(), m, k, *args, 128, y32.data_ptr(), nat.F32, n, ws.data_ptr(), nbytes,
                         status.data_ptr(), 0, stream)
    assert rc == 0, lib.mixfp4_status_string(rc)
    ystar = oracle.linear(xr, wq)
    assert oracle.relative_l2(y32.cpu().numpy(), ystar) <= TOL
    assert np.all(np.abs(ys[0].float().cpu().numpy() - ystar) <= np.abs(ystar) * 2.0 ** -7 + 1e-4 * np.abs(ystar).max())
    assert int(status.item()) == 0
