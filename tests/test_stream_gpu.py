"""The stream layout (1152-byte chunks of 16 rows x 128 K elements) and the decode kernel that
streams it, through the C ABI.

Layout: a pure permutation of the canonical bytes, checked against a numpy restatement of the
addressing rule and by a round trip.  Linear: the oracle is y* = x.float() @ dequant.float().T on the
reference's bf16 dequantized weight (oracle.linear); fp32 outputs must be within 1e-3 relative
Frobenius error (observed ~1e-6: only the fp32 summation order differs), bf16 outputs within one
bf16 ulp.  Shapes cover ragged row counts, K tails, a single chunk per tile, fewer tiles than SMs,
the BASELINE config-2 layer shapes at M = 1, 4, 16 (the benched path), grouped launches and the
prefill GEMM reading the same buffer."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3


def to_kernel_word(w: np.ndarray) -> np.ndarray:
    """Bit order of a 32-bit code word in the kernel/stream layouts (csrc/decode.cuh)."""
    w = w.astype(np.uint32)
    out = w & np.uint32(0x77777777)
    for i in range(4):
        out |= ((w >> np.uint32(4 * i + 3)) & np.uint32(1)) << np.uint32(8 * i + 7)
        out |= ((w >> np.uint32(4 * (4 + i) + 3)) & np.uint32(1)) << np.uint32(8 * i + 3)
    return out


def numpy_stream(codes: np.ndarray, scales: np.ndarray, fmt: np.ndarray, n: int, kpad: int) -> np.ndarray:
    tiles, subs = (n + 15) // 16, kpad // 128
    out = np.zeros((tiles, subs, 1152), dtype=np.uint8)
    out[:, :, 1024:] = 1                                            # padding rows: scale byte 0x01
    words = to_kernel_word(codes.reshape(n, kpad // 8, 4).copy().view(np.uint32)[..., 0])     # [n, kpad/8]
    bits = (fmt[:, :, None] >> np.arange(8, dtype=np.uint8)) & 1                               # [n, kpad/128, 8]
    sb = (scales & 0x7F) | (bits.reshape(n, -1).astype(np.uint8) << 7)                         # [n, kpad/16]
    for r in range(n):
        t, rr = divmod(r, 16)
        out[t, :, rr * 64:(rr + 1) * 64] = words[r].reshape(subs, 16).view(np.uint8).reshape(subs, 64)
        out[t, :, 1024 + rr * 8:1024 + (rr + 1) * 8] = sb[r].reshape(subs, 8)
    return out.reshape(-1)


def pack(n, k, seed):
    w = synth.student_t_weight(n, k, seed)
    return w, mx.quantize_packed(w.cuda())[0]


def oracle_y(x: torch.Tensor, w: torch.Tensor):
    ref = oracle.quantize(w.float().numpy())
    return oracle.linear(x.float().numpy(), oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16")))


@pytest.mark.parametrize("n,k", [(33, 70), (64, 512), (200, 1000), (16, 128), (1024, 4096)])
def test_stream_layout_is_the_stated_permutation(n, k):
    _, p = pack(n, k, n + k)
    s = p.to_stream_layout()
    assert s.layout == "stream" and s.lut is not None and s.codes.numel() == ((n + 15) // 16) * (p.kpad // 128) * 1152
    want = numpy_stream(p.codes.cpu().numpy(), p.scales.cpu().numpy(), p.fmt.cpu().numpy(), n, p.kpad)
    assert np.array_equal(s.codes.cpu().numpy(), want)
    back = s.to_canonical()
    assert torch.equal(back.codes, p.codes) and torch.equal(back.scales, p.scales) and torch.equal(back.fmt, p.fmt)
    assert torch.equal(s.format_ids(), p.format_ids()) and torch.equal(s.selected_scales(), p.selected_scales())
    via_kernel = p.to_kernel_layout().to_stream_layout()
    assert torch.equal(via_kernel.codes, s.codes)


def test_dequant_from_stream_layout():
    _, p = pack(100, 384, 3)
    s = p.to_stream_layout()
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        assert torch.equal(mx.dequantize(s, dt), mx.dequantize(p, dt))


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("n,k", [(50, 70), (33, 131), (16, 14336), (1000, 512), (4800, 256), (4736, 1024), (7000, 128),
                                 (272, 1152), (8, 4096)])
def test_stream_gemv_matches_oracle(m, n, k):
    w, p = pack(n, k, 3 * n + k)
    x = synth.activations(m, k, seed=m)
    s = p.to_stream_layout()
    ystar = oracle_y(x, w)
    no_table = mx.PackedWeight(s.codes, s.scales, None, s.global_scale, s.n, s.k, None, "stream", None)
    for q in (s, no_table):
        y = mx.mixfp4_linear(x.cuda(), q, out_dtype=torch.float32).cpu().numpy()
        assert y.shape == (m, n)
        assert oracle.relative_l2(y, ystar) <= TOL


@pytest.mark.parametrize("name,n,k", [("q", 4096, 4096), ("kv", 1024, 4096), ("gate", 14336, 4096), ("down", 4096, 14336)])
def test_config2_layer_shapes_match_oracle(name, n, k):
    """The benched path (stream layout, prebuilt table) on the Llama-3-8B layer shapes at M = 1, 4, 16."""
    w, p = pack(n, k, len(name) + n)
    s = p.to_stream_layout()
    ref = oracle.quantize(w.float().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    for m in (1, 4, 16):
        x = synth.activations(m, k, seed=10 + m)
        y = mx.mixfp4_linear(x.cuda(), s, out_dtype=torch.float32, overlap_previous=True).cpu().numpy()
        err = oracle.relative_l2(y, oracle.linear(x.float().numpy(), wq))
        assert err <= 2e-5, f"{name} M={m}: {err:.3e}"       # summation order only; the stated bound is 1e-3
    assert mx.decode_status() == 0


@pytest.mark.parametrize("ns", [(4096, 1024, 1024), (14336, 14336)])
def test_grouped_config2_launches_match_oracle(ns):
    """q/k/v (6144 x 4096 in 3 segments) and gate/up (28672 x 4096 in 2) as one launch each."""
    k = 4096
    ws = [synth.student_t_weight(n, k, seed=50 + i) for i, n in enumerate(ns)]
    packs = [mx.quantize_packed(w.cuda())[0].to_stream_layout() for w in ws]
    for m in (1, 4, 16):
        x = synth.activations(m, k, seed=20 + m)
        ys = mx.mixfp4_linear_grouped(x.cuda(), packs, out_dtype=torch.float32, overlap_previous=True)
        for y, w in zip(ys, ws):
            assert oracle.relative_l2(y.cpu().numpy(), oracle_y(x, w)) <= 2e-5


@pytest.mark.parametrize("m", [1, 4, 8, 11, 16])
@pytest.mark.parametrize("ns", [(1024, 256, 256), (40, 17, 1000), (5000,), (16, 16)])
def test_grouped_stream_launch_matches_oracle_and_separate_launches(m, ns):
    k = 1024
    x = synth.activations(m, k, seed=11)
    ws = [synth.student_t_weight(n, k, seed=n) for n in ns]
    packs = [mx.quantize_packed(w.cuda())[0].to_stream_layout() for w in ws]
    for dt in (torch.float32, torch.bfloat16):
        together = mx.mixfp4_linear_grouped(x.cuda(), packs, out_dtype=dt)
        for y, p, w in zip(together, packs, ws):
            assert y.shape == (m, p.n)
            ystar = oracle_y(x, w)
            if dt == torch.float32:
                assert oracle.relative_l2(y.cpu().numpy(), ystar) <= TOL
            else:
                assert np.all(np.abs(y.float().cpu().numpy() - ystar) <= np.abs(ystar) * 2.0 ** -7 + 1e-30)


def test_runs_are_deterministic_and_overlapped_chain_matches_plain_chain():
    ws = [pack(1024, 1024, s)[1].to_stream_layout() for s in range(6)]
    x = synth.activations(1, 1024, 77).cuda()

    def chain(overlap):
        h = x
        for p in ws:
            h = mx.mixfp4_linear(h, p, overlap_previous=overlap)
        return h

    plain = chain(False)
    for _ in range(5):
        assert torch.equal(chain(True), plain)
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            out = chain(True)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, plain)


def test_x_too_large_for_shared_memory_takes_the_staged_kernel():
    # M = 16 rows of K = 14336 (458 KB of x) cannot stay resident: same buffer, x staged through the rings
    w, p = pack(96, 14336, 4)
    s = p.to_stream_layout()
    for m in (8, 16):
        x = synth.activations(m, 14336, seed=m)
        y = mx.mixfp4_linear(x.cuda(), s, out_dtype=torch.float32).cpu().numpy()
        assert oracle.relative_l2(y, oracle_y(x, w)) <= TOL


def test_unaligned_x_and_bf16_output():
    w, p = pack(48, 200, 7)
    s = p.to_stream_layout()
    base = synth.activations(6, 260, 8).cuda()
    x = base[:, 3:203]                                   # rows not 16-byte aligned
    y = mx.mixfp4_linear(x, s, out_dtype=torch.float32).cpu().numpy()
    assert oracle.relative_l2(y, oracle_y(x.cpu(), w)) <= TOL
    yb = mx.mixfp4_linear(x, s).float().cpu().numpy()
    ystar = oracle_y(x.cpu(), w)
    assert np.all(np.abs(yb - ystar) <= np.abs(ystar) * 2.0 ** -7 + 1e-30)


@pytest.mark.parametrize("m", [17, 200, 512])
@pytest.mark.parametrize("n,k", [(272, 1152), (1000, 512), (4096, 1024)])
def test_prefill_gemm_reads_the_stream_layout(m, n, k):
    w, p = pack(n, k, n + 2 * k)
    x = synth.activations(m, k, seed=m)
    y = mx.mixfp4_linear(x.cuda(), p.to_stream_layout(), out_dtype=torch.float32)
    assert mx.gemm_status() == 0
    assert oracle.relative_l2(y.cpu().numpy(), oracle_y(x, w)) <= TOL
    assert torch.equal(y, mx.mixfp4_linear(x.cuda(), p.to_kernel_layout(), out_dtype=torch.float32))


def test_prefill_gemm_pairs_and_rotation_on_stream_layout():
    # 1024 tokens: the CTA-pair kernel; H128 folded into the weight and applied to x by the call
    n, k, m = 2048, 1024, 1024
    w = synth.student_t_weight(n, k, 5)
    wr = mx.apply_transform(w.cuda(), "H128")
    p = mx.quantize_packed(wr, rotation="H128")[0]
    x = synth.activations(m, k, seed=6).cuda()
    ys = mx.mixfp4_linear(x, p.to_stream_layout(), out_dtype=torch.float32)
    yk = mx.mixfp4_linear(x, p.to_kernel_layout(), out_dtype=torch.float32)
    assert mx.gemm_status() == 0
    assert torch.equal(ys, yk)
