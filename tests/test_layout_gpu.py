"""The kernel layout is a pure bit permutation of the canonical packed layout: round trip
is the identity, every kernel computes the same thing from either layout, and the prebuilt
decode table changes nothing."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import synth

pytestmark = pytest.mark.gpu


def pack(n, k, seed):
    w = synth.student_t_weight(n, k, seed)
    return w, mx.quantize_packed(w.cuda())[0]


@pytest.mark.parametrize("n,k", [(33, 70), (64, 512), (200, 1000), (1024, 4096)])
def test_round_trip_is_identity(n, k):
    _, p = pack(n, k, n + k)
    kl = p.to_kernel_layout()
    assert kl.layout == "kernel" and kl.fmt is None and kl.lut is not None
    back = kl.to_canonical()
    assert torch.equal(back.codes, p.codes) and torch.equal(back.scales, p.scales) and torch.equal(back.fmt, p.fmt)
    # same multiset of bits per 32-bit code word, format bit moved into the scale byte
    a = p.codes.cpu().numpy().view(np.uint32)
    b = kl.codes.cpu().numpy().view(np.uint32)
    popcount = lambda v: np.unpackbits(v.view(np.uint8)).reshape(v.shape + (32,)).sum(-1)
    assert np.array_equal(popcount(a), popcount(b))
    assert torch.equal(kl.format_ids(), p.format_ids()) and torch.equal(kl.selected_scales(), p.selected_scales())


def test_dequant_is_layout_independent():
    _, p = pack(96, 384, 3)
    assert torch.equal(mx.dequantize(p.to_kernel_layout()), mx.dequantize(p))
    assert torch.equal(mx.dequantize(p.to_kernel_layout(), torch.float32), mx.dequantize(p, torch.float32))


@pytest.mark.parametrize("m", [1, 5, 16, 200])
def test_linear_is_layout_and_table_independent(m):
    w, p = pack(272, 1152, 9)
    x = synth.activations(m, 1152, m).cuda()
    ref = mx.mixfp4_linear(x, p, out_dtype=torch.float32)
    kl = p.to_kernel_layout()
    assert torch.equal(mx.mixfp4_linear(x, kl, out_dtype=torch.float32), ref)
    no_table = mx.PackedWeight(kl.codes, kl.scales, None, kl.global_scale, kl.n, kl.k, None, "kernel", None)
    assert torch.equal(mx.mixfp4_linear(x, no_table, out_dtype=torch.float32), ref)
    wq = oracle.bf16_bits_to_f32(oracle.dequant(oracle.quantize(w.float().numpy()), "bf16"))
    assert oracle.relative_l2(ref.cpu().numpy(), oracle.linear(x.float().cpu().numpy(), wq)) <= 1e-3


def test_overlapped_launch_chain_matches_plain_chain():
    """A chain of dependent decode GEMVs launched as programmatic dependents gives the same
    numbers as the plain chain."""
    ws = [pack(1024, 1024, s)[1].to_kernel_layout() for s in range(6)]
    x = synth.activations(1, 1024, 77).cuda()
    torch.cuda.synchronize()

    def chain(overlap):
        h = x
        for p in ws:
            h = mx.mixfp4_linear(h, p, overlap_previous=overlap)
        return h

    plain = chain(False)
    for _ in range(5):
        assert torch.equal(chain(True), plain)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 9, 13, 16])
@pytest.mark.parametrize("n,k", [(50, 70), (33, 131), (16, 14336), (1000, 512), (4800, 256), (4736, 1024), (7000, 128)])
def test_kernel_layout_gemv_matches_oracle(m, n, k):
    # ragged row counts (last tile partly outside N), K tails, fewer tiles than SMs and more
    # tiles than warp groups: both instances of the one-CTA-per-SM decode kernel
    w = synth.student_t_weight(n, k, seed=3 * n + k)
    x = synth.activations(m, k, seed=m)
    packed = mx.quantize_packed(w.cuda())[0].to_kernel_layout()
    ref = oracle.quantize(w.float().numpy())
    ystar = oracle.linear(x.float().numpy(), oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16")))
    for p in (packed, packed.with_decode_table()):
        y = mx.mixfp4_linear(x.cuda(), p, out_dtype=torch.float32).cpu().numpy()
        assert oracle.relative_l2(y, ystar) <= 1e-3


@pytest.mark.parametrize("m", [1, 4, 8, 11, 16])
@pytest.mark.parametrize("ns", [(1024, 256, 256), (4096, 1024), (40, 17, 1000), (5000,)])
def test_grouped_launch_equals_separate_launches(m, ns):
    k = 1024
    x = synth.activations(m, k, seed=11).cuda()
    packs = [mx.quantize_packed(synth.student_t_weight(n, k, seed=n).cuda())[0].to_kernel_layout().with_decode_table()
             for n in ns]
    for dt in (torch.float32, torch.bfloat16):
        together = mx.mixfp4_linear_grouped(x, packs, out_dtype=dt)
        for y, p in zip(together, packs):
            assert y.shape == (m, p.n)
            assert torch.equal(y, mx.mixfp4_linear(x, p, out_dtype=dt))


def test_grouped_falls_back_for_prefill_and_canonical():
    k = 512
    x = synth.activations(40, k, seed=2).cuda()
    packs = [mx.quantize_packed(synth.student_t_weight(n, k, seed=n).cuda())[0] for n in (64, 96)]
    ys = mx.mixfp4_linear_grouped(x, packs, out_dtype=torch.float32)
    for y, p in zip(ys, packs):
        assert torch.equal(y, mx.mixfp4_linear(x, p, out_dtype=torch.float32))
