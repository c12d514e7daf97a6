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
