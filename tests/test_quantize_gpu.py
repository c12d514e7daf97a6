"""GPU parity of the quantize / dequant kernels (through the C ABI) against the golden
fixtures produced by the reference and against the CPU oracle.  Everything is bit-exact."""

import hashlib

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import synth
from tests.golden_io import digests, quant_cases

pytestmark = pytest.mark.gpu
CASES = quant_cases()
TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def case_tensor(case) -> torch.Tensor:
    raw = case.data["x"]
    if case.dtype == "float32":
        t = torch.from_numpy(raw.copy())
    else:
        t = torch.from_numpy(raw.view(np.int16).copy()).view(TORCH_DTYPE[case.dtype])
    return t.reshape(case.shape)


def raw_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy().view(np.uint32)


def same_bits(a: torch.Tensor, b: np.ndarray) -> bool:
    return np.array_equal(raw_bits(a).reshape(-1), b.reshape(-1).view(raw_bits(a).dtype))


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_packed_bytes_match_reference(case):
    x = case_tensor(case).cuda()
    packed, dq, stats = mx.quantize_packed(x, mode=case.mode, want_dequant=True, want_stats=True)
    d = case.data
    assert np.array_equal(packed.codes.cpu().numpy(), d["codes"])
    assert np.array_equal(packed.scales.cpu().numpy(), d["scales"])
    assert np.array_equal(packed.fmt.cpu().numpy(), d["fmt"])
    assert same_bits(packed.global_scale, d["global_scale"])
    assert np.array_equal(packed.format_ids().cpu().numpy(), d["format_ids"])
    for key in ("e2_errors", "e0_errors", "e2_scales", "e0_scales"):
        assert same_bits(stats[key], d[key]), key
    assert same_bits(packed.selected_scales(), d["selected_scales"])
    assert same_bits(dq, d["dequant"])
    assert same_bits(mx.dequantize(packed, x.dtype), d["dequant"])


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_public_api_matches_reference(case):
    x = case_tensor(case)
    for tensor in (x.cuda(), x):  # device tensor and host tensor (copied in and out)
        out = mx.quant_mixfp4_granularity(tensor, format_region=case.mode, operand_role=case.role)
        assert out.shape == x.shape and out.dtype == x.dtype and out.device == tensor.device
        assert same_bits(out, case.data["dequant"])
    res = mx.quant_mixfp4_granularity(x.cuda(), format_region=case.mode, operand_role=case.role, return_stats=True)
    assert np.array_equal(res.format_ids.cpu().numpy(), case.data["format_ids"])
    assert same_bits(res.selected_scales, case.data["selected_scales"])
    assert same_bits(res.e2_errors, case.data["e2_errors"]) and same_bits(res.e0_errors, case.data["e0_errors"])
    assert res.summary["num_scale_blocks"] == case.data["format_ids"].size
    assert res.summary["e0_count"] == int(case.data["format_ids"].sum())
    assert res.summary["tail_padding_values"] == (-x.shape[-1]) % 16


def test_strided_and_unaligned_inputs():
    base = synth.seeded((33, 200), 5, torch.bfloat16).cuda()
    view = base[:, 3:150]                      # row stride 200, start offset 6 bytes: scalar path
    ref = oracle.quantize(view.float().cpu().numpy())
    packed, dq, _ = mx.quantize_packed(view, want_dequant=True)
    assert np.array_equal(packed.codes.cpu().numpy(), ref.codes)
    assert np.array_equal(packed.scales.cpu().numpy(), ref.scales)
    assert np.array_equal(packed.fmt.cpu().numpy(), ref.fmt)
    assert np.array_equal(raw_bits(dq), oracle.dequant(ref, "bf16"))


def test_deterministic():
    # reference: tests/test_quant_core.py:160-165
    x = synth.seeded((8, 64), 123).cuda()
    a = mx.quant_mixfp4_granularity(x, return_stats=True)
    b = mx.quant_mixfp4_granularity(x, return_stats=True)
    assert torch.equal(a.dequant, b.dequant) and torch.equal(a.format_ids, b.format_ids)
    assert a.summary == b.summary


def test_zero_tensor_is_finite_and_exact():
    # reference: tests/test_quant_core.py:168-173
    x = torch.zeros((9, 70), dtype=torch.bfloat16, device="cuda")
    for mode in ("all_e2m1", "all_e0m3", "oracle16"):
        out = mx.quant_mixfp4_granularity(x, format_region=mode)
        assert torch.equal(out, x) and torch.isfinite(out).all()


def test_oracle_not_worse_than_either_fixed_format():
    # reference: tests/test_quant_core.py:56-62
    x = synth.seeded((17, 79), 3).cuda()
    err = {m: mx.quant_mixfp4_granularity(x, format_region=m, return_stats=True).summary["selected_weight_error"]
           for m in ("oracle16", "all_e2m1", "all_e0m3")}
    assert err["oracle16"] <= err["all_e2m1"] + 1e-6 and err["oracle16"] <= err["all_e0m3"] + 1e-6


def test_shard_with_whole_tensor_amax_equals_slice_of_whole():
    w = synth.student_t_weight(64, 512, 9).cuda()
    whole, _, _ = mx.quantize_packed(w)
    amax = mx.tensor_amax(w)
    top, _, _ = mx.quantize_packed(w[:32], amax=amax)            # split N
    assert torch.equal(top.codes, whole.codes[:32]) and torch.equal(top.fmt, whole.fmt[:32])
    right, _, _ = mx.quantize_packed(w[:, 256:], amax=amax)      # split K on a multiple of 128
    ks = whole.k_shard(256, 512)
    assert torch.equal(right.codes, ks.codes) and torch.equal(right.scales, ks.scales)
    assert torch.equal(right.fmt, ks.fmt)


FULL = [
    ("config1_w_4096x4096", lambda: synth.config1(0)[0]),
    ("student_t_q_4096x4096_s0", lambda: synth.student_t_weight(4096, 4096, 0)),
    ("student_t_kv_1024x4096_s1", lambda: synth.student_t_weight(1024, 4096, 1)),
]


@pytest.mark.parametrize("name,make", FULL, ids=[f[0] for f in FULL])
def test_full_size_against_oracle_and_reference_digests(name, make):
    w = make()
    packed, dq, _ = mx.quantize_packed(w.cuda(), want_dequant=True)
    ref = oracle.quantize(w.float().numpy())
    codes, scales, fmt = (t.cpu().numpy() for t in (packed.codes, packed.scales, packed.fmt))
    assert np.array_equal(codes, ref.codes)
    assert np.array_equal(scales, ref.scales)
    assert np.array_equal(fmt, ref.fmt)
    assert np.float32(packed.global_scale.item()) == ref.global_scale
    assert np.array_equal(raw_bits(dq), oracle.dequant(ref, "bf16"))
    info = digests()["cases"][name]
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    if sha(raw_bits(w)) == info["input_sha256"]:   # same random draw as the fixture's torch build
        assert sha(codes) == info["codes_sha256"] and sha(scales) == info["scales_sha256"]
        assert sha(fmt) == info["fmt_sha256"] and sha(raw_bits(dq)) == info["dequant_sha256"]


def test_largest_8b_layer_against_oracle():
    """gate/up projection shape 14336 x 4096 (config 2): bytes equal to the oracle's, and the
    quantize -> dequantize -> quantize round trip is idempotent on codes."""
    w = synth.student_t_weight(14336, 4096, 3)
    wd = w.cuda()
    packed, dq, _ = mx.quantize_packed(wd, want_dequant=True)
    ref = oracle.quantize(w.float().numpy())
    assert np.array_equal(packed.codes.cpu().numpy(), ref.codes)
    assert np.array_equal(packed.scales.cpu().numpy(), ref.scales)
    assert np.array_equal(packed.fmt.cpu().numpy(), ref.fmt)
    again = mx.quant_mixfp4_granularity(dq)
    err1 = (dq.float() - wd.float()).square().sum().item()
    err2 = (again.float() - wd.float()).square().sum().item()
    assert err2 <= err1 * 1.05       # re-quantizing a quantized tensor does not drift


@pytest.mark.parametrize("mode", ["n8k64", "k64_row", "n64k64", "n8k16", "layer"])
def test_coarse_regions_full_size_against_oracle(mode):
    """q projection shape 4096 x 4096: region choices, bytes and dequantized tensor equal to the
    oracle's; every block of a region carries the region's format; a coarse choice is never
    better than the per-block choice and never worse than the better fixed format."""
    w = synth.student_t_weight(4096, 4096, 4)
    wd = w.cuda()
    packed, dq, stats = mx.quantize_packed(wd, mode=mode, want_dequant=True, want_stats=True)
    ref = oracle.quantize(w.float().numpy(), mode)
    assert np.array_equal(packed.codes.cpu().numpy(), ref.codes)
    assert np.array_equal(packed.scales.cpu().numpy(), ref.scales)
    assert np.array_equal(packed.fmt.cpu().numpy(), ref.fmt)
    assert np.array_equal(raw_bits(dq), oracle.dequant(ref, "bf16"))
    rr, rg = oracle.REGIONS[mode] if mode != "layer" else (4096, 256)
    ids = packed.format_ids()
    tiles = ids.reshape(4096 // rr, rr, 256 // rg, rg)
    assert torch.equal(tiles, tiles[:, :1, :, :1].expand_as(tiles))
    e2, e0 = stats["e2_errors"].double(), stats["e0_errors"].double()
    chosen = torch.where(ids.bool(), e0, e2).sum().item()
    assert torch.minimum(e2, e0).sum().item() <= chosen <= min(e2.sum().item(), e0.sum().item()) * (1 + 1e-9)


def test_column_regions_on_an_activation_with_ragged_edges_against_oracle():
    """m16k16 on a [M, K] activation whose rows do not fill the last region and whose block columns leave a
    remainder after the whole chunks of 32 (K = 1104 + 8: 70 columns, the last block partial): both summation
    orders of the column sums are in play."""
    x = synth.activations(200, 1112, 9, outlier_fraction=0.02)
    packed, dq, _ = mx.quantize_packed(x.cuda(), mode="m16k16", want_dequant=True, region=(16, 1))
    ref = oracle.quantize(x.float().numpy(), "m16k16")
    assert np.array_equal(packed.codes.cpu().numpy(), ref.codes)
    assert np.array_equal(packed.scales.cpu().numpy(), ref.scales)
    assert np.array_equal(packed.fmt.cpu().numpy(), ref.fmt)
    assert np.array_equal(raw_bits(dq), oracle.dequant(ref, "bf16"))
    got = mx.fake_quantize_activations(x.cuda(), "m16k16")
    assert np.array_equal(raw_bits(got), oracle.dequant(ref, "bf16"))


def test_reciprocal_division_is_ieee_exact():
    """Exhaustive on-device proof behind the quantizer's fast division (see
    mixfp4_selftest_division): zero disagreements with IEEE division."""
    from mixfp4_b200 import _native as nat
    out = torch.ones(1, dtype=torch.int64, device="cuda")
    rc = nat.lib().mixfp4_selftest_division(out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert int(out.item()) == 0
