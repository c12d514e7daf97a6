"""GPU parity of the candidate-level surface of the reference (project_quant/__init__.py:3-5):
``build_candidates`` / ``CandidateBlocks`` and the element-wise ``quantize_e2m1`` / ``quantize_e0m3``.
Every field is compared bit for bit with fixtures produced by the reference
(tests/golden/make_golden.py) and with the CPU oracle on larger tensors."""

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import synth
from tests.golden_io import candidate_cases, quant_cases
from tests.test_quantize_gpu import case_tensor

pytestmark = pytest.mark.gpu
CASES = {c.name: c for c in quant_cases()}
CAND = candidate_cases()


def f32_bits(t) -> np.ndarray:
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return a.astype(np.float32, copy=False).view(np.uint32)


def nibbles_to_levels(nib: np.ndarray, levels) -> np.ndarray:
    mag = np.asarray(levels, np.float32)[nib & 7]
    return np.where(nib & 8, -mag, mag).astype(np.float32)


@pytest.mark.parametrize("name", [n for n in CAND if n != "probe"])
def test_build_candidates_matches_reference(name):
    case, want = CASES[name], CAND[name]
    x = case_tensor(case)
    for tensor in (x.cuda(), x):
        c = mx.build_candidates(tensor, operand_role=case.role)
        rows, k, groups, kp, tail = (int(v) for v in want["meta"])
        assert (c.rows, c.k, c.groups, c.padded_k, c.tail_padding) == (rows, k, groups, kp, tail)
        assert c.original_shape == tuple(x.shape) and c.source_dtype == x.dtype and c.operand_role == case.role
        assert c.scale_rule == "standard" and c.global_scale.ndim == 0 and c.e2_codes.device == tensor.device
        assert np.array_equal(f32_bits(c.grouped_original), want["grouped_original"].view(np.uint32))
        assert np.array_equal(f32_bits(c.e2_dequant), want["e2_dequant"].view(np.uint32))
        assert np.array_equal(f32_bits(c.e0_dequant), want["e0_dequant"].view(np.uint32))
        d = case.data
        assert np.array_equal(f32_bits(c.e2_codes).reshape(rows, -1),
                              nibbles_to_levels(d["e2_nibbles"], mx.E2M1_LEVELS).view(np.uint32))
        assert np.array_equal(f32_bits(c.e0_codes).reshape(rows, -1),
                              nibbles_to_levels(d["e0_nibbles"], mx.E0M3_LEVELS).view(np.uint32))
        for key in ("e2_scales", "e0_scales", "e2_errors", "e0_errors"):
            assert np.array_equal(f32_bits(getattr(c, key)), d[key].view(np.uint32)), key
        assert f32_bits(c.global_scale.reshape(1))[0] == d["global_scale"].view(np.uint32)[0]
        assert c.e2_scale_expansion_ids.dtype == torch.uint8 and not bool(c.e2_scale_expansion_ids.any())
        assert c.e0_scale_expansion_ids.shape == (rows, groups)


def test_build_candidates_full_size_against_oracle():
    w = synth.student_t_weight(1024, 4096, 4)
    c = mx.build_candidates(w.cuda())
    ref = oracle.quantize(w.float().numpy(), "oracle16", stats=True, nibbles=True)
    assert np.array_equal(f32_bits(c.e2_errors), ref.e2_errors.view(np.uint32))
    assert np.array_equal(f32_bits(c.e0_errors), ref.e0_errors.view(np.uint32))
    assert np.array_equal(f32_bits(c.e2_codes).reshape(1024, -1), nibbles_to_levels(ref.e2_nibbles, mx.E2M1_LEVELS).view(np.uint32))
    assert np.array_equal(f32_bits(c.e0_codes).reshape(1024, -1), nibbles_to_levels(ref.e0_nibbles, mx.E0M3_LEVELS).view(np.uint32))
    for mode, got in (("all_e2m1", c.e2_dequant), ("all_e0m3", c.e0_dequant)):
        want = oracle.dequant(oracle.quantize(w.float().numpy(), mode), "f32")
        assert np.array_equal(f32_bits(got).reshape(1024, -1), want.view(np.uint32))
    # the per-block choice of the reference (core.py:115-127) from the candidate fields
    ids = (c.e0_errors < c.e2_errors).to(torch.uint8)
    assert np.array_equal(ids.cpu().numpy(), ref.format_ids())


def test_build_candidates_error_conventions():
    with pytest.raises(ValueError, match="fixes scale_group_size=16"):
        mx.build_candidates(torch.zeros((4, 32)), scale_group_size=32)
    with pytest.raises(TypeError, match="floating point"):
        mx.build_candidates(torch.zeros((4, 32), dtype=torch.int32))
    with pytest.raises(ValueError, match=r"\[N,K\]"):
        mx.build_candidates(torch.zeros((2, 4, 32)))
    with pytest.raises(ValueError, match="unknown scale_rule"):
        mx.build_candidates(torch.zeros((4, 32)), scale_rule="other")
    with pytest.raises(NotImplementedError):
        mx.build_candidates(torch.zeros((4, 32)), scale_rule="four_over_six")


def test_codebook_quantizers_match_reference_probe():
    probe = CAND["probe"]
    x = torch.from_numpy(probe["x"].copy())
    for fn, key in ((mx.quantize_e2m1, "e2m1"), (mx.quantize_e0m3, "e0m3")):
        for tensor in (x.cuda(), x):
            y = fn(tensor)
            assert y.dtype == x.dtype and y.device == tensor.device and y.shape == x.shape
            assert np.array_equal(f32_bits(y), probe[key].view(np.uint32)), key
    # the reference's own level test (tests/test_quant_core.py:34-41)
    dense = torch.linspace(-10, 10, 80001, dtype=torch.float32).cuda()
    assert sorted(set(mx.quantize_e2m1(dense).abs().tolist())) == list(mx.E2M1_LEVELS)
    assert sorted(set(mx.quantize_e0m3(dense).abs().tolist())) == list(mx.E0M3_LEVELS)
    # other dtypes and shapes keep dtype and shape
    h = torch.randn((3, 5, 7), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    assert mx.quantize_e0m3(h).shape == h.shape and mx.quantize_e0m3(h).dtype == torch.bfloat16
    want = oracle.round_codebook(h.float().cpu().numpy(), False)
    assert np.array_equal(f32_bits(mx.quantize_e2m1(h).float()), want.view(np.uint32))


def test_e0_four_over_six_candidate_matches_reference_and_oracle():
    from tests.golden_io import four_over_six_e0_cases
    for name, d in four_over_six_e0_cases().items():
        g = torch.from_numpy(d["grouped"].copy())
        for tensor in (g.cuda(), g):
            c = mx.build_scaled_candidate(tensor, format_name="e0m3", scale_rule="four_over_six")
            assert c.codes.device == tensor.device and c.codes.shape == g.shape and c.scales.shape == g.shape[:-1]
            for key in ("codes", "dequant", "scales", "errors"):
                assert np.array_equal(f32_bits(getattr(c, key)), d[key].view(np.uint32)), (name, key)
            assert np.array_equal(c.expansion_ids.cpu().numpy(), d["expansion_ids"]), name
    # a larger tensor against the oracle
    w = synth.student_t_weight(512, 2048, 9).float().reshape(512, -1, 16)
    c = mx.build_scaled_candidate(w.cuda(), format_name="e0m3", scale_rule="four_over_six")
    want = oracle.e0_four_over_six(w.numpy())
    for key in ("codes", "dequant", "scales", "errors"):
        assert np.array_equal(f32_bits(getattr(c, key)), want[key].view(np.uint32)), key
    assert np.array_equal(c.expansion_ids.cpu().numpy(), want["expansion_ids"]) and int(want["expansion_ids"].sum()) > 0
    with pytest.raises(NotImplementedError):
        mx.build_scaled_candidate(w.cuda(), format_name="e2m1", scale_rule="four_over_six")
    with pytest.raises(ValueError, match="unknown scale_rule"):
        mx.build_scaled_candidate(w.cuda(), format_name="e0m3", scale_rule="other")


def test_standard_scaled_candidate_matches_build_candidates():
    case = CASES["t_19x131_s10"]
    x = case_tensor(case).cuda()
    cand = mx.build_candidates(x)
    for fmt, key in (("e2m1", "e2"), ("e0m3", "e0")):
        c = mx.build_scaled_candidate(cand.grouped_original, format_name=fmt, scale_rule="standard")
        assert torch.equal(c.codes, getattr(cand, key + "_codes")) and torch.equal(c.dequant, getattr(cand, key + "_dequant"))
        assert torch.equal(c.scales, getattr(cand, key + "_scales")) and torch.equal(c.errors, getattr(cand, key + "_errors"))
        assert not bool(c.expansion_ids.any())
