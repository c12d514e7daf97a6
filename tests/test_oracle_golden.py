"""Pins the CPU oracle against fixtures produced by the reference itself (CPU only)."""

import hashlib

import numpy as np
import pytest

import oracle
from tests.golden_io import digests, quant_cases, rotation_cases

CASES = quant_cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_quantizer_matches_reference(case):
    x = case.x_f32()
    p = oracle.quantize(x, case.mode, stats=True, nibbles=True)
    d = case.data
    assert np.float32(p.global_scale).view(np.uint32) == d["global_scale"].view(np.uint32)[0]
    # both candidates, block by block (bit patterns of the fp32 errors decide the selector)
    assert np.array_equal(p.e2_nibbles, d["e2_nibbles"])
    assert np.array_equal(p.e0_nibbles, d["e0_nibbles"])
    assert np.array_equal(p.e2_scales.view(np.uint32), d["e2_scales"].view(np.uint32))
    assert np.array_equal(p.e0_scales.view(np.uint32), d["e0_scales"].view(np.uint32))
    assert np.array_equal(p.e2_errors.view(np.uint32), d["e2_errors"].view(np.uint32))
    assert np.array_equal(p.e0_errors.view(np.uint32), d["e0_errors"].view(np.uint32))
    # the packed bytes
    assert np.array_equal(p.format_ids(), d["format_ids"])
    assert np.array_equal(p.codes, d["codes"])
    assert np.array_equal(p.scales, d["scales"])
    assert np.array_equal(p.fmt, d["fmt"])
    assert np.array_equal(p.selected_scales().view(np.uint32), d["selected_scales"].view(np.uint32))


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_dequant_matches_reference(case):
    p = oracle.quantize(case.x_f32(), case.mode)
    d = case.data
    if case.dtype == "bfloat16":
        got = oracle.dequant(p, "bf16").reshape(d["dequant"].shape)
        assert np.array_equal(got, d["dequant"])
    elif case.dtype == "float32":
        got = oracle.dequant(p, "f32").reshape(d["dequant"].shape)
        assert np.array_equal(got.view(np.uint32), d["dequant"].view(np.uint32))
    else:  # float16: the oracle decodes to fp32, the cast is numpy's RNE
        got = oracle.dequant(p, "f32").astype(np.float16).reshape(d["dequant"].shape)
        assert np.array_equal(got.view(np.uint16), d["dequant"])


def _rotation_keys():
    return sorted(k[: -len("__x")] for k in rotation_cases() if k.endswith("__x"))


@pytest.mark.parametrize("key", _rotation_keys())
def test_rotation_matches_reference(key):
    z = rotation_cases()
    name, tag = key.split("__")
    size = int(name.split("H")[1].split("_")[0])
    signs = z.get(f"{name}__signs")
    x, y = z[key + "__x"], z[key + "__y"]
    if tag.startswith("bf16"):
        got = oracle.fwht(oracle.bf16_bits_to_f32(x), size, signs=signs, bf16_stages=True)
        assert np.array_equal(oracle.f32_to_bf16_bits(got), y)
    else:
        got = oracle.fwht(x, size, signs=signs)
        assert np.array_equal(got.view(np.uint32), y.view(np.uint32))


def test_zero_tensor_is_exact():
    # reference: tests/test_quant_core.py:168-173
    for mode in ("oracle16", "all_e2m1", "all_e0m3"):
        p = oracle.quantize(np.zeros((9, 70), np.float32), mode)
        assert p.global_scale == np.float32(1.0)
        assert not oracle.dequant(p, "f32").any()
        assert not p.codes.any() and (p.scales == 1).all()
        assert int(p.format_ids().sum()) == (9 * 5 if mode == "all_e0m3" else 0)


def test_linear_oracle_matches_numpy_float64():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 96)).astype(np.float32)
    w = rng.standard_normal((7, 96)).astype(np.float32)
    ref = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    assert np.array_equal(oracle.linear(x, w), ref)


@pytest.mark.parametrize("name", sorted(digests()["cases"]))
def test_full_size_digests(name):
    """Full-size tensors: the oracle's packed bytes hash to what the reference produced."""
    import torch
    from mixfp4_b200 import synth

    info = digests()["cases"][name]
    if name.startswith("config1"):
        w = synth.config1(0)[0]
    elif "_q_" in name:
        w = synth.student_t_weight(4096, 4096, 0)
    else:
        w = synth.student_t_weight(1024, 4096, 1)
    raw = w.view(torch.int16).numpy().view(np.uint16)
    if hashlib.sha256(raw.tobytes()).hexdigest() != info["input_sha256"]:
        pytest.skip("this torch build draws different random numbers than the fixture's")
    p = oracle.quantize(oracle.bf16_bits_to_f32(raw))
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    assert sha(p.codes) == info["codes_sha256"]
    assert sha(p.scales) == info["scales_sha256"]
    assert sha(p.fmt) == info["fmt_sha256"]
    assert sha(oracle.dequant(p, "bf16")) == info["dequant_sha256"]
    assert int(np.float32(p.global_scale).view(np.uint32)) == info["global_scale_bits"]
    assert int(p.format_ids().sum()) == info["e0_blocks"]


def test_torch_port_matches_c_oracle():
    """The eager-op port that the benchmark times produces the same bytes as the C oracle."""
    import torch
    from mixfp4_b200 import synth
    from oracle import torch_port

    for w in (synth.student_t_weight(96, 400, 4), synth.seeded((17, 79), 3), synth.gaussian_outlier_weight(64, 256, 2)):
        out, parts = torch_port.quantize_dequant(w, return_parts=True)
        p = oracle.quantize(w.float().numpy(), stats=True)
        assert np.array_equal(parts["format_ids"].numpy(), p.format_ids())
        assert np.array_equal(parts["e2_errors"].numpy().view(np.uint32), p.e2_errors.view(np.uint32))
        assert np.array_equal(parts["e0_errors"].numpy().view(np.uint32), p.e0_errors.view(np.uint32))
        assert np.array_equal(parts["scales"].numpy(), p.selected_scales())
        ref = oracle.dequant(p, "bf16" if w.dtype == torch.bfloat16 else "f32")
        got = out.view(torch.int16).numpy().view(np.uint16) if w.dtype == torch.bfloat16 else out.numpy()
        assert np.array_equal(got.reshape(-1), ref.reshape(-1))


def test_codebook_rounding_matches_reference_probe():
    # quantize_e2m1 / quantize_e0m3 of the reference on its own dense level probe plus tie values
    # (tests/golden/make_golden.py: candidate_case_list); signed zeros compared as bit patterns
    from tests.golden_io import candidate_cases
    probe = candidate_cases()["probe"]
    for key, e0 in (("e2m1", False), ("e0m3", True)):
        got = oracle.round_codebook(probe["x"], e0)
        assert np.array_equal(got.view(np.uint32), probe[key].view(np.uint32)), key
    levels = sorted(set(np.abs(oracle.round_codebook(np.linspace(-10, 10, 80001, dtype=np.float32), False)).tolist()))
    assert levels == list(oracle.E2M1_LEVELS)


def test_both_candidates_dequantized_values_match_reference():
    # build_candidates' float32 e2_dequant / e0_dequant: the oracle with the format forced
    from tests.golden_io import candidate_cases
    cases = {c.name: c for c in quant_cases()}
    for name, d in candidate_cases().items():
        if name == "probe":
            continue
        x = cases[name].x_f32()
        rows, k, groups, kp, tail = (int(v) for v in d["meta"])
        assert (rows, k) == x.shape and kp == groups * 16 and tail == (-k) % 16
        xp = np.pad(x, ((0, 0), (0, tail)))
        assert np.array_equal(xp.reshape(rows, groups, 16).view(np.uint32), d["grouped_original"].view(np.uint32))
        for mode, key in (("all_e2m1", "e2_dequant"), ("all_e0m3", "e0_dequant")):
            got = oracle.dequant(oracle.quantize(xp, mode), "f32")
            assert np.array_equal(got.reshape(rows, groups, 16).view(np.uint32), d[key].view(np.uint32)), (name, key)


def test_e0_four_over_six_candidate_matches_reference():
    # scale_rule "four_over_six", E0M3 side (project_quant/scale.py:64-103, 207-225), incl. the crafted
    # boundary tensor of the reference's tests and blocks whose unclamped scale rounds to zero
    from tests.golden_io import four_over_six_e0_cases
    picked = 0
    for name, d in four_over_six_e0_cases().items():
        got = oracle.e0_four_over_six(d["grouped"])
        for key in ("codes", "dequant", "scales", "errors"):
            assert np.array_equal(got[key].view(np.uint32), d[key].view(np.uint32)), (name, key)
        assert np.array_equal(got["expansion_ids"], d["expansion_ids"]), name
        picked += int(d["expansion_ids"].sum())
    assert picked > 0            # the expanded scale wins somewhere in the fixtures
