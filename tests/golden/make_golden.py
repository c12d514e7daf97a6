"""Generate the golden fixtures by running the reference implementation itself.

Run from the repository root in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/mixfp4

It imports ``project_quant`` from that checkout (read-only), runs the reference's
CPU path on small seeded tensors and writes

    tests/golden/quant_cases.npz      inputs + per-block results of the quantizer
    tests/golden/rotation_cases.npz   inputs + outputs of the block-Hadamard bank
    tests/golden/digests.json         SHA-256 of the packed bytes for full-size tensors
    tests/golden/four_over_six_e0_cases.npz  the E0M3 candidate under scale_rule "four_over_six"
    tests/golden/candidate_cases.npz  build_candidates fields (both candidates' dequantized values)
                                      and the two codebook quantizers on a dense probe

The reference has no packed form, so its per-block results (level values, E4M3
scale values, format ids) are packed here by a small host adapter into the layout
the product uses; the adapter only re-encodes values, it computes nothing.
Nothing at test time reads the reference checkout: tests read these files only.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from mixfp4_b200 import synth  # noqa: E402

E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as a numpy array (bf16/fp16 -> uint16, fp32 -> float32)."""
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def level_nibbles(codes: torch.Tensor, e0m3: bool) -> np.ndarray:
    """fp32 level values -> 4-bit codes (sign<<3 | level index), one per byte."""
    mag = codes.abs()
    if e0m3:
        idx = mag.to(torch.int64)
    else:
        table = torch.tensor(E2M1_LEVELS)
        idx = torch.bucketize(mag, table)  # exact matches: position of the equal entry
        assert torch.equal(table[idx], mag)
    sign = torch.signbit(codes).to(torch.int64)
    return ((sign << 3) | idx).to(torch.uint8).numpy()


def pack(nibbles: np.ndarray, scale_values: np.ndarray, format_ids: np.ndarray, k: int):
    """Pack per-element nibbles [rows, G*16], fp32 scale values [rows, G] and format
    ids [rows, G] into codes/scales/fmt byte arrays padded to K multiple of 128."""
    rows, g = format_ids.shape
    kp = (k + 127) // 128 * 128
    nib = np.zeros((rows, kp), np.uint8)
    nib[:, : g * 16] = nibbles
    codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    sc = np.full((rows, kp // 16), 0x01, np.uint8)
    sc[:, :g] = torch.from_numpy(scale_values).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    ids = np.zeros((rows, kp // 16), np.uint8)
    ids[:, :g] = format_ids
    fmt = np.packbits(ids, axis=1, bitorder="little")
    return codes, sc, fmt


def run_quant_case(pq, x: torch.Tensor, mode: str, role: str) -> dict:
    cand = pq.build_candidates(x, operand_role=role)
    res = pq.quant_mixfp4_granularity(x, format_region=mode, operand_role=role, return_stats=True)
    rows, g = cand.rows, cand.groups
    n2 = level_nibbles(cand.e2_codes, False).reshape(rows, g * 16)
    n0 = level_nibbles(cand.e0_codes, True).reshape(rows, g * 16)
    ids = res.format_ids.numpy().astype(np.uint8)
    sel = np.where(np.repeat(ids, 16, axis=1).astype(bool), n0, n2)
    codes, sc, fmt = pack(sel, res.selected_scales.numpy(), ids, cand.k)
    # the scale bytes must decode to exactly the reference's scale values
    assert torch.equal(torch.from_numpy(sc[:, :g].copy()).view(torch.float8_e4m3fn).float(), res.selected_scales)
    return {
        "x": bits(x),
        "dequant": bits(res.dequant),
        "format_ids": ids,
        "selected_scales": res.selected_scales.numpy(),
        "e2_scales": cand.e2_scales.numpy(), "e0_scales": cand.e0_scales.numpy(),
        "e2_errors": cand.e2_errors.numpy(), "e0_errors": cand.e0_errors.numpy(),
        "e2_nibbles": n2, "e0_nibbles": n0,
        "global_scale": np.array([float(cand.global_scale)], np.float32),
        "codes": codes, "scales": sc, "fmt": fmt,
    }


def quant_case_list():
    """(name, tensor, mode, role): the seeded tensors of the reference's own unit tests
    (tests/test_quant_core.py) plus distribution, dtype and range edge cases."""
    s = synth.seeded
    cases = [
        ("t_9x70_s0", s((9, 70), 0), "oracle16", "weight_b"),
        ("t_17x79_s3", s((17, 79), 3), "oracle16", "weight_b"),
        ("t_17x79_s3_e2", s((17, 79), 3), "all_e2m1", "weight_b"),
        ("t_17x79_s3_e0", s((17, 79), 3), "all_e0m3", "weight_b"),
        ("t_16x128_s5", s((16, 128), 5), "oracle16", "weight_b"),
        ("t_32x128_s9", s((32, 128), 9), "oracle16", "weight_b"),
        ("t_19x131_s10", s((19, 131), 10), "oracle16", "weight_b"),
        ("t_64x128_s11", s((64, 128), 11), "oracle16", "weight_b"),
        ("t_9x80_s12", s((9, 80), 12), "oracle16", "weight_b"),
        ("t_7x19_s16", s((7, 19), 16), "oracle16", "weight_b"),
        ("t_8x64_s123", s((8, 64), 123), "oracle16", "weight_b"),
        ("t_11x64_s17_bf16", s((11, 64), 17, torch.bfloat16), "oracle16", "weight_b"),
        ("t_2x17x70_s14_act", s((2, 17, 70), 14), "oracle16", "activation_a"),
        ("t_3x5x19_s16_act", s((3, 5, 19), 16), "oracle16", "activation_a"),
        ("zeros_9x70_bf16", torch.zeros((9, 70), dtype=torch.bfloat16), "oracle16", "weight_b"),
        ("gauss_outlier_64x512_bf16", synth.gaussian_outlier_weight(64, 512, 0), "oracle16", "weight_b"),
        ("student_t_48x384_bf16", synth.student_t_weight(48, 384, 1), "oracle16", "weight_b"),
        ("student_t_48x384_fp16", synth.student_t_weight(48, 384, 2, dtype=torch.float16), "oracle16", "weight_b"),
        ("acts_outlier_33x256_bf16", synth.activations(33, 256, 3, outlier_fraction=0.02), "oracle16", "activation_a"),
    ]
    # wide dynamic range: a few huge entries push most blocks into the E4M3 subnormal
    # scale range (normalized values above 6 saturate) and many blocks to the 2^-9 floor
    g = torch.Generator().manual_seed(77)
    wide = torch.randn((24, 256), generator=g) * torch.exp2(torch.randint(-30, 4, (24, 256), generator=g).float())
    cases.append(("wide_range_24x256_f32", wide, "oracle16", "weight_b"))
    cases.append(("wide_range_24x256_bf16", wide.to(torch.bfloat16), "oracle16", "weight_b"))
    tiny = (torch.randn((8, 96), generator=g) * 1e-30)
    cases.append(("tiny_8x96_f32", tiny, "oracle16", "weight_b"))
    big = (torch.randn((8, 96), generator=g) * 1e30)
    cases.append(("huge_8x96_f32", big, "oracle16", "weight_b"))
    # values sitting exactly on rounding boundaries of both codebooks
    grid = torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 7.0])
    ties = torch.stack([grid * (1 if i % 2 == 0 else -1) * 2.0 ** (i // 2 - 3) for i in range(12)])
    ties = torch.cat([ties, ties.flip(1), ties * 1.0000001, ties * 0.9999999], dim=1)
    cases.append(("ties_12x64_f32", ties.contiguous(), "oracle16", "weight_b"))
    # coarse format regions (project_quant/region.py): ragged rows and K16 columns against the
    # region grid, one region row only, bf16 sources, activations folded to [M, K]
    cases += [
        ("reg_64x256_s21", s((64, 256), 21), "n8k64", "weight_b"),
        ("reg_100x1120_s22", s((100, 1120), 22), "n8k64", "weight_b"),
        ("reg_70x200_s23", s((70, 200), 23), "n8k64", "weight_b"),
        ("reg_5x1000_s24", s((5, 1000), 24), "n8k64", "weight_b"),
        ("reg_48x384_st_bf16", synth.student_t_weight(48, 384, 1), "n8k64", "weight_b"),
        ("reg_64x512_go_bf16", synth.gaussian_outlier_weight(64, 512, 0), "k64_row", "weight_b"),
        ("reg_33x200_s25_k64row", s((33, 200), 25), "k64_row", "weight_b"),
        ("reg_33x200_s25_k32row", s((33, 200), 25), "k32_row", "weight_b"),
        ("reg_70x328_s26_n2k64", s((70, 328), 26), "n2k64", "weight_b"),
        ("reg_70x328_s26_n4k64", s((70, 328), 26), "n4k64", "weight_b"),
        ("reg_70x328_s26_n16k64", s((70, 328), 26), "n16k64", "weight_b"),
        ("reg_70x328_s26_n32k64", s((70, 328), 26), "n32k64", "weight_b"),
        ("reg_130x328_s27_n64k64", s((130, 328), 27), "n64k64", "weight_b"),
        ("reg_2x17x200_s28_act_m8k64", s((2, 17, 200), 28), "m8k64", "activation_a"),
        ("reg_33x256_act_k64row_bf16", synth.activations(33, 256, 3, outlier_fraction=0.02), "k64_row", "activation_a"),
        # regions one block wide (columns left of / inside / right of the whole 32-column chunks) and "layer"
        ("reg_64x384_s31_n8k16", s((64, 384), 31), "n8k16", "weight_b"),
        ("reg_70x1120_s32_n8k16", s((70, 1120), 32), "n8k16", "weight_b"),
        ("reg_48x512_st_bf16_n8k16", synth.student_t_weight(48, 512, 2), "n8k16", "weight_b"),
        ("reg_2x17x200_s33_act_m16k16", s((2, 17, 200), 33), "m16k16", "activation_a"),
        ("reg_40x1104_act_m16k16_bf16", synth.activations(40, 1104, 4, outlier_fraction=0.02), "m16k16", "activation_a"),
        ("reg_64x256_s34_layer", s((64, 256), 34), "layer", "weight_b"),
        ("reg_33x200_s35_act_layer", s((33, 200), 35), "layer", "activation_a"),
    ]
    neg_zero = torch.zeros((4, 32))
    neg_zero[:, ::2] = -0.0
    neg_zero[0, 5] = 1.0
    neg_zero[1, 7] = -1e-12
    cases.append(("neg_zero_4x32_f32", neg_zero, "oracle16", "weight_b"))
    return cases


def rotation_case_list(rot):
    g = torch.Generator().manual_seed(24)
    x150 = torch.randn((7, 150), generator=g)
    g2 = torch.Generator().manual_seed(31)
    x300 = (torch.randn((5, 300), generator=g2) * 3).to(torch.bfloat16)
    x512 = synth.activations(9, 512, 5, outlier_fraction=0.02)
    out = {}
    for spec in rot.TRANSFORM_BANK:
        if spec.block_size is None:
            continue
        for tag, x in (("f32_7x150", x150), ("bf16_5x300", x300), ("bf16_9x512", x512)):
            key = f"{spec.name}__{tag}"
            out[key + "__x"] = bits(x)
            out[key + "__y"] = bits(rot.apply_transform(x, spec))
        if spec.seed is not None:
            out[f"{spec.name}__signs"] = rot.signed_vector(spec.block_size, spec.seed, device="cpu", dtype=torch.float32).numpy()
    return out


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def digest_cases(pq) -> dict:
    """Full-size tensors: only hashes of the packed bytes are stored."""
    torch.set_num_threads(os.cpu_count() or 1)
    todo = {
        "config1_w_4096x4096": lambda: synth.config1(0)[0],
        "student_t_q_4096x4096_s0": lambda: synth.student_t_weight(4096, 4096, 0),
        "student_t_kv_1024x4096_s1": lambda: synth.student_t_weight(1024, 4096, 1),
    }
    out = {}
    for name, make in todo.items():
        w = make()
        cand = pq.build_candidates(w)
        ids = (cand.e0_errors < cand.e2_errors)
        dq = pq.quant_mixfp4_granularity(w)
        rows, g = cand.rows, cand.groups
        n2 = level_nibbles(cand.e2_codes, False).reshape(rows, g * 16)
        n0 = level_nibbles(cand.e0_codes, True).reshape(rows, g * 16)
        idn = ids.numpy().astype(np.uint8)
        sel = np.where(np.repeat(idn, 16, axis=1).astype(bool), n0, n2)
        scale_values = torch.where(ids, cand.e0_scales, cand.e2_scales).numpy()
        codes, sc, fmt = pack(sel, scale_values, idn, cand.k)
        out[name] = {
            "shape": list(w.shape), "dtype": str(w.dtype).replace("torch.", ""),
            "input_sha256": sha(bits(w)),
            "codes_sha256": sha(codes), "scales_sha256": sha(sc), "fmt_sha256": sha(fmt),
            "dequant_sha256": sha(bits(dq)),
            "global_scale_bits": int(np.array([float(cand.global_scale)], np.float32).view(np.uint32)[0]),
            "e0_blocks": int(ids.sum()), "blocks": int(ids.numel()),
            "exact_ties": int((cand.e0_errors == cand.e2_errors).sum()),
        }
        print(name, out[name]["e0_blocks"] / out[name]["blocks"], flush=True)
    return out


CANDIDATE_CASES = ("t_17x79_s3", "t_19x131_s10", "t_11x64_s17_bf16", "t_2x17x70_s14_act", "zeros_9x70_bf16",
                   "student_t_48x384_fp16", "wide_range_24x256_f32", "neg_zero_4x32_f32")


def candidate_case_list(pq) -> dict:
    """Fields of the reference's build_candidates that quant_cases.npz does not hold (the float32
    dequantized values of both candidates), and quantize_e2m1 / quantize_e0m3 on the dense probe of
    the reference's own level test (tests/test_quant_core.py:34-41) plus tie and edge values."""
    out = {}
    wanted = {name: (x, role) for name, x, _, role in quant_case_list() if name in CANDIDATE_CASES}
    for name in CANDIDATE_CASES:
        x, role = wanted[name]
        cand = pq.build_candidates(x, operand_role=role)
        out[f"{name}__e2_dequant"] = cand.e2_dequant.numpy().copy()
        out[f"{name}__e0_dequant"] = cand.e0_dequant.numpy().copy()
        out[f"{name}__grouped_original"] = cand.grouped_original.numpy().copy()
        out[f"{name}__meta"] = np.array([cand.rows, cand.k, cand.groups, cand.padded_k, cand.tail_padding], np.int64)
    probe = torch.linspace(-10, 10, 80001, dtype=torch.float32)
    ties = torch.tensor([0.0, -0.0, 0.25, 0.24999998509883881, 0.2500000298023224, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.5,
                         1.5, 2.4999998, 6.0, 6.5, 7.5, 8.0, 1e-30, 3e38, 4.5, 5.5, -0.1, -0.3, -2.5, -3.5, -6.5, -7.5],
                        dtype=torch.float32)
    x = torch.cat([probe, ties, -ties, torch.randn(4096, generator=torch.Generator().manual_seed(5)) * 3])
    out["probe__x"] = x.numpy().copy()
    out["probe__e2m1"] = pq.quantize_e2m1(x).numpy().copy()
    out["probe__e0m3"] = pq.quantize_e0m3(x).numpy().copy()
    return out


def four_over_six_case_list(pq) -> dict:
    """The E0M3 candidate under scale_rule "four_over_six" (project_quant/scale.py:64-103, 207-225; the
    E2M1 side needs an upstream that is absent).  Inputs: seeded tensors of the reference's tests, a
    wide dynamic range, an all-zero tensor, and the crafted boundary tensor of
    tests/test_quant_core.py:216-226."""
    from project_quant.scale import build_scaled_candidate, compute_global_scale
    s = synth.seeded
    g = torch.Generator().manual_seed(78)
    wide = torch.randn((24, 256), generator=g) * torch.exp2(torch.randint(-30, 4, (24, 256), generator=g).float())
    boundary = torch.zeros((128, 64), dtype=torch.bfloat16)
    boundary[0, 0] = 5.625
    boundary[1, :16] = torch.tensor([1.2891, -0.9062, 0.4258, -0.3438, 1.3984, -1.8125, 2.7500, 1.7969,
                                     -0.7227, -2.0625, -0.3262, -2.3438, -0.4883, -0.6875, 0.2168, -1.0547],
                                    dtype=torch.bfloat16)
    cases = {"s18_16x128_bf16": s((16, 128), 18, torch.bfloat16), "s3_17x80": s((17, 80), 3), "wide_24x256": wide,
             "zeros_4x32": torch.zeros((4, 32)), "boundary_128x64_bf16": boundary,
             "student_t_48x384_bf16": synth.student_t_weight(48, 384, 1)}
    out = {}
    for name, x in cases.items():
        grouped = x.float().reshape(x.shape[0], -1, 16)
        cand = build_scaled_candidate(grouped, format_name="e0m3", global_scale=compute_global_scale(grouped, "four_over_six"),
                                      scale_rule="four_over_six")
        out[f"{name}__grouped"] = grouped.numpy().copy()
        out[f"{name}__codes"] = cand.codes.numpy().copy()
        out[f"{name}__dequant"] = cand.dequant.numpy().copy()
        out[f"{name}__scales"] = cand.scales.numpy().copy()
        out[f"{name}__errors"] = cand.errors.numpy().copy()
        out[f"{name}__expansion_ids"] = cand.expansion_ids.numpy().copy()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    ap.add_argument("--skip-digests", action="store_true")
    ap.add_argument("--only-candidates", action="store_true", help="write candidate_cases.npz only")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import project_quant as pq
    from project_quant import rotation as rot

    np.savez_compressed(os.path.join(HERE, "candidate_cases.npz"), **candidate_case_list(pq))
    np.savez_compressed(os.path.join(HERE, "four_over_six_e0_cases.npz"), **four_over_six_case_list(pq))
    if args.only_candidates:
        return

    quant = {}
    names = []
    for name, x, mode, role in quant_case_list():
        r = run_quant_case(pq, x, mode, role)
        names.append(f"{name}|{mode}|{role}|{str(x.dtype).replace('torch.', '')}|{'x'.join(map(str, x.shape))}")
        for key, value in r.items():
            quant[f"{name}__{key}"] = value
    quant["__cases__"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **quant)
    np.savez_compressed(os.path.join(HERE, "rotation_cases.npz"), **rotation_case_list(rot))
    if not args.skip_digests:
        with open(os.path.join(HERE, "digests.json"), "w") as f:
            json.dump({"torch": torch.__version__, "cases": digest_cases(pq)}, f, indent=1, sort_keys=True)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
