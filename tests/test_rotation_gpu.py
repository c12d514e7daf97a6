"""GPU parity of the FWHT kernel: bit-exact against fixtures from the reference's
apply_transform (fp32 and bf16 inputs, whole transform bank, K tails), plus the
properties the reference tests (tests/test_permutation_rotation.py:121-136)."""

import numpy as np
import pytest
import torch

import oracle
from mixfp4_b200 import rotation as rot
from mixfp4_b200 import synth
from tests.golden_io import rotation_cases

pytestmark = pytest.mark.gpu


def _keys():
    return sorted(k[: -len("__x")] for k in rotation_cases() if k.endswith("__x"))


@pytest.mark.parametrize("key", _keys())
def test_apply_transform_matches_reference(key):
    z = rotation_cases()
    name, tag = key.split("__")
    x, y = z[key + "__x"], z[key + "__y"]
    if tag.startswith("bf16"):
        xt = torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).cuda()
        got = rot.apply_transform(xt, name).cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got, y)
    else:
        got = rot.apply_transform(torch.from_numpy(x.copy()).cuda(), name).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), y.view(np.uint32))


def test_single_rounding_mode_matches_oracle():
    x = synth.activations(37, 1000, 8, outlier_fraction=0.01)          # K tail of 104
    got = rot.apply_transform(x.cuda(), "H128", rounding="once").cpu()
    ref = oracle.f32_to_bf16_bits(oracle.fwht(x.float().numpy(), 128))
    assert np.array_equal(got.view(torch.int16).numpy().view(np.uint16), ref)
    assert torch.equal(got[:, 896:], x[:, 896:])                       # tail passes through


def test_rotation_dense_equivalence_and_orthogonality():
    g = torch.Generator().manual_seed(24)
    x = torch.randn((7, 150), generator=g).cuda()
    for spec in rot.TRANSFORM_BANK:
        dense = rot.dense_transform_matrix(spec, 150, device="cuda")
        torch.testing.assert_close(rot.apply_transform(x, spec), x @ dense, rtol=2e-6, atol=2e-6)
        torch.testing.assert_close(dense.T @ dense, torch.eye(150, device="cuda"), rtol=2e-6, atol=2e-6)


def test_high_precision_rotation_equivalence():
    g = torch.Generator().manual_seed(25)
    x = torch.randn((11, 150), generator=g).cuda()
    w = torch.randn((19, 150), generator=g).cuda()
    for spec in rot.TRANSFORM_BANK:
        check = rot.verify_rotation_equivalence(x, w, spec)
        assert check["passed"], check


def test_in_place_and_involution():
    x = synth.seeded((64, 512), 2).cuda()
    y = rot.apply_transform(x, "H64")
    back = rot.apply_transform(y, "H64")                               # H is symmetric orthogonal
    torch.testing.assert_close(back, x, rtol=1e-5, atol=1e-5)
    assert rot.fwht(x[:, :128].contiguous()).shape == (64, 128)
    with pytest.raises(ValueError, match="power of two"):
        rot.fwht(x[:, :100].contiguous())


def test_single_rounding_h128_on_whole_blocks_with_special_values():
    """K a multiple of 128, 16-bit input, one rounding: the kernel the prefill GEMM runs in front of itself
    (a pair of lanes per block, packed fp32 operations, reciprocal-form division for a whole lane).  Rows
    with zeros, negative zeros, constants (every output but one cancels to zero), values far below 2^-100,
    infinities and NaN take the lane-by-lane division instead and must give the same bits as the oracle."""
    x = synth.activations(96, 1024, 12, outlier_fraction=0.02).float()
    x[3] = 0.0
    x[4] = -0.0
    x[5] = 1.5
    x[6, ::2] = 0.0
    x[7] *= 1e-36
    x[8, 5] = float("inf")
    x[9, 130] = float("nan")
    x[10, :128] = -0.0
    x[11, 256:384] = 3.0e38
    xb = x.to(torch.bfloat16)
    got = rot.apply_transform(xb.cuda(), "H128", rounding="once").cpu().view(torch.int16).numpy().view(np.uint16)
    with np.errstate(all="ignore"):
        ref = oracle.f32_to_bf16_bits(oracle.fwht(xb.float().numpy(), 128))
    nan = np.isnan(oracle.bf16_bits_to_f32(ref))
    assert np.array_equal(np.isnan(oracle.bf16_bits_to_f32(got)), nan)
    assert np.array_equal(got[~nan], ref[~nan])
    # the same through fp16 and against the general kernel (a K tail keeps it off the whole-block kernel)
    xh = synth.activations(64, 512, 13).to(torch.float16)
    whole = rot.apply_transform(xh.cuda(), "H128", rounding="once").cpu()
    tail = rot.apply_transform(torch.cat([xh, xh[:, :16]], dim=1).cuda(), "H128", rounding="once").cpu()
    assert torch.equal(whole, tail[:, :512])


@pytest.mark.parametrize("rounding,dtype", [("once", torch.bfloat16), ("reference", torch.bfloat16), ("reference", torch.float16)])
def test_h128_whole_blocks_at_prefill_size_match_oracle(rounding, dtype):
    """The two whole-block kernels on an activation tensor of the prefill benchmark's size (2048 x 4096, 1 % of
    the channels scaled by 30), every output bit against the oracle."""
    x = synth.activations(2048, 4096, 31, outlier_fraction=0.01).to(dtype)
    got = rot.apply_transform(x.cuda(), "H128", rounding=rounding).cpu()
    xf = x.float().numpy()
    if rounding == "once":
        ref = oracle.f32_to_bf16_bits(oracle.fwht(xf, 128))
        assert np.array_equal(got.view(torch.int16).numpy().view(np.uint16), ref)
    elif dtype == torch.bfloat16:
        ref = oracle.f32_to_bf16_bits(oracle.fwht(xf, 128, bf16_stages=True))
        assert np.array_equal(got.view(torch.int16).numpy().view(np.uint16), ref)
    else:
        # fp16 stages: the general kernel (reached through a K tail) is the reference-checked form
        tail = rot.apply_transform(torch.cat([x, x[:, :16]], dim=1).cuda(), "H128", rounding=rounding).cpu()
        assert torch.equal(got, tail[:, :4096])
