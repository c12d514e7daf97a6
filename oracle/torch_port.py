"""PyTorch-eager restatement of the reference's CPU path -- TEST / BASELINE INFRASTRUCTURE.

The reference is a Python package that cannot travel to the benchmark machine, so its
CPU cost is reproduced by this port: the same sequence of whole-tensor eager ops
(about forty elementwise passes over [rows, K/16, 16] fp32 intermediates, both
candidates built in full, then a select), run with all host threads.  It is what the
benchmark times as ``cpu_baseline`` / ``--impl reference``; the tests check that it
produces the same bytes as the C oracle.  Nothing in the product imports it.

Steps follow project_quant/candidates.py:62-106, scale.py:28-61, codebook.py:12-43 and
core.py:115-143 of the reference.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _round_e2m1(n: torch.Tensor) -> torch.Tensor:
    mag = n.abs()
    safe = mag + (mag == 0).to(mag.dtype)
    exp = torch.floor(torch.log2(safe)).clamp(min=0)
    pow2 = torch.pow(2.0, exp)
    q = torch.floor(mag / pow2 * 2.0 + 0.5) * pow2 / 2.0
    return n.sign() * q.clamp(max=6.0)


def _round_e0m3(n: torch.Tensor) -> torch.Tensor:
    return n.sign() * n.abs().round().clamp(max=7.0)


def _candidate(blocks: torch.Tensor, scaled: torch.Tensor, gs: torch.Tensor, qmax: float, rounder):
    ideal = (scaled.abs().amax(dim=-1, keepdim=True) / qmax * 1.0).clamp(min=2.0 ** -9, max=448.0)
    scale = ideal.to(torch.float8_e4m3fn).to(torch.float32)
    normalized = torch.where(scale != 0, scaled / scale, torch.zeros_like(scaled))
    codes = rounder(normalized)
    dequant = codes * scale * gs
    errors = ((dequant - blocks) ** 2).sum(dim=-1)
    return codes, dequant, scale.squeeze(-1), errors


@torch.no_grad()
def quantize_dequant(x: torch.Tensor, *, return_parts: bool = False):
    """The reference's quant_mixfp4_granularity(x) with its defaults (oracle16, mse,
    standard): returns the dequantized tensor in x.dtype."""
    k = x.shape[-1]
    rows = x.numel() // k
    src = x.detach().reshape(rows, k).to(torch.float32)
    pad = (-k) % 16
    if pad:
        src = F.pad(src, (0, pad))
    blocks = src.reshape(rows, -1, 16)
    amax = blocks.abs().amax()
    gs = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    c2, d2, s2, e2 = _candidate(blocks, blocks / gs, gs, 6.0, _round_e2m1)
    c0, d0, s0, e0 = _candidate(blocks, blocks / gs, gs, 7.0, _round_e0m3)
    pick = e0 < e2
    chosen = torch.where(pick[..., None], d0, d2).reshape(rows, -1)
    out = chosen[:, :k].reshape(x.shape).to(x.dtype)
    if return_parts:
        return out, {"format_ids": pick.to(torch.uint8), "scales": torch.where(pick, s0, s2),
                     "e2_errors": e2, "e0_errors": e0, "global_scale": gs,
                     "codes": torch.where(pick[..., None], c0, c2)}
    return out


@torch.no_grad()
def linear(x: torch.Tensor, dequant_weight_f32: torch.Tensor) -> torch.Tensor:
    """The reference's linear: stock F.linear on the dequantized weight
    (project_quant/modeling.py:629), in fp32."""
    return F.linear(x.float(), dequant_weight_f32)
