"""Readers for the fixtures under tests/golden/ (written by tests/golden/make_golden.py)."""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@dataclass
class QuantCase:
    name: str
    mode: str
    role: str
    dtype: str
    shape: tuple
    data: dict

    def x_f32(self) -> np.ndarray:
        """Input up-cast to fp32 exactly as the reference does (x.to(float32)), shape [rows, K]."""
        raw = self.data["x"]
        if self.dtype == "bfloat16":
            v = (raw.astype(np.uint32) << 16).view(np.float32)
        elif self.dtype == "float16":
            v = raw.view(np.float16).astype(np.float32)
        else:
            v = raw.astype(np.float32)
        return v.reshape(-1, self.shape[-1])


def quant_cases() -> list[QuantCase]:
    z = np.load(os.path.join(GOLDEN, "quant_cases.npz"))
    out = []
    for entry in z["__cases__"]:
        name, mode, role, dtype, shape = str(entry).split("|")
        data = {k.split("__", 1)[1]: z[k] for k in z.files if k.startswith(name + "__")}
        out.append(QuantCase(name, mode, role, dtype, tuple(int(s) for s in shape.split("x")), data))
    return out


def candidate_cases() -> dict:
    """name -> {e2_dequant, e0_dequant, grouped_original, meta} plus 'probe' -> {x, e2m1, e0m3}."""
    z = np.load(os.path.join(GOLDEN, "candidate_cases.npz"))
    out: dict = {}
    for key in z.files:
        name, field = key.split("__", 1)
        out.setdefault(name, {})[field] = z[key]
    return out


def four_over_six_e0_cases() -> dict:
    """name -> {grouped, codes, dequant, scales, errors, expansion_ids} of the E0M3 candidate under the
    reference's scale_rule "four_over_six"."""
    z = np.load(os.path.join(GOLDEN, "four_over_six_e0_cases.npz"))
    out: dict = {}
    for key in z.files:
        name, field = key.split("__", 1)
        out.setdefault(name, {})[field] = z[key]
    return out


def rotation_cases() -> dict:
    z = np.load(os.path.join(GOLDEN, "rotation_cases.npz"))
    return {k: z[k] for k in z.files}


def digests() -> dict:
    with open(os.path.join(GOLDEN, "digests.json")) as f:
        return json.load(f)
