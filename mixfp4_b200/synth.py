"""Seeded synthetic weights and activations for the benchmark configurations.

Real Llama checkpoints and the reference's evaluation datasets are not
available offline, so every measurement and parity case uses tensors drawn from a
seeded CPU generator with the shapes and value distributions the configurations
name.  Everything is generated in fp32 on the CPU and then rounded to bf16, so
the CPU oracle and the GPU kernels see identical bytes.
"""

from __future__ import annotations

import torch

# (name, N, K) of one Llama-3-8B decoder layer's linears; multiplicity per layer is 1 each
# except that "kv" stands for k_proj and v_proj and "gate_up" for gate_proj and up_proj.
LLAMA3_8B_LAYERS = (
    ("q", 4096, 4096, 1),
    ("kv", 1024, 4096, 2),
    ("o", 4096, 4096, 1),
    ("gate_up", 14336, 4096, 2),
    ("down", 4096, 14336, 1),
)
LLAMA3_8B_NUM_LAYERS = 32

# Llama-3-70B: hidden 8192, kv 1024, FFN 28672, 80 layers.
LLAMA3_70B_LAYERS = (
    ("q", 8192, 8192, 1),
    ("kv", 1024, 8192, 2),
    ("o", 8192, 8192, 1),
    ("gate_up", 28672, 8192, 2),
    ("down", 8192, 28672, 1),
)
LLAMA3_70B_NUM_LAYERS = 80


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def seeded(shape, seed: int = 0, dtype=torch.float32) -> torch.Tensor:
    """``randn`` from a seeded CPU generator (the reference tests' helper,
    tests/test_quant_core.py:18-20)."""
    return torch.randn(tuple(shape), generator=_gen(seed), dtype=torch.float32).to(dtype)


def gaussian_outlier_weight(n: int, k: int, seed: int = 0, *, std: float = 0.02,
                            outlier_fraction: float = 0.005, outlier_gain: float = 20.0,
                            dtype=torch.bfloat16, generator: torch.Generator | None = None) -> torch.Tensor:
    """N(0, std^2) weight with a fraction of input channels (columns) scaled up."""
    g = generator if generator is not None else _gen(seed)
    w = torch.randn((n, k), generator=g, dtype=torch.float32) * std
    count = int(round(k * outlier_fraction))
    if count > 0:
        idx = torch.randperm(k, generator=g)[:count]
        w[:, idx] *= outlier_gain
    return w.to(dtype)


def student_t_weight(n: int, k: int, seed: int = 0, *, df: int = 4, scale: float = 0.02,
                     dtype=torch.bfloat16) -> torch.Tensor:
    """Student-t(df) * scale, built as z / sqrt(chi2_df / df) from df + 1 normal draws."""
    g = _gen(seed)
    z = torch.randn((n, k), generator=g, dtype=torch.float32)
    chi2 = torch.zeros((n, k), dtype=torch.float32)
    for _ in range(df):
        d = torch.randn((n, k), generator=g, dtype=torch.float32)
        chi2.addcmul_(d, d)
    return (z / torch.sqrt(chi2 / df) * scale).to(dtype)


def activations(m: int, k: int, seed: int = 0, *, outlier_fraction: float = 0.0,
                outlier_gain: float = 30.0, dtype=torch.bfloat16,
                generator: torch.Generator | None = None) -> torch.Tensor:
    """N(0,1) activations; optionally a fraction of channels scaled up (prefill configs)."""
    g = generator if generator is not None else _gen(seed)
    x = torch.randn((m, k), generator=g, dtype=torch.float32)
    count = int(k * outlier_fraction)
    if count > 0:
        idx = torch.randperm(k, generator=g)[:count]
        x[:, idx] *= outlier_gain
    return x.to(dtype)


def config1(seed: int = 0, n: int = 4096, k: int = 4096, m: int = 16):
    """Single linear: Gaussian weight with 0.5% outlier input channels (x20), X ~ N(0,1)."""
    g = _gen(seed)
    w = gaussian_outlier_weight(n, k, generator=g)
    x = activations(m, k, generator=g)
    return w, x
