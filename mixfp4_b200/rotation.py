"""Normalised block-Hadamard transform bank, executed by the CUDA FWHT kernel.

Mirrors the interface of the reference's ``project_quant/rotation.py``
(TransformSpec / TRANSFORM_BANK :12-29, get_transform :32-38, signed_vector :41-44,
fwht :47-58, apply_transform :61-75, hadamard_matrix :78-84, dense_transform_matrix
:87-100, verify_rotation_equivalence :103-118): same names, same argument meaning,
same errors.  ``apply_transform`` on a bf16/fp16 tensor reproduces the reference
bit for bit (it rounds to the tensor dtype after every butterfly stage, as eager
PyTorch does); ``rounding="once"`` keeps fp32 through all stages and rounds once,
which is what the rotation pass in front of the prefill GEMM computes.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native as nat


@dataclass(frozen=True)
class TransformSpec:
    name: str
    block_size: int | None
    seed: int | None = None
    deployability: str = "potentially_foldable"


TRANSFORM_BANK = (
    TransformSpec("identity", None, deployability="exact_foldable"),
    TransformSpec("H16", 16),
    TransformSpec("H32", 32),
    TransformSpec("H64", 64),
    TransformSpec("H128", 128),
    TransformSpec("random_signed_H64_seed0", 64, 0),
    TransformSpec("random_signed_H64_seed1", 64, 1),
    TransformSpec("random_signed_H64_seed2", 64, 2),
    TransformSpec("random_signed_H64_seed3", 64, 3),
)

_SUPPORTED_SIZES = (16, 32, 64, 128)
_sign_cache: dict[tuple, torch.Tensor] = {}


def get_transform(value: str | TransformSpec) -> TransformSpec:
    if isinstance(value, TransformSpec):
        return value
    for spec in TRANSFORM_BANK:
        if spec.name.lower() == str(value).lower():
            return spec
    raise ValueError(f"unknown transform {value!r}")


def signed_vector(size: int, seed: int, *, device, dtype) -> torch.Tensor:
    """+-1 vector drawn from a seeded CPU generator (the draw defines the transform)."""
    generator = torch.Generator(device="cpu").manual_seed(seed)
    signs = torch.randint(0, 2, (size,), generator=generator, dtype=torch.int64).mul(2).sub(1)
    return signs.to(device=device, dtype=dtype)


def _device_signs(size: int, seed: int, device) -> torch.Tensor:
    key = (size, seed, str(device))
    if key not in _sign_cache:
        _sign_cache[key] = signed_vector(size, seed, device=device, dtype=torch.float32).contiguous()
    return _sign_cache[key]


def _run_fwht(x: torch.Tensor, size: int, signs: torch.Tensor | None, stagewise: bool,
              out: torch.Tensor | None = None) -> torch.Tensor:
    if x.dtype not in nat.DTYPE_CODE:
        raise TypeError("x must be bfloat16, float16 or float32")
    if size not in _SUPPORTED_SIZES:
        raise NotImplementedError(f"the FWHT kernel supports block sizes {_SUPPORTED_SIZES}, got {size}")
    host = not x.is_cuda
    src = x.cuda() if host else x
    if src.stride(-1) != 1 or not src.is_contiguous():
        src = src.contiguous()
    k = src.shape[-1]
    rows = src.numel() // k
    dst = out if out is not None else torch.empty_like(src)
    with torch.cuda.device(src.device):
        st = nat.lib().mixfp4_fwht(src.data_ptr(), dst.data_ptr(), nat.DTYPE_CODE[src.dtype], rows, k, k, k,
                                   size, nat.ptr(signs), 1 if stagewise else 0, nat.stream_ptr(src.device))
    nat.check("mixfp4_fwht", st)
    return dst.to(x.device) if host else dst


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform over the whole last dimension."""
    size = x.shape[-1]
    if size <= 0 or size & (size - 1):
        raise ValueError("FWHT final dimension must be a positive power of two")
    return _run_fwht(x, size, None, stagewise=True)


def apply_transform(x: torch.Tensor, value: str | TransformSpec, *, rounding: str = "reference") -> torch.Tensor:
    """Block-Hadamard along the last axis; a tail shorter than the block passes through.

    rounding="reference": round to x.dtype after every stage (bit-equal to the reference
    on bf16/fp16 inputs; no effect for fp32).  rounding="once": fp32 stages, one rounding.
    """
    spec = get_transform(value)
    if spec.block_size is None:
        return x
    if rounding not in ("reference", "once"):
        raise ValueError("rounding must be 'reference' or 'once'")
    size = spec.block_size
    if x.shape[-1] // size == 0:
        return x
    if size not in _SUPPORTED_SIZES:
        raise NotImplementedError(f"the FWHT kernel supports block sizes {_SUPPORTED_SIZES}, got {size}")
    dev = x.device if x.is_cuda else torch.device("cuda", torch.cuda.current_device())
    signs = _device_signs(size, spec.seed, dev) if spec.seed is not None else None
    return _run_fwht(x, size, signs, stagewise=(rounding == "reference"))


def hadamard_matrix(size: int, *, device=None, dtype=torch.float32) -> torch.Tensor:
    if size <= 0 or size & (size - 1):
        raise ValueError("Hadamard size must be a positive power of two")
    matrix = torch.ones((1, 1), device=device, dtype=dtype)
    while matrix.shape[0] < size:
        top = torch.cat((matrix, matrix), 1)
        matrix = torch.cat((top, torch.cat((matrix, -matrix), 1)), 0)
    return matrix / (size ** 0.5)


def dense_transform_matrix(value: str | TransformSpec, k: int, *, device=None, dtype=torch.float32) -> torch.Tensor:
    """The K x K matrix T with apply_transform(x) == x @ T."""
    spec = get_transform(value)
    matrix = torch.eye(k, device=device, dtype=dtype)
    if spec.block_size is None:
        return matrix
    size = spec.block_size
    base = hadamard_matrix(size, device=device, dtype=dtype)
    if spec.seed is not None:
        base = torch.diag(signed_vector(size, spec.seed, device=device, dtype=dtype)) @ base
    for start in range(0, k // size * size, size):
        matrix[start:start + size, start:start + size] = base
    return matrix


@torch.no_grad()
def verify_rotation_equivalence(x: torch.Tensor, weight: torch.Tensor, value: str | TransformSpec) -> dict:
    """Checks (xT)(wT)^T == x w^T in fp32, as the reference's model adapter does before folding."""
    spec = get_transform(value)
    reference = x.float() @ weight.float().T
    rotated = apply_transform(x.float(), spec) @ apply_transform(weight.float(), spec).T
    delta = rotated.to(reference.device) - reference
    relative = torch.linalg.vector_norm(delta) / torch.linalg.vector_norm(reference).clamp_min(1e-30)
    return {
        "transform": spec.name,
        "deployability": spec.deployability,
        "max_abs_error": float(delta.abs().max().item()),
        "relative_l2_error": float(relative.item()),
        "passed": bool(relative <= 2e-5),
    }
