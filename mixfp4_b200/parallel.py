"""Tensor-parallel sharding of mixed-FP4 linears over the GPUs of one node.

The reference is single-GPU (project_quant/modeling.py:168 pins everything to cuda:0); this
module is the multi-GPU form of its per-layer loop (modeling.py:604-639).  One process per
GPU, torch.distributed (NCCL over NVLink on GPUs, gloo in the CPU tests) for the plumbing:

* column parallel (q/k/v, gate, up): the weight is split along N, x is replicated, every
  rank keeps its slice of y -- no collective;
* row parallel (o, down): the weight is split along K at multiples of 128 (whole format
  bytes, whole Hadamard blocks), x arrives split, every rank produces a partial [M, N] and
  the partials are summed with one all-reduce.

Quantization blocks are 1 x 16 row segments, so a shard quantized with the WHOLE tensor's
amax has exactly the bytes of the corresponding slice of the whole packed tensor; the only
exchange quantization needs is a max-all-reduce of one float per tensor.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

K_SHARD_MULTIPLE = 128


def shard_bounds(size: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """[start, stop) of rank's shard of an axis of length size; shard edges are multiples of
    `multiple`, the last shard takes the remainder."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    units = -(-size // multiple)
    per, extra = divmod(units, world)
    start_u = rank * per + min(rank, extra)
    stop_u = start_u + per + (1 if rank < extra else 0)
    return min(start_u * multiple, size), min(stop_u * multiple, size)


def layer_owner(layer_index: int, world: int) -> int:
    """Layer-sharded model quantization: layer l is quantized by rank l mod world."""
    return layer_index % world


def reduce_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """Whole-tensor max|w| from per-shard values (one float, MAX all-reduce, in place)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


def shard_weight(w: torch.Tensor, kind: str, world: int, rank: int) -> torch.Tensor:
    """The rank's slice of a dense [N, K] weight: kind 'column' splits N, 'row' splits K."""
    n, k = w.shape
    if kind == "column":
        a, b = shard_bounds(n, world, rank)
        return w[a:b]
    if kind == "row":
        a, b = shard_bounds(k, world, rank, K_SHARD_MULTIPLE)
        return w[:, a:b]
    raise ValueError("kind must be 'column' or 'row'")


def quantize_shard(w_shard: torch.Tensor, group=None, **kwargs):
    """Quantize this rank's shard with the whole tensor's scale (CUDA path)."""
    from .quant import quantize_packed, tensor_amax
    x2 = w_shard if w_shard.is_contiguous() else w_shard.contiguous()
    amax = reduce_amax(tensor_amax(x2), group)
    return quantize_packed(x2, amax=amax, **kwargs)[0]


class ColumnParallelMixFP4Linear(torch.nn.Module):
    """y_shard = x @ W[n0:n1]^T; the output stays sharded along N."""

    def __init__(self, packed_shard):
        super().__init__()
        from .linear import MixFP4Linear
        self.inner = MixFP4Linear(packed_shard)

    def forward(self, x, **kw):
        return self.inner(x, **kw)


class RowParallelMixFP4Linear(torch.nn.Module):
    """y = sum over ranks of x[:, k0:k1] @ W[:, k0:k1]^T (all-reduce of the partials)."""

    def __init__(self, packed_shard, group=None):
        super().__init__()
        from .linear import MixFP4Linear
        self.inner = MixFP4Linear(packed_shard)
        self.group = group

    def forward(self, x_shard, **kw):
        y = self.inner(x_shard, **kw)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, group=self.group)
        return y
