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


def row_parallel_fused_ok(m: int, k_total: int, n: int, world: int, slot_floats: int,
                          multiple: int = K_SHARD_MULTIPLE) -> bool:
    """Whether a row-parallel layer [n, k_total] split over `world` ranks runs the fused GEMV +
    all-reduce for m rows of x.  Decided from global quantities only -- the LARGEST K shard any
    rank holds under shard_bounds -- so every rank takes the same branch even when the shards are
    unequal.  Host arithmetic (no GPU needed)."""
    from . import _native as nat
    largest = max(b - a for a, b in (shard_bounds(k_total, world, r, multiple) for r in range(world)))
    return 1 <= m <= 8 and m * n <= slot_floats and bool(nat.lib().mixfp4_gemv_x_fits(m, largest, 1))


class ColumnParallelMixFP4Linear(torch.nn.Module):
    """y_shard = x @ W[n0:n1]^T; the output stays sharded along N."""

    def __init__(self, packed_shard):
        super().__init__()
        from .linear import MixFP4Linear
        self.inner = MixFP4Linear(packed_shard)

    def forward(self, x, **kw):
        return self.inner(x, **kw)


class PeerCommunicator:
    """Peer-memory exchange area of the fused row-parallel GEMV + all-reduce (one per process).

    slot_floats: the largest M * N a fused call will produce.  The ranks of `group` exchange
    the buffers' IPC handles through torch.distributed; afterwards no host communication
    happens on the data path.  All ranks must issue the same sequence of fused calls.
    """

    def __init__(self, slot_floats: int, group=None, device=None):
        import ctypes
        from . import _native as nat
        self._nat = nat
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.slot_floats = int(slot_floats)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            nat.check("mixfp4_comm_create", nat.lib().mixfp4_comm_create(self.rank, self.world, self.slot_floats,
                                                                         ctypes.byref(handle)))
            self.handle = handle
            if self.world > 1:
                nbytes = nat.lib().mixfp4_comm_handle_bytes()
                mine = ctypes.create_string_buffer(nbytes)
                nat.check("mixfp4_comm_handle", nat.lib().mixfp4_comm_handle(self.handle, mine))
                everyone = [None] * self.world
                dist.all_gather_object(everyone, bytes(mine.raw), group=group)
                blob = ctypes.create_string_buffer(b"".join(everyone), nbytes * self.world)
                nat.check("mixfp4_comm_open", nat.lib().mixfp4_comm_open(self.handle, blob))
                dist.barrier(group=group)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def close(self) -> None:
        if getattr(self, "handle", None) is not None:
            torch.cuda.synchronize(self.device)
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)      # nobody unmaps while a peer may still write
            self._nat.lib().mixfp4_comm_destroy(self.handle)
            self.handle = None

    def fused_ok(self, m: int, k_total: int, n: int, multiple: int = K_SHARD_MULTIPLE) -> bool:
        """row_parallel_fused_ok for this communicator's world size and buffer."""
        return row_parallel_fused_ok(m, k_total, n, self.world, self.slot_floats, multiple)

    def linear(self, x_shard: torch.Tensor, packed_shard, *, out_dtype: torch.dtype | None = None,
               overlap_previous: bool = False) -> torch.Tensor | None:
        """sum over ranks of x_shard @ W_shard^T in one kernel per rank, or None when the shape does
        not qualify (more than 8 rows of x, canonical layout, x too large for shared memory).  Callers
        whose ranks hold unequal shards decide with ``fused_ok`` first."""
        nat = self._nat
        k = packed_shard.k
        m = x_shard.numel() // max(1, x_shard.shape[-1])
        if not (1 <= m <= 8 and packed_shard.layout in ("kernel", "stream") and packed_shard.rotation is None
                and x_shard.dtype == torch.bfloat16 and x_shard.shape[-1] == k and m * packed_shard.n <= self.slot_floats):
            return None
        out_dtype = x_shard.dtype if out_dtype is None else out_dtype
        x2 = x_shard.reshape(-1, k)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = torch.empty((m, packed_shard.n), dtype=out_dtype, device=x_shard.device)
        with torch.cuda.device(x_shard.device):
            st = nat.lib().mixfp4_gemv_allreduce(
                self.handle, x2.data_ptr(), m, x2.stride(0), packed_shard.codes.data_ptr(), nat.ptr(packed_shard.scales),
                packed_shard.global_scale.data_ptr(), nat.ptr(packed_shard.lut), packed_shard.n, k,
                packed_shard.layout_code, y.data_ptr(), nat.DTYPE_CODE[out_dtype], y.stride(0), self.status.data_ptr(),
                nat.gemv_flags(overlap_previous, packed_shard.lut), nat.stream_ptr(x_shard.device))
        if st == nat.E_SHAPE:
            return None
        nat.check("mixfp4_gemv_allreduce", st)
        return y.reshape(*x_shard.shape[:-1], packed_shard.n)


class RowParallelMixFP4Linear(torch.nn.Module):
    """y = sum over ranks of x[:, k0:k1] @ W[:, k0:k1]^T.  With a PeerCommunicator decode shapes run
    the GEMV with the all-reduce fused in; otherwise fp32 partial sums are added by torch.distributed
    and rounded to the output type afterwards.  `k_total` is the unsharded K: the choice between the
    two forms is made from it (not from this rank's shard), so all ranks agree even when the shards
    are unequal."""

    def __init__(self, packed_shard, group=None, comm: PeerCommunicator | None = None, k_total: int | None = None):
        super().__init__()
        from .linear import MixFP4Linear
        self.inner = MixFP4Linear(packed_shard)
        self.group = group
        self.comm = comm
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.k_total = int(k_total) if k_total is not None else packed_shard.k * world

    def forward(self, x_shard, **kw):
        m = x_shard.numel() // max(1, x_shard.shape[-1])
        if (self.comm is not None and self.comm.world > 1 and self.inner.rotation is None
                and self.comm.fused_ok(m, self.k_total, self.inner.out_features)):
            y = self.comm.linear(x_shard, self.inner.packed, out_dtype=kw.get("out_dtype"),
                                 overlap_previous=kw.get("overlap_previous", False))
            if y is None:
                raise RuntimeError("the fused row-parallel kernel refused a shape fused_ok accepted")
            return y
        out_dtype = kw.get("out_dtype") or x_shard.dtype
        y = self.inner(x_shard, **{**kw, "out_dtype": torch.float32})
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, group=self.group)
        return y.to(out_dtype)
