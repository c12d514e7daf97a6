"""Tensor-parallel linears on several GPUs of one node (skipped where fewer GPUs are visible; the
single-GPU emulation of the peer packets lives in test_wait_limit_gpu.py).  One process per GPU.

* The row-parallel decode linear with the all-reduce fused into the GEMV kernel: at world size 2 the
  result equals GEMV + NCCL all-reduce bit for bit (a + b in either order), at any world size it is
  identical on all ranks, within 1e-3 of the oracle on the UNSHARDED weight, and it survives many
  launches in a row (sequence numbers, both buffer parities) including replays of a captured graph.
* ColumnParallelMixFP4Linear / RowParallelMixFP4Linear: unequal K shards (K/128 not divisible by the
  world size), the fused branch (M = 1), the NCCL branch on fp32 partial sums (M = 300, and without
  a communicator), every rank taking the same branch; all against the oracle."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results, layout: str = "stream"):
    import torch.distributed as dist
    import mixfp4_b200 as mx
    from mixfp4_b200 import parallel, synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from datetime import timedelta
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=timedelta(seconds=90))
    try:
        n, k = 1000, 2048
        w = synth.student_t_weight(n, k, seed=5)
        a, b = parallel.shard_bounds(k, world, rank, parallel.K_SHARD_MULTIPLE)
        shard = parallel.quantize_shard(w[:, a:b].cuda())
        shard = shard.to_stream_layout() if layout == "stream" else shard.to_kernel_layout().with_decode_table()
        comm = parallel.PeerCommunicator(slot_floats=8 * n)
        outs = []
        for it, m in enumerate([1, 4, 8, 1, 2, 3, 1, 1]):          # an odd and an even count per parity
            x = synth.activations(m, k, seed=100 + it).cuda()
            xs = x[:, a:b].contiguous()
            fused = comm.linear(xs, shard, out_dtype=torch.float32)
            assert fused is not None
            ref = mx.mixfp4_linear(xs, shard, out_dtype=torch.float32)
            dist.all_reduce(ref)
            if world == 2:
                assert torch.equal(fused, ref), f"launch {it}: fused all-reduce differs from GEMV + all_reduce"
            else:
                assert float((fused - ref).norm() / ref.norm()) <= 1e-5
            outs.append((x.cpu(), fused.cpu()))
        # captured graph: four fused launches per replay, replayed three times
        x = synth.activations(1, k, seed=7).cuda()
        xs = x[:, a:b].contiguous()
        expect = comm.linear(xs, shard, out_dtype=torch.float32).clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                ys = [comm.linear(xs, shard, out_dtype=torch.float32, overlap_previous=i > 0) for i in range(4)]
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            for y in ys:
                assert torch.equal(y, expect)
        assert comm.status.item() == 0
        # both ranks hold the same bits
        mine = outs[-1][1].cuda()
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        assert all(torch.equal(t, both[0]) for t in both)
        if rank == 0:
            results.put((w, outs))
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


def _spawn(target, world, *extra):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, results) + extra) for r in range(world)]
    for p in procs:
        p.start()
    out = results.get()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    return out


@pytest.mark.parametrize("world,layout", [(2, "stream"), (2, "kernel"), (4, "stream"), (8, "stream")])
def test_fused_row_parallel_gemv_allreduce(world, layout):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import oracle
    w, outs = _spawn(_worker, world, layout)
    # the sharded, fused result against the oracle on the whole (unsharded) weight
    ref = oracle.quantize(w.float().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    for x, y in outs:
        assert oracle.relative_l2(y.numpy(), oracle.linear(x.float().numpy(), wq)) <= 1e-3


def _layer_worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist
    import mixfp4_b200 as mx
    from mixfp4_b200 import parallel, synth
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=timedelta(seconds=90))
    try:
        n, k = 640, 1152                          # 9 blocks of 128 along K: unequal shards at any world size > 1
        w = synth.student_t_weight(n, k, seed=21)
        comm = parallel.PeerCommunicator(slot_floats=8 * n)
        a, b = parallel.shard_bounds(k, world, rank, parallel.K_SHARD_MULTIPLE)
        row_shard = parallel.quantize_shard(w[:, a:b].cuda())
        fused_layer = parallel.RowParallelMixFP4Linear(row_shard, comm=comm, k_total=k)
        nccl_layer = parallel.RowParallelMixFP4Linear(row_shard, k_total=k)
        c, d = parallel.shard_bounds(n, world, rank)
        col_layer = parallel.ColumnParallelMixFP4Linear(parallel.quantize_shard(w[c:d].cuda()))
        outs = []
        for m in (1, 300):
            x = synth.activations(m, k, seed=m).cuda()
            xs = x[:, a:b].contiguous()
            assert comm.fused_ok(m, k, n) == (m <= 8)
            y_fused = fused_layer(xs, out_dtype=torch.float32)
            y_nccl = nccl_layer(xs, out_dtype=torch.float32)
            assert float((y_fused - y_nccl).norm() / y_nccl.norm()) <= 1e-5
            y_bf16 = fused_layer(xs)
            assert y_bf16.dtype == torch.bfloat16
            y_col = col_layer(x, out_dtype=torch.float32)
            assert y_col.shape == (m, d - c)
            parts = [torch.empty((m, parallel.shard_bounds(n, world, r)[1] - parallel.shard_bounds(n, world, r)[0]),
                                 dtype=torch.float32, device="cuda") for r in range(world)]
            if len({p.shape for p in parts}) == 1:
                dist.all_gather(parts, y_col)
                y_col_full = torch.cat(parts, dim=1)
            else:
                y_col_full = None
            outs.append((x.cpu(), y_fused.cpu(), y_nccl.cpu(), y_bf16.float().cpu(),
                         None if y_col_full is None else y_col_full.cpu(), (c, d), y_col.cpu()))
        assert comm.status.item() == 0
        if rank == 0:
            results.put((w, outs))
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_and_row_parallel_layers(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import oracle
    w, outs = _spawn(_layer_worker, world)
    ref = oracle.quantize(w.float().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    for x, y_fused, y_nccl, y_bf16, y_col_full, (c, d), y_col in outs:
        ystar = oracle.linear(x.float().numpy(), wq)
        assert oracle.relative_l2(y_fused.numpy(), ystar) <= 1e-3
        assert oracle.relative_l2(y_nccl.numpy(), ystar) <= 1e-3
        # bf16 output: one bf16 ulp of the value, plus the fp32 summation noise that matters where an output
        # cancels to nearly zero
        floor = 1e-5 * float(np.sqrt(np.mean(ystar.astype(np.float64) ** 2)))
        assert np.all(np.abs(y_bf16.numpy() - ystar) <= np.abs(ystar) * 2.0 ** -7 + floor)
        assert oracle.relative_l2(y_col.numpy(), ystar[:, c:d]) <= 1e-3
        if y_col_full is not None:
            assert oracle.relative_l2(y_col_full.numpy(), ystar) <= 1e-3


def test_fused_allreduce_world_one_is_the_plain_gemv():
    import mixfp4_b200 as mx
    from mixfp4_b200 import parallel, synth
    w = synth.student_t_weight(300, 1024, seed=9)
    packed = mx.quantize_packed(w.cuda())[0].to_stream_layout()
    comm = parallel.PeerCommunicator(slot_floats=8 * 300)
    for m in (1, 8, 3):
        x = synth.activations(m, 1024, seed=m).cuda()
        assert torch.equal(comm.linear(x, packed, out_dtype=torch.float32), mx.mixfp4_linear(x, packed, out_dtype=torch.float32))
    assert comm.linear(synth.activations(9, 1024, seed=1).cuda(), packed) is None       # more than 8 rows: not fused
    assert comm.status.item() == 0
    comm.close()
