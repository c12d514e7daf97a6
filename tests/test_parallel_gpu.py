"""Row-parallel decode linear with the all-reduce fused into the GEMV kernel, on two GPUs of one
node (skipped on a single-GPU machine).  One process per GPU; the fused result must equal the
separate GEMV + NCCL all-reduce bit for bit at world size 2 (a + b in either order), be identical
on both ranks, stay within 1e-3 of the oracle, and survive many launches in a row (the packet
sequence numbers and the two buffer parities) including replays of a captured CUDA graph."""

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


def _worker(rank: int, world: int, port: int, results):
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
        shard = parallel.quantize_shard(w[:, a:b].cuda()).to_kernel_layout().with_decode_table()
        comm = parallel.PeerCommunicator(slot_floats=8 * n)
        outs = []
        for it, m in enumerate([1, 4, 8, 1, 2, 3, 1, 1]):          # an odd and an even count per parity
            x = synth.activations(m, k, seed=100 + it).cuda()
            xs = x[:, a:b].contiguous()
            fused = comm.linear(xs, shard, out_dtype=torch.float32)
            assert fused is not None
            ref = mx.mixfp4_linear(xs, shard, out_dtype=torch.float32)
            dist.all_reduce(ref)
            assert torch.equal(fused, ref), f"launch {it}: fused all-reduce differs from GEMV + all_reduce"
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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_row_parallel_gemv_allreduce_two_gpus():
    import torch.multiprocessing as mp
    import oracle
    ctx = mp.get_context("spawn")
    results = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for port in [_free_port()] for r in range(2)]
    for p in procs:
        p.start()
    w, outs = results.get()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # the sharded, fused result against the oracle on the whole (unsharded) weight
    ref = oracle.quantize(w.float().numpy())
    wq = oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16"))
    for x, y in outs:
        assert oracle.relative_l2(y.numpy(), oracle.linear(x.float().numpy(), wq)) <= 1e-3


def test_fused_allreduce_world_one_is_the_plain_gemv():
    import mixfp4_b200 as mx
    from mixfp4_b200 import parallel, synth
    w = synth.student_t_weight(300, 1024, seed=9)
    packed = mx.quantize_packed(w.cuda())[0].to_kernel_layout().with_decode_table()
    comm = parallel.PeerCommunicator(slot_floats=8 * 300)
    for m in (1, 8, 3):
        x = synth.activations(m, 1024, seed=m).cuda()
        assert torch.equal(comm.linear(x, packed, out_dtype=torch.float32), mx.mixfp4_linear(x, packed, out_dtype=torch.float32))
    assert comm.linear(synth.activations(9, 1024, seed=1).cuda(), packed) is None       # more than 8 rows: not fused
    assert comm.status.item() == 0
    comm.close()
