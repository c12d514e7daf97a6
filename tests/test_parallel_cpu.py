"""World-size-2 gloo test of the tensor-parallel host logic (no GPU): shard bounds, the
max-all-reduce of the tensor amax, "shard bytes == slice of the whole tensor's bytes", and
the row-parallel all-reduce of partial sums.  The CPU oracle stands in for the kernels."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mixfp4_b200 import parallel, synth


def test_shard_bounds_cover_and_align():
    for size, world, mult in [(4096, 8, 128), (14336, 8, 128), (1000, 3, 128), (50, 4, 1), (28672, 8, 128)]:
        edges = [parallel.shard_bounds(size, world, r, mult) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == size
        for (a, b), (c, d) in zip(edges, edges[1:]):
            assert b == c and a <= b
        assert all(a % mult == 0 for a, _ in edges)
    assert [parallel.layer_owner(l, 4) for l in range(6)] == [0, 1, 2, 3, 0, 1]
    with pytest.raises(ValueError):
        parallel.shard_bounds(10, 2, 2)


def test_row_parallel_branch_is_decided_from_global_quantities():
    # the fused GEMV + all-reduce keeps x in shared memory; whether it fits is asked for the largest K
    # shard, so ranks with unequal shards agree (m = 8, K = 20 blocks of 128 over 3 ranks: shards of
    # 896, 896 and 768 columns)
    k = 20 * 128
    shards = [b - a for a, b in (parallel.shard_bounds(k, 3, r, 128) for r in range(3))]
    assert shards == [896, 896, 768]
    for m in (1, 8):
        assert parallel.row_parallel_fused_ok(m, k, 4096, 3, 8 * 4096)
    assert not parallel.row_parallel_fused_ok(9, k, 4096, 3, 16 * 4096)          # more than 8 rows
    assert not parallel.row_parallel_fused_ok(8, k, 4096, 3, 4096)               # receive buffer too small
    # near the shared-memory limit the answer follows the largest shard, never this rank's own
    big = 8 * 14336
    fits_whole = parallel.row_parallel_fused_ok(8, big, 4096, 8, 8 * 4096)       # shards of 14336: too large
    assert not fits_whole
    assert parallel.row_parallel_fused_ok(8, 8 * 4096, 4096, 8, 8 * 4096)        # shards of 4096 fit
    # 113 blocks over 2 ranks: 57 and 56 blocks -- both ranks answer for 57
    from mixfp4_b200 import _native as nat
    k2 = 113 * 128
    want = bool(nat.lib().mixfp4_gemv_x_fits(8, 57 * 128, 1))
    assert parallel.row_parallel_fused_ok(8, k2, 1024, 2, 8 * 1024) == want


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synth.student_t_weight(64, 512, 5).float()
        x = synth.activations(3, 512, 6).float()
        whole = oracle.quantize(w.numpy())
        ok = True
        for kind in ("column", "row"):
            shard = parallel.shard_weight(w, kind, world, rank).contiguous()
            amax = parallel.reduce_amax(shard.abs().amax().reshape(1).clone())
            gs = float(np.float32(amax.item()) / np.float32(2688.0))
            ok &= np.float32(gs) == whole.global_scale
            p = oracle.quantize(shard.numpy(), global_scale_in=gs)
            if kind == "column":
                a, b = parallel.shard_bounds(64, world, rank)
                ok &= np.array_equal(p.codes, whole.codes[a:b]) and np.array_equal(p.scales, whole.scales[a:b])
                ok &= np.array_equal(p.fmt, whole.fmt[a:b])
            else:
                a, b = parallel.shard_bounds(512, world, rank, 128)
                ok &= np.array_equal(p.codes, whole.codes[:, a // 2:b // 2])
                ok &= np.array_equal(p.scales, whole.scales[:, a // 16:b // 16])
                ok &= np.array_equal(p.fmt, whole.fmt[:, a // 128:b // 128])
                # row parallel: partial products summed by all-reduce equal the full linear
                wq = oracle.bf16_bits_to_f32(oracle.dequant(p, "bf16"))
                part = torch.from_numpy(oracle.linear(x[:, a:b].contiguous().numpy(), wq))
                dist.all_reduce(part)
                full = oracle.linear(x.numpy(), oracle.bf16_bits_to_f32(oracle.dequant(whole, "bf16")))
                ok &= oracle.relative_l2(part.numpy(), full) <= 1e-6
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_quantize_and_row_parallel_reduce():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}
