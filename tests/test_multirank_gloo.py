"""The multi-GPU path on CPU: two gloo ranks, batch sharded, no collective on the data path.

Each rank computes its slice with the CPU oracle (the CUDA kernels need a GPU; what is tested here is the
host-side sharding logic the benchmark and a multi-GPU caller use): slices tile the batch exactly, a
broadcast operand is replicated and its gradient is the all-reduced sum, and the timing reduction is a max.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import crandn, np_c


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gelib_b200 import sharding
        from oracle import oracle as O
        B, l1, l2, l, n = 7, 1, 2, 2, 3
        x = crandn(1, 1, 2 * l1 + 1, n)            # broadcast operand: batch 1
        y = crandn(2, B, 2 * l2 + 1, n)
        g = crandn(3, B, 2 * l + 1, n * n)
        ys, gs = sharding.shard_batch(y, rank, world), sharding.shard_batch(g, rank, world)
        xs = sharding.shard_batch(x, rank, world)
        assert xs.shape[0] == 1
        b, e = sharding.shard_bounds(B, rank, world)
        r = np.zeros((e - b, 2 * l + 1, n * n), np.complex64)
        O.add_CGproduct(r, np_c(xs), np_c(ys))
        xg = np.zeros((1, 2 * l1 + 1, n), np.complex64)
        O.add_CGproduct_back0(xg, np_c(gs), np_c(ys))
        xg_t = torch.from_numpy(xg)
        sharding.allreduce_broadcast_grad(xg_t)
        t = sharding.max_over_ranks(10.0 + rank)
        out[rank] = (b, e, r, xg_t.numpy().copy(), t)
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_the_batch():
    from oracle import oracle as O
    O.build()
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    B, l1, l2, l, n = 7, 1, 2, 2, 3
    x, y, g = crandn(1, 1, 3, n), crandn(2, B, 5, n), crandn(3, B, 5, n * n)
    want = np.zeros((B, 5, n * n), np.complex64)
    O.add_CGproduct(want, np_c(x), np_c(y))
    xg_want = np.zeros((1, 3, n), np.complex64)
    O.add_CGproduct_back0(xg_want, np_c(g), np_c(y))
    covered = []
    for rank in range(world):
        b, e, r, xg, t = out[rank]
        covered.append((b, e))
        assert np.array_equal(r, want[b:e])                   # cells are independent: bit-identical slices
        assert np.allclose(xg, xg_want, rtol=1e-5, atol=1e-5)  # summed over ranks
        assert t == 11.0                                      # max over ranks
    assert covered == [(0, 4), (4, 7)]


def test_shard_bounds_tile_the_batch():
    from gelib_b200.sharding import shard_bounds
    for total in (0, 1, 7, 4096, 262144):
        for world in (1, 2, 3, 4, 8):
            ends = [shard_bounds(total, r, world) for r in range(world)]
            assert ends[0][0] == 0 and ends[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ends[:-1], ends[1:]))
            sizes = [e - b for b, e in ends]
            assert max(sizes) - min(sizes) <= 1
