"""Host-side multi-GPU logic with CPU ranks (gloo, world size 2): partitions and the (O, LSE) exchange."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import HD, ROOT


def test_partitions_cover_everything():
    from blockgtq_b200.sharding import block_partition, chunk_bounds, owner_of_append
    for n, w in [(16, 1), (16, 8), (17, 4), (3, 8), (256, 8)]:
        seen = []
        for r in range(w):
            lo, hi = block_partition(n, w, r)
            seen += list(range(lo, hi))
        assert seen == list(range(n))
    for T, w in [(131072, 8), (1000, 4), (255, 2), (0, 2), (131073, 8)]:
        cov = []
        for r in range(w):
            lo, hi = chunk_bounds(T, w, r)
            assert lo % 256 == 0 or lo == T
            cov += list(range(lo, hi))
        assert cov == list(range(T))
        own = owner_of_append(T, w)
        lo, hi = chunk_bounds(T + 1, w, own)
        assert lo <= T < hi


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from blockgtq_b200.sharding import chunk_bounds, gather_partials
        from oracle import bgtq_oracle as O
        rng = np.random.default_rng(0)                      # same data on every rank
        B, n_q, T = 2, 4, 700
        q = rng.normal(size=(B, n_q, HD)).astype(np.float16)
        k = (rng.normal(size=(B, T, HD)) * 2).astype(np.float16)
        v = rng.normal(size=(B, T, HD)).astype(np.float16)
        lo, hi = chunk_bounds(T, world + 1, rank)           # world+1 chunks: the last one stays empty on purpose
        o = np.zeros((B, n_q, HD), np.float32)
        lse = np.zeros((B, n_q), np.float32)
        for b in range(B):
            ob, lb = O.attend_fp16(q[b], k[b, lo:hi], v[b, lo:hi], 0.0884)
            o[b], lse[b] = ob, lb
        if rank == world - 1:                                 # last rank also covers the remaining tokens
            lo2, hi2 = chunk_bounds(T, world + 1, world)
            for b in range(B):
                o2, l2 = O.attend_fp16(q[b], k[b, lo2:hi2], v[b, lo2:hi2], 0.0884)
                m, ll = O.combine(np.stack([o[b], o2]), np.stack([lse[b], l2]))
                o[b], lse[b] = m, ll
        po, pl = gather_partials(torch.from_numpy(o), torch.from_numpy(lse))
        assert po.shape == (B, n_q, world, HD) and pl.shape == (B, n_q, world)
        worst = 0.0
        for b in range(B):
            got, _ = O.combine(po[b].permute(1, 0, 2).numpy(), pl[b].permute(1, 0).numpy())
            want, _ = O.attend_fp16(q[b], k[b], v[b], 0.0884)
            worst = max(worst, float(np.abs(got - want).max()))
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


def test_sequence_chunk_exchange_gloo_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world and max(ret.values()) < 1e-5, dict(ret)
