"""Two GPUs: a sequence-sharded cache (each rank holds a chunk of the tokens) must give the same attention
as one GPU holding everything, with both exchange transports (NCCL all-gather, peer-memory stores).
Skipped where fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, transport, ret):
    import sys
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import HD, synth_head
    from blockgtq_b200 import BlockGTQKVManager
    from blockgtq_b200.sharding import SequenceShard, chunk_bounds
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        gen = torch.Generator().manual_seed(2024)               # same data on every rank
        B, n_kv, gqa, T, steps = 2, 2, 2, 600, 3
        n_q = n_kv * gqa
        cal = [synth_head(gen, 256, gqa) for _ in range(n_kv)]
        k_all = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)])
        v_all = torch.randn(B, n_kv, T, HD, generator=gen).half()
        qs = (torch.randn(steps, B, n_q, 1, HD, generator=gen) * 2).half()
        ks = torch.randn(steps, B, n_kv, 1, HD, generator=gen).half()
        vs = torch.randn(steps, B, n_kv, 1, HD, generator=gen).half()

        def manager(lo, hi):
            m = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=hi - lo + steps + 8, batch_size=B, k_avg_bits=3.0,
                                  v_bits=3, device=dev)
            m.calibrate(0, torch.stack([c[0] for c in cal]).float(), torch.stack([c[1] for c in cal]).float())
            if hi > lo:
                m._append_tokens(0, k_all[:, :, lo:hi].to(dev), v_all[:, :, lo:hi].to(dev), 0)
            else:
                m._ensure_storage()
            m.seq_len = hi - lo
            return m

        full = manager(0, T)
        lo, hi = chunk_bounds(T, world, rank)
        part = manager(lo, hi)
        SequenceShard(part, transport=transport)
        worst = 0.0
        for s in range(steps):
            want = full.append_and_attend(0, qs[s].to(dev), ks[s].to(dev), vs[s].to(dev))
            full.increment_seq_len()
            got = part.append_and_attend(0, qs[s].to(dev), ks[s].to(dev), vs[s].to(dev))
            part.increment_seq_len()
            torch.cuda.synchronize()
            worst = max(worst, (got.float() - want.float()).abs().max().item())
        part.check_status()
        ret[rank] = worst
        # graphs that captured a collective must be gone before the communicator is destroyed
        part.release_graphs()
        del part, full
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["nccl", "p2p"])
def test_sequence_shard_two_gpus_matches_one_gpu(transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), transport, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(ret.values()) <= 2e-3, dict(ret)
