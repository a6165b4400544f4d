"""The peer-memory exchange of a sequence-sharded cache (combine + publish, bounded wait + merge), driven on
ONE GPU: the buffers, flags and counters of two "ranks" live side by side in this process and the kernels of
both run one after the other on one stream, so no kernel ever waits for a kernel that has not run yet.  The
two-GPU run of the same protocol is tests/test_gpu_multi.py."""
import numpy as np
import pytest
import torch

from blockgtq_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD = 128


class _Rank:
    def __init__(self, rank, world, rows):
        self.rank, self.world = rank, world
        self.stride = rows * (HD + 1)
        self.buf = torch.zeros(2 * world * self.stride, dtype=torch.float32, device=DEV)
        self.flags = torch.zeros(16, dtype=torch.int32, device=DEV)
        self.seq = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.tickets = torch.zeros(2, dtype=torch.int32, device=DEV)
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)


def _ptrs(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


def _merge(rk, B, n_q, out):
    L = _lib.lib()
    _lib.check(L.bgtq_exchange_merge(rk.buf.data_ptr(), rk.world, rk.stride, rk.world * rk.stride, rk.flags.data_ptr(),
                                     rk.seq.data_ptr(), B, n_q, out.data_ptr(), out.stride(0), out.stride(1),
                                     rk.status.data_ptr(), rk.tickets[1:].data_ptr(), _lib.stream_ptr(DEV)),
               "bgtq_exchange_merge")


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("B,gqa", [(2, 2), (24, 4), (48, 2)])
def test_two_rank_exchange_protocol_on_one_gpu(fused, B, gqa):
    """Three steps (both buffer parities, the step counter advancing on the device): every rank's merged
    output must equal the merge of the two ranks' combine results computed directly.  The larger shapes have
    more rows than SMs, where the combine (and its publishing tail) runs as the four-heads-per-CTA kernel
    (gqa 4) or the lean one-row variant (gqa 2)."""
    from blockgtq_b200.layer import combine, combine_ranks
    L = _lib.lib()
    n_kv, S, world = 2, 5, 2
    n_q, rows = n_kv * gqa, B * n_kv * gqa
    gen = torch.Generator(device=DEV).manual_seed(0)
    ranks = [_Rank(r, world, rows) for r in range(world)]
    bufs, flags = _ptrs([r.buf for r in ranks]), _ptrs([r.flags for r in ranks])
    v_rot = torch.linalg.qr(torch.randn(n_kv, HD, HD, generator=gen, device=DEV))[0].contiguous()
    for step in range(3):
        parts, msgs = [], []
        for rk in ranks:
            po = torch.randn(B, n_q, S, HD, generator=gen, device=DEV)
            pl = torch.randn(B, n_q, S, generator=gen, device=DEV) * 3
            if rk.rank == 1 and step == 1:
                pl[:] = -float("inf")                          # a rank without tokens
            pl[0, 0, 2] = -float("inf")
            parts.append((po, pl))
            _o16, o32, lse = combine(po, pl, n_kv, v_rot=v_rot, want_f32=True, want_lse=True)
            msgs.append(torch.cat([o32.reshape(-1), lse.reshape(-1)]))
        want = combine_ranks(torch.stack(msgs), B, n_q)
        for rk, (po, pl) in zip(ranks, parts):
            if fused:
                _lib.check(L.bgtq_combine_publish(
                    po.data_ptr(), pl.data_ptr(), S, v_rot.data_ptr(), B, n_q, n_kv, bufs.data_ptr(),
                    rk.rank * rk.stride, world * rk.stride, flags.data_ptr(), rk.rank, world, rk.seq.data_ptr(),
                    rk.tickets.data_ptr(), 0, _lib.stream_ptr(DEV)), "bgtq_combine_publish")
            else:
                msg = msgs[rk.rank].contiguous()
                _lib.check(L.bgtq_exchange_publish(
                    msg.data_ptr(), rk.stride, bufs.data_ptr(), rk.rank * rk.stride, world * rk.stride,
                    flags.data_ptr(), rk.rank, world, rk.seq.data_ptr(), rk.tickets.data_ptr(),
                    _lib.stream_ptr(DEV)), "bgtq_exchange_publish")
        for rk in ranks:
            out = torch.full((B, n_q, HD), float("nan"), dtype=torch.float16, device=DEV)
            _merge(rk, B, n_q, out)
            torch.cuda.synchronize()
            assert int(rk.status.item()) == 0 and int(rk.seq.item()) == step + 1
            # the exchange's merge adds the ranks with one fused multiply-add chain, the direct merge in two
            # halves: fp32 results one ulp apart, which at these sizes flips an fp16 rounding now and then
            diff = (out.float() - want.float()).abs()
            assert bool((diff <= 2.0 ** -10 * want.float().abs().clamp(min=2.0 ** -14)).all()), f"step {step} rank {rk.rank}"
            if B == 2:
                assert torch.equal(out, want), f"step {step} rank {rk.rank}"
            assert int(rk.flags[0].item()) == step + 1 and int(rk.flags[1].item()) == step + 1
            assert rk.tickets.eq(0).all()


def test_merge_gives_up_when_a_peer_never_publishes():
    """The merge's wait is bounded: with one of two flags never raised it reports status 3, writes zeros and
    returns; the context stays usable (a correct exchange right afterwards succeeds)."""
    L = _lib.lib()
    B, n_q, world = 1, 4, 2
    rows = B * n_q
    ranks = [_Rank(r, world, rows) for r in range(world)]
    bufs, flags = _ptrs([r.buf for r in ranks]), _ptrs([r.flags for r in ranks])
    msg = torch.randn(ranks[0].stride, device=DEV)
    rk = ranks[0]
    _lib.check(L.bgtq_exchange_publish(msg.data_ptr(), rk.stride, bufs.data_ptr(), 0, world * rk.stride,
                                       flags.data_ptr(), 0, world, rk.seq.data_ptr(), rk.tickets.data_ptr(),
                                       _lib.stream_ptr(DEV)), "bgtq_exchange_publish")
    out = torch.full((B, n_q, HD), float("nan"), dtype=torch.float16, device=DEV)
    _merge(rk, B, n_q, out)
    torch.cuda.synchronize()
    assert int(rk.status.item()) == 3
    assert out.eq(0).all()
    # the late peer arrives; the next merge of the same step number succeeds
    rk.status.zero_()
    rk.seq.zero_()
    r1 = ranks[1]
    _lib.check(L.bgtq_exchange_publish(msg.data_ptr(), r1.stride, bufs.data_ptr(), r1.stride, world * r1.stride,
                                       flags.data_ptr(), 1, world, r1.seq.data_ptr(), r1.tickets.data_ptr(),
                                       _lib.stream_ptr(DEV)), "bgtq_exchange_publish")
    _merge(rk, B, n_q, out)
    torch.cuda.synchronize()
    assert int(rk.status.item()) == 0 and torch.isfinite(out).all() and not out.eq(0).all()
