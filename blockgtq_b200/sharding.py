"""Multi-GPU partitioning of the packed-cache decode path (one process per GPU).

Two schemes, both new relative to the reference (which is single-GPU):

* **batch x KV-head partition** -- every (batch entry, KV head) owns its cache rows, tables and
  query group, so ranks simply hold disjoint slices and no collective touches the data path
  (:func:`block_partition`).
* **sequence chunks** for one long sequence -- rank r caches tokens ``chunk_bounds(T, W, r)``; each
  rank runs the split-KV decode over its chunk and produces one normalised partial
  ``(O (B, n_q, 128) fp32, LSE (B, n_q) fp32)``; the partials are exchanged with ONE all-gather of a
  fused ``(B, n_q, 129)`` fp32 buffer (16.5 KB per layer for 32 query heads) and merged by the combine
  kernel on every rank (:func:`gather_partials`, :func:`sharded_attend`).  Remote partials are only
  ever read from the local receive buffer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

HD = 128

__all__ = ["block_partition", "chunk_bounds", "owner_of_append", "pack_partial", "gather_partials",
           "sharded_attend", "SequenceShard"]


def block_partition(n_items: int, world: int, rank: int):
    """Contiguous share [lo, hi) of ``n_items`` for ``rank``; sizes differ by at most one."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def chunk_bounds(n_tokens: int, world: int, rank: int, align: int = 256):
    """Token range [lo, hi) of a sequence cached on ``rank``: equal chunks rounded up to ``align``
    tokens (the decode kernel's tile), the last ranks may get a shorter or empty chunk."""
    per = -(-n_tokens // world)
    per = -(-per // align) * align
    lo = min(n_tokens, rank * per)
    return lo, min(n_tokens, lo + per)


def owner_of_append(n_tokens: int, world: int, align: int = 256) -> int:
    """Rank that stores token index ``n_tokens`` (the next appended token)."""
    per = -(-max(n_tokens + 1, 1) // world)
    per = -(-per // align) * align
    return min(world - 1, n_tokens // per)


def pack_partial(o32: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
    """(B, n_q, 128) fp32 + (B, n_q) fp32 -> one (B, n_q, 129) fp32 message."""
    return torch.cat([o32, lse.unsqueeze(-1)], dim=-1).contiguous()


def gather_partials(o32: torch.Tensor, lse: torch.Tensor, group=None):
    """All-gather every rank's (O, LSE) partial.

    Returns ``(part_o (B, n_q, W, 128), part_lse (B, n_q, W))`` in rank order, the layout the combine
    kernel takes as "splits".  A rank with no tokens sends LSE = -inf and is ignored by the merge."""
    world = dist.get_world_size(group)
    msg = pack_partial(o32, lse)
    buf = torch.empty((world,) + tuple(msg.shape), dtype=msg.dtype, device=msg.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(buf, msg, group=group)          # one ncclAllGather
    else:                                                           # CPU ranks (tests): per-rank views of buf
        dist.all_gather(list(buf.unbind(0)), msg, group=group)
    part_o = buf[..., :HD].permute(1, 2, 0, 3).contiguous()
    part_lse = buf[..., HD].permute(1, 2, 0).contiguous()
    return part_o, part_lse


def sharded_attend(mgr, layer_idx: int, q: torch.Tensor, group=None, *, n_splits: int = None,
                   seq_len: int = None) -> torch.Tensor:
    """Decode attention for one long sequence whose cache is split across the ranks of ``group``:
    local split-KV decode + combine -> all-gather of (O, LSE) -> final combine.  ``mgr`` is this
    rank's :class:`BlockGTQKVManager` holding only its own chunk; ``seq_len`` = number of its cached
    tokens to attend over (default: all).  Returns (B, n_q, 128) fp16."""
    from .layer import combine
    _out, o32, lse = mgr.attend(layer_idx, q, seq_len, n_splits=n_splits, want_partial=True)
    part_o, part_lse = gather_partials(o32, lse, group)
    out, _, _ = combine(part_o, part_lse, mgr.n_kv)
    return out


class SequenceShard:
    """Attach sequence sharding to a :class:`BlockGTQKVManager` that holds this rank's chunk of one
    long sequence, so that ``mgr.append_and_attend`` returns the attention over ALL ranks' tokens.

    Per layer the manager then runs, inside its replayed CUDA graph: query rotation (+ the append on
    the rank that owns the tail), split-KV decode over the local chunk, a combine that writes the
    local ``[O fp32 | LSE]`` message in place, ONE all-gather of the messages, and the merge of the
    gathered messages (``bgtq_combine_ranks``).  Every rank must call ``append_and_attend`` for every
    layer with the same query; only the owner's ``k_new`` / ``v_new`` are used.  Remote results are
    read from the local receive buffer only."""

    def __init__(self, mgr, group=None, owner: int = None, transport: str = "nccl"):
        """``transport``: "nccl" = one ``all_gather_into_tensor`` per layer; "p2p" = the library's
        peer-memory exchange (``bgtq_exchange_publish`` / ``bgtq_exchange_merge``) on buffers from
        ``torch.distributed._symmetric_memory`` (single node, NVLink peers)."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.is_owner = self.rank == (self.world - 1 if owner is None else owner)
        mgr._ensure_storage()
        self.B, self.n_q = mgr.B, mgr.n_q
        rows = mgr.B * mgr.n_q
        dev = mgr.device
        self.stride = rows * (HD + 1)                    # floats per message (a multiple of 4 when rows is)
        self.msg = torch.zeros(self.stride, dtype=torch.float32, device=dev)
        self.msg_o = self.msg[:rows * HD].view(mgr.B, mgr.n_q, HD)
        self.msg_lse = self.msg[rows * HD:].view(mgr.B, mgr.n_q)
        self.transport = transport
        self._status = mgr._status
        if transport == "p2p":
            if self.stride % 4:
                raise ValueError("peer-memory exchange needs batch * query heads to be a multiple of 4")
            import torch.distributed._symmetric_memory as symm_mem
            grp = dist.group.WORLD if group is None else group
            self._buf = symm_mem.empty(2 * self.world * self.stride, dtype=torch.float32, device=dev)
            self._flags = symm_mem.empty(max(self.world, 16), dtype=torch.int32, device=dev)
            self._buf.zero_()
            self._flags.zero_()
            h_buf = symm_mem.rendezvous(self._buf, grp)
            h_flg = symm_mem.rendezvous(self._flags, grp)
            self._peer_bufs = torch.tensor(list(h_buf.buffer_ptrs), dtype=torch.int64, device=dev)
            self._peer_flags = torch.tensor(list(h_flg.buffer_ptrs), dtype=torch.int64, device=dev)
            self._seq = torch.zeros(1, dtype=torch.int32, device=dev)
            self._tickets = torch.zeros(2, dtype=torch.int32, device=dev)
            self._handles = (h_buf, h_flg)
            torch.cuda.synchronize(dev)
            dist.barrier(group)                          # nobody publishes before every flag is zero
        else:
            self.gathered = torch.zeros(self.world, self.stride, dtype=torch.float32, device=dev)
            self.all_gather()                            # communicator set-up outside any graph capture
            torch.cuda.synchronize(dev) if dev.type == "cuda" else None
        mgr._exchange = self

    def combine_publish(self, part_o, part_lse, n_kv, v_rot, programmatic=False):
        """Peer-memory transport: merge this rank's split partials and store the result straight into every
        rank's exchange buffer (one launch; ``exchange_and_merge`` then only waits and merges)."""
        from . import _lib
        B, n_q, S, _ = part_o.shape
        _lib.check(_lib.lib().bgtq_combine_publish(
            _lib.ptr(part_o), _lib.ptr(part_lse), S, _lib.ptr(v_rot), B, n_q, n_kv, _lib.ptr(self._peer_bufs),
            self.rank * self.stride, self.world * self.stride, _lib.ptr(self._peer_flags), self.rank, self.world,
            _lib.ptr(self._seq), _lib.ptr(self._tickets), _lib.COMBINE_PROGRAMMATIC if programmatic else 0,
            _lib.stream_ptr(part_o.device)), "bgtq_combine_publish")
        _lib.count_launch()
        self._published = True

    def exchange_and_merge(self, out):
        """Make every rank's message visible here and merge them into ``out`` (B, n_q, 128) fp16."""
        if self.transport == "p2p":
            from . import _lib
            L, sp = _lib.lib(), _lib.stream_ptr(self.msg.device)
            if not getattr(self, "_published", False):      # message produced by a plain combine: publish it
                _lib.check(L.bgtq_exchange_publish(
                    _lib.ptr(self.msg), self.stride, _lib.ptr(self._peer_bufs), self.rank * self.stride,
                    self.world * self.stride, _lib.ptr(self._peer_flags), self.rank, self.world, _lib.ptr(self._seq),
                    _lib.ptr(self._tickets), sp), "bgtq_exchange_publish")
                _lib.count_launch()
            self._published = False
            _lib.check(L.bgtq_exchange_merge(
                _lib.ptr(self._buf), self.world, self.stride, self.world * self.stride, _lib.ptr(self._flags),
                _lib.ptr(self._seq), self.B, self.n_q, _lib.ptr(out), out.stride(0), out.stride(1),
                _lib.ptr(self._status), _lib.ptr(self._tickets[1:]), sp), "bgtq_exchange_merge")
            _lib.count_launch()
            return out
        from .layer import combine_ranks
        self.all_gather()
        return combine_ranks(self.gathered, self.B, self.n_q, out=out)

    def all_gather(self):
        if dist.get_backend(self.group) == "nccl":
            dist.all_gather_into_tensor(self.gathered, self.msg, group=self.group)
        else:
            dist.all_gather(list(self.gathered.unbind(0)), self.msg, group=self.group)
