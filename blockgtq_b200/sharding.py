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

    def __init__(self, mgr, group=None, owner: int = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.is_owner = self.rank == (self.world - 1 if owner is None else owner)
        rows = mgr.B * mgr.n_q
        dev = mgr.device
        self.msg = torch.zeros(rows * (HD + 1), dtype=torch.float32, device=dev)
        self.msg_o = self.msg[:rows * HD].view(mgr.B, mgr.n_q, HD)
        self.msg_lse = self.msg[rows * HD:].view(mgr.B, mgr.n_q)
        self.gathered = torch.zeros(self.world, rows * (HD + 1), dtype=torch.float32, device=dev)
        self.all_gather()                      # communicator set-up outside any graph capture
        torch.cuda.synchronize(dev) if dev.type == "cuda" else None
        mgr._exchange = self

    def all_gather(self):
        if dist.get_backend(self.group) == "nccl":
            dist.all_gather_into_tensor(self.gathered, self.msg, group=self.group)
        else:
            dist.all_gather(list(self.gathered.unbind(0)), self.msg, group=self.group)
