"""Greedy RoPE-block bit allocation (host side).

Mirrors the contract of the reference's ``greedy_bit_allocation``
(blockgtq/allocator.py:20-55): every block starts at ``min_bits`` and the
remaining budget is handed out one bit at a time to the block with the
largest ``s_i * 4**(-b_i)``; a block at ``max_bits`` is never chosen; ties go
to the lowest index; allocation stops early when no block has a positive
priority.  The result must be *identical* to the reference because the bit
map fixes the packed layout of every (layer, KV-head).

The priorities are exact in float64 (a float32 score times a power of two),
so any evaluation order gives the same winners.  This implementation keeps
the priority vector and only refreshes the entry that changed.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["greedy_bit_allocation"]


def greedy_bit_allocation(scores: torch.Tensor, total_budget: int,
                          min_bits: int = 1, max_bits: int = 8) -> torch.Tensor:
    """Return an int64 ``(n_blocks,)`` bit map summing to ``total_budget``.

    ``scores`` are per-RoPE-block importances (>= 0).  If the budget exceeds
    what the blocks can absorb the result saturates at ``max_bits``; if it is
    below ``n_blocks * min_bits`` every block keeps ``min_bits``.
    """
    n = len(scores)
    bits = np.full(n, int(min_bits), dtype=np.int64)
    left = int(total_budget) - int(bits.sum())
    if left <= 0:
        return torch.from_numpy(bits)

    s = scores.detach().cpu().float().numpy().astype(np.float64)
    prio = s * np.power(4.0, -bits.astype(np.float64))
    prio[bits >= max_bits] = -1.0

    while left > 0:
        i = int(np.argmax(prio))          # first index wins ties
        if prio[i] <= 0.0:
            break
        bits[i] += 1
        left -= 1
        prio[i] = -1.0 if bits[i] >= max_bits else s[i] * 4.0 ** (-float(bits[i]))
    return torch.from_numpy(bits)
