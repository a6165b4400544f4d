"""``BlockGTQKVManager``: the bit-packed KV cache with fused decode attention,
mirroring blockgtq/packed_kv_manager.py (constructor, methods, storage
attributes and shapes), with each layer step running as a handful of CUDA
launches covering every batch entry and KV head at once:

    rotate_q -> encode (K and V of the new token, written in place) -> decode -> combine

Extensions beyond the reference class (all off by default):
  * ``n_sink`` / ``recent_window`` / ``block_size``: the three-region policy of
    blockgtq/unaccelerated.py:163-244 on the packed path -- the first ``n_sink``
    tokens and a recent window stay in fp16 buffers, everything between is
    packed; the fp16 region is attended by its own kernel and merged by LSE.
  * ``token_range`` on :meth:`attend`: lets a rank attend a slice of the sequence
    and return (O, LSE) for a cross-GPU merge.
"""
from __future__ import annotations

import os

import math

import torch

from . import _lib
from .calib import packed_v_bytes
from .layer import (HD, LayerTables, buffer_attn, combine, combine_ranks, decode, decode_grid_size, decode_partition,
                    default_splits, encode, rotate_q,
                    step_prepare)
from .quantizer import BlockGTQQuantizer, build_batched_encode_args

__all__ = ["BlockGTQKVManager", "decode_step"]


class BlockGTQKVManager:
    def __init__(self, n_layers: int, n_q_heads: int, n_kv_heads: int, head_dim: int, max_seq_len: int,
                 batch_size: int = 1, k_avg_bits: float = 3.0, v_bits: int = 3, device="cuda",
                 n_sink: int = 0, recent_window: int = 0, block_size: int = 1,
                 min_bits: int = 1, max_bits: int = 8, rotation_threshold: int = 2,
                 use_cuda_graph: bool = None, k_mixed: bool = False, v_nibble: bool = False):
        if head_dim != HD:
            raise ValueError("head_dim must be 128")
        if n_kv_heads > 8 or n_q_heads // n_kv_heads > 8:
            raise ValueError("at most 8 KV heads per layer and 8 query heads per KV head are supported")
        self.n_layers, self.n_q, self.n_kv, self.hd = n_layers, n_q_heads, n_kv_heads, head_dim
        self.max_T, self.B = max_seq_len, batch_size
        self.k_avg_bits, self.v_bits = k_avg_bits, v_bits
        self.device = torch.device(device)
        self.gqa_ratio = n_q_heads // n_kv_heads
        self.scale = 1.0 / math.sqrt(head_dim)
        self._seq_len = 0                     # tokens appended so far (all regions)
        self._pos_dirty = True
        self._quant_opts = dict(min_bits=min_bits, max_bits=max_bits, rotation_threshold=rotation_threshold)
        self.quantizers = [[None] * n_kv_heads for _ in range(n_layers)]
        self._kernel_args = [[None] * n_kv_heads for _ in range(n_layers)]
        self._batched_args = [None] * n_layers
        self._layers = [None] * n_layers
        self._max_k_packed_bytes = 0
        self._max_n_groups = 0
        self._k_packed = self._k_norms = self._v_packed = self._v_norms = None
        self._part_dev = self._part_key = None
        # three-region policy
        self.n_sink, self.recent_window, self.block_size = int(n_sink), int(recent_window), int(block_size)
        self._buffered = self.n_sink > 0 or self.recent_window > 0
        self._buf_cap = self.n_sink + self.recent_window + self.block_size if self._buffered else 0
        self._k_buf = self._v_buf = None
        self.n_packed = 0                     # tokens in the packed region
        self._status = None
        # storage layout: bit-packed (this class in the reference) or the production cache's
        # nibble/raw "mixed" K rows with corrected norms and 4-bit V rows (production_cache.py:60-86)
        self.k_mixed, self.v_nibble = bool(k_mixed), bool(v_nibble)
        self.programmatic = True              # chain the step's kernels as programmatic dependent launches
        self._exchange = None                 # sequence sharding: see sharding.SequenceShard
        self._enc_flags = (_lib.ENC_K_MIXED if k_mixed else 0) | (_lib.ENC_V_NIBBLE if v_nibble else 0)
        self._dec_flags = (_lib.DEC_K_MIXED if k_mixed else 0) | (_lib.DEC_V_NIBBLE if v_nibble else 0)
        # single-token decode steps are captured once per layer and replayed (the reference graphs only
        # its T=1 encode, packed_kv_manager.py:182-257); needs the plain (unbuffered) cache
        # (with fp16 regions the captured step needs one-token blocks, the policy's default)
        graphable = (not self._buffered) or (self.block_size == 1 and self.recent_window >= 1)
        self._use_graph = graphable if use_cuda_graph is None else bool(use_cuda_graph)
        if self._use_graph and not graphable:
            raise ValueError("CUDA-graph replay with fp16 sink/recent buffers needs block_size == 1 and a window")
        self._graphs = [dict() for _ in range(n_layers)]      # per layer: {rope fused or not: CUDA graph}
        self._g_qkv = self._g_out = self._pos = None

    @property
    def seq_len(self) -> int:
        return self._seq_len

    @seq_len.setter
    def seq_len(self, value: int):
        self._seq_len = int(value)
        self._pos_dirty = True

    # -- calibration -----------------------------------------------------------------
    def calibrate(self, layer_idx: int, q_data: torch.Tensor, k_data: torch.Tensor):
        """Per-head tables for one layer; data (N, hd) shared or (n_kv, N, hd) per head
        (packed_kv_manager.py:85-114)."""
        if q_data.dim() == 2:
            q_data = q_data.unsqueeze(0).expand(self.n_kv, -1, -1)
            k_data = k_data.unsqueeze(0).expand(self.n_kv, -1, -1)
        for hi in range(self.n_kv):
            qz = BlockGTQQuantizer(head_dim=self.hd, avg_bits=self.k_avg_bits, device=self.device,
                                   **self._quant_opts)
            qz.calibrate(q_data[hi], k_data[hi])
            qz.init_v_quantizer(v_bits=self.v_bits, seed=42 + hi)
            self.quantizers[layer_idx][hi] = qz
            ka = qz.build_kernel_args()
            self._kernel_args[layer_idx][hi] = ka
            self._max_k_packed_bytes = max(self._max_k_packed_bytes, ka["total_packed_bytes"])
            self._max_n_groups = max(self._max_n_groups, qz._n_groups)
        self._batched_args[layer_idx] = build_batched_encode_args(self.quantizers[layer_idx], device=self.device)
        self._layers[layer_idx] = self._batched_args[layer_idx]["_layer"]

    def set_quantizers(self, layer_idx: int, quantizers: list):
        """Install already calibrated quantisers for a layer."""
        for hi, qz in enumerate(quantizers):
            self.quantizers[layer_idx][hi] = qz
            self._kernel_args[layer_idx][hi] = qz.build_kernel_args()
            self._max_k_packed_bytes = max(self._max_k_packed_bytes, qz._total_packed_bytes)
            self._max_n_groups = max(self._max_n_groups, qz._n_groups)
        self._batched_args[layer_idx] = build_batched_encode_args(quantizers, device=self.device)
        self._layers[layer_idx] = self._batched_args[layer_idx]["_layer"]

    def _ensure_storage(self):
        if self._k_packed is not None:
            return
        vpb = self.hd // 2 if self.v_nibble else packed_v_bytes(self.hd, self.v_bits)
        if self.k_mixed:
            self._max_k_packed_bytes = max(lt.max_mixed_bytes for lt in self._layers if lt is not None)
        # token capacity rounded up so 64-token tiles never leave the allocation
        cap = ((self.max_T + 63) // 64) * 64
        shape = (self.n_layers, self.B, self.n_kv, cap)
        dev = self.device
        self._k_packed = torch.zeros(*shape, self._max_k_packed_bytes, dtype=torch.uint8, device=dev)[:, :, :, :self.max_T]
        # norm rows of an even number of fp16 values: the decode kernel then reads a token's norms two per load
        self._k_norms = torch.zeros(*shape, self._norm_row_groups(), dtype=torch.float16, device=dev)[:, :, :, :self.max_T]
        self._v_packed = torch.zeros(*shape, vpb, dtype=torch.uint8, device=dev)[:, :, :, :self.max_T]
        self._v_norms = torch.zeros(*shape, dtype=torch.float16, device=dev)[:, :, :, :self.max_T]
        self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        # scratch reused by every layer step (stream ordered): rotated queries and split partials
        self._n_splits = default_splits(self.B, self.n_kv, self.max_T) if dev.type == "cuda" else 1
        # item ranges of the step's decode launches (one table for every layer: same shape, same length),
        # refreshed when the cache length changes the way the kernel cuts it into items
        self._part_key = None
        self._part_dev = None
        if dev.type == "cuda":
            self._part_cta = decode_grid_size(self.B, self.n_kv, self._n_splits)
            self._part_host = torch.empty(self._part_cta + 5, dtype=torch.int32)
            self._part_dev = torch.full((self._part_cta + 5,), -1, dtype=torch.int32, device=dev)
            for lt in self._layers:
                if lt is not None:
                    lt.set_partition(self._part_dev)
                    # the cache rows every decode launch of this manager reads (16-byte aligned slices: the
                    # token capacity is a multiple of 64)
                    lt.set_row_strides(self._max_k_packed_bytes, self._norm_row_groups(), vpb, 1, mixed=self.k_mixed)
                    # In a layer step the launch before the decode is the append (one new row + the rotated
                    # query), and the position is advanced between steps: the decode may start streaming early.
                    if not os.environ.get("BGTQ_DEC_NO_EARLY_FETCH"):
                        lt.set_early_fetch(1)
        self._prepare_decode_plans()
        self._q_rot = torch.empty(self.B, self.n_q, self.hd, dtype=torch.float16, device=dev)
        self._part_o = torch.empty(self.B, self.n_q, self._n_splits, self.hd, dtype=torch.float32, device=dev)
        self._part_lse = torch.empty(self.B, self.n_q, self._n_splits, dtype=torch.float32, device=dev)
        self._g_qkv = torch.zeros(self.n_layers, self.B, self.n_q + 2 * self.n_kv, 1, self.hd, dtype=torch.float16,
                                  device=dev)
        self._g_out = torch.zeros(self.n_layers, self.B, self.n_q, self.hd, dtype=torch.float16, device=dev)
        self._pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self._g_rope = torch.zeros(2, self.B, self.hd, dtype=torch.float16, device=dev)     # cos, sin of the step
        self._buf_o = torch.zeros(self.B, self.n_q, self.hd, dtype=torch.float32, device=dev)
        self._buf_lse = torch.zeros(self.B, self.n_q, dtype=torch.float32, device=dev)
        if self._buffered:
            self._k_buf = torch.zeros(self.n_layers, self.B, self.n_kv, self._buf_cap, self.hd,
                                      dtype=torch.float16, device=dev)
            self._v_buf = torch.zeros_like(self._k_buf)

    def _norm_row_groups(self) -> int:
        return self._max_n_groups + (self._max_n_groups & 1)

    def _prepare_decode_plans(self):
        """Build every layer's decode plan (table image + kernel specialised for the layer, a second or two of
        NVRTC each) up front and on several host threads, instead of one by one at the first decode step."""
        if self.device.type != "cuda":
            return
        from concurrent.futures import ThreadPoolExecutor
        layers = [lt for lt in self._layers if lt is not None]
        pd = _lib.DEC_PROGRAMMATIC
        flag_sets = {self._dec_flags, self._dec_flags | pd}
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:     # one layer per job: its flag
            list(ex.map(lambda lt: [lt.plan(f) for f in sorted(flag_sets)], layers))  # variants share one kernel

    # -- encode --------------------------------------------------------------------------
    def _encode_kv(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, t_start: int, t_end: int):
        """Encode (B, n_kv, S, hd) fp16 into packed rows [t_start, t_end): one launch, written in place
        (packed_kv_manager.py:138-180)."""
        self._ensure_storage()
        li = layer_idx
        assert k.shape[2] == t_end - t_start
        encode(self._layers[li], k.to(torch.float16), v.to(torch.float16), t_start,
               self._k_packed[li], self._k_norms[li], self._v_packed[li], self._v_norms[li], flags=self._enc_flags)

    def init_from_cache(self, past_key_value):
        """Bulk-encode an HF cache after prefill (packed_kv_manager.py:259-266).  Accepts the
        legacy ``key_cache``/``value_cache`` lists, the ``layers[i].keys/values`` layout of newer
        transformers, or a plain sequence of (k, v) pairs."""
        T = 0
        for li in range(self.n_layers):
            k, v = _layer_kv(past_key_value, li)
            T = k.shape[2]
            self._append_tokens(li, k, v, 0)
        self.seq_len = T

    # -- three-region bookkeeping ------------------------------------------------------------
    # Non-sink token i (i = position - n_sink) lives in ring slot n_sink + i % ring while it is
    # "recent"; once  (#non-sink tokens) - n_flushed >= block_size + recent_window  the oldest
    # block_size recent tokens are quantised into packed rows [n_flushed, n_flushed + block_size)
    # (flush rule of blockgtq/unaccelerated.py:226-233).  n_flushed depends only on the token count.
    def _flushed(self, n_non_sink: int) -> int:
        need = self.block_size + self.recent_window
        if n_non_sink < need:
            return 0
        return ((n_non_sink - need) // self.block_size + 1) * self.block_size

    def _region_sizes(self, seq_len: int, flushed: int = None):
        """(fp16 sink tokens, packed tokens, fp16 recent tokens) for ``seq_len`` appended tokens."""
        if not self._buffered:
            return 0, seq_len, 0
        sink = min(seq_len, self.n_sink)
        avail = max(0, seq_len - self.n_sink)
        if flushed is None:
            flushed = self._flushed(avail)
        return sink, flushed, avail - flushed

    def _ring_slots(self, lo: int, hi: int) -> torch.Tensor:
        ring = self._buf_cap - self.n_sink
        return torch.tensor([self.n_sink + i % ring for i in range(lo, hi)], dtype=torch.long, device=self.device)

    def _append_tokens(self, li: int, k: torch.Tensor, v: torch.Tensor, t: int, defer_flush: bool = False):
        """Append S tokens with absolute positions t .. t+S-1 to layer ``li``.

        With ``defer_flush`` the new tokens only enter the fp16 buffers (the caller attends first and
        then calls :meth:`_flush`, the order the reference's post-forward hook produces for a decode
        step).  Returns the (before, after) packed-region sizes."""
        S = k.shape[2]
        if not self._buffered:
            self._encode_kv(li, k, v, t, t + S)
            return t, t + S
        self._ensure_storage()
        k, v = k.to(torch.float16), v.to(torch.float16)
        kb, vb = self._k_buf[li], self._v_buf[li]
        ns = self.n_sink
        a0, a1 = max(0, t - ns), max(0, t + S - ns)
        f0, f1 = self._flushed(a0), self._flushed(a1)
        n_sink_new = max(0, min(ns, t + S) - t)
        if n_sink_new:
            kb[:, :, t:t + n_sink_new] = k[:, :, :n_sink_new]
            vb[:, :, t:t + n_sink_new] = v[:, :, :n_sink_new]
        if defer_flush:
            if a1 - f0 > self._buf_cap - ns:
                raise RuntimeError("recent ring overflow: flush before appending more tokens")
            lo = a0
        else:
            self._flush(li, f0, min(f1, a0))                   # tokens already resident in the ring
            lo = max(f1, a0)
            if f1 > a0:                                        # new tokens that go straight to packed rows
                s0, s1 = max(f0, a0) + ns - t, f1 + ns - t
                encode(self._layers[li], k[:, :, s0:s1], v[:, :, s0:s1], max(f0, a0), self._k_packed[li],
                       self._k_norms[li], self._v_packed[li], self._v_norms[li], flags=self._enc_flags)
        if a1 > lo:                                            # new tokens that stay recent
            slots = self._ring_slots(lo, a1)
            kb.index_copy_(2, slots, k[:, :, lo + ns - t:a1 + ns - t])
            vb.index_copy_(2, slots, v[:, :, lo + ns - t:a1 + ns - t])
        return f0, f1

    def _flush(self, li: int, f_lo: int, f_hi: int):
        """Quantise ring-resident non-sink tokens [f_lo, f_hi) into packed rows [f_lo, f_hi)."""
        if f_hi <= f_lo:
            return
        slots = self._ring_slots(f_lo, f_hi)
        encode(self._layers[li], self._k_buf[li].index_select(2, slots), self._v_buf[li].index_select(2, slots),
               f_lo, self._k_packed[li], self._k_norms[li], self._v_packed[li], self._v_norms[li],
               flags=self._enc_flags)

    # -- graph replay of one layer step ----------------------------------------------------------
    def static_qkv(self, layer_idx: int = 0) -> torch.Tensor:
        """(B, n_q + 2 n_kv, 1, hd) fp16 input buffer of layer ``layer_idx``'s captured step: rows [0, n_q)
        are the query heads, then the new K heads, then the new V heads.  Writing a step's inputs here (for
        instance as the output of a fused QKV projection or an H2D copy) and passing these views to
        :meth:`append_and_attend` skips the staging copies.  ``static_qkv_all()`` is the whole
        (n_layers, B, n_q + 2 n_kv, 1, hd) buffer."""
        self._ensure_storage()
        return self._g_qkv[layer_idx]

    def static_qkv_all(self) -> torch.Tensor:
        self._ensure_storage()
        return self._g_qkv

    def static_inputs(self, layer_idx: int = 0):
        b = self.static_qkv(layer_idx)
        return b[:, :self.n_q], b[:, self.n_q:self.n_q + self.n_kv], b[:, self.n_q + self.n_kv:]

    def static_outputs(self) -> torch.Tensor:
        """(n_layers, B, n_q, hd) fp16: where the captured layer steps leave their results."""
        self._ensure_storage()
        return self._g_out

    def _sync_pos(self):
        if self._pos_dirty:
            self._pos.fill_(self._seq_len)
            self._pos_dirty = False
        self._refresh_partition()

    def _step_decode_pos_add(self) -> int:
        """What the step's decode adds to the device-side position to get its live token count."""
        if self._buffered:
            return -(self.n_sink + self.recent_window)
        return 1 if (self._exchange is None or self._exchange.is_owner) else 0

    def _refresh_partition(self):
        """Keep the decode launches' item-range table in step with the cache length.  The table depends on the
        length only through the number of items per (batch, head) pair and their size, which change every few
        hundred tokens; a table made for another length is ignored by the kernel, so this is about balance
        only."""
        if self._part_dev is None or torch.cuda.is_current_stream_capturing():
            return      # (inside a caller's capture the table is refreshed by increment_seq_len, outside it)
        n_tok = max(0, min(self.max_T, self._seq_len + self._step_decode_pos_add()))
        units = (n_tok + 31) // 32
        c_units = max(1, -(-units // self._n_splits))
        key = (-(-units // c_units), c_units)
        if key == self._part_key:
            return
        self._part_key = key
        decode_partition(self.B, self.n_kv, n_tok, self._n_splits, self._part_cta, out=self._part_host)
        self._part_dev.copy_(self._part_host)      # stream ordered: lands before the next step's launches

    def _layer_step(self, li: int, rope: bool = False):
        """rotate_q -> append K,V at *pos -> decode over [0, *pos + 1) -> combine, all on static buffers."""
        lt = self._layers[li]
        gq, gk, gv = self.static_inputs(li)
        baked = all(self.quantizers[li][h]._q_perm_baked for h in range(self.n_kv))
        # the three kernels are chained as programmatic dependents: each sets up its static tables while
        # the one before it drains, and waits on the device before touching the step's data
        pd = self.programmatic
        ex = self._exchange
        q_rot = self._q_rot
        if baked:                   # queries arrive in the packed-K basis already: stage them without allocating
            self._q_rot.copy_(gq[:, :, 0])
        if self._buffered:          # three regions, everything derived from the device-side token count
            ns, win = self.n_sink, self.recent_window
            step_prepare(lt, None if baked else gq, gk, gv, 0, self._k_packed[li], self._k_norms[li],
                         self._v_packed[li], self._v_norms[li], q_rot=self._q_rot, pos_dev=self._pos,
                         flags=self._enc_flags | (_lib.ENC_PROGRAMMATIC if pd else 0), status=self._status,
                         ring=(self._k_buf[li], self._v_buf[li], ns, win))
            decode(lt, q_rot, self._k_packed[li], self._k_norms[li], self._v_packed[li], self._v_norms[li],
                   0, self.max_T, n_splits=self._n_splits, scale=self.scale, status=self._status,
                   part_o=self._part_o, part_lse=self._part_lse, pos_dev=self._pos, pos_add=-(ns + win),
                   flags=self._dec_flags | (_lib.DEC_PROGRAMMATIC if pd else 0))
            buffer_attn(gq, self._k_buf[li], self._v_buf[li], self.n_kv, self.scale, sink_cap=ns, ring_size=win + 1,
                        pos_dev=self._pos, out=(self._buf_o, self._buf_lse))
            combine(self._part_o, self._part_lse, self.n_kv, v_rot=lt.v_rot, buf_o=self._buf_o, buf_lse=self._buf_lse,
                    out=self._g_out[li], programmatic=pd)
            return
        if ex is None or ex.is_owner:
            step_prepare(lt, None if baked else gq, gk, gv, 0, self._k_packed[li], self._k_norms[li],
                         self._v_packed[li], self._v_norms[li], q_rot=self._q_rot, pos_dev=self._pos,
                         flags=self._enc_flags | (_lib.ENC_PROGRAMMATIC if pd else 0), status=self._status,
                         rope=(self._g_rope[0], self._g_rope[1]) if rope else None)
        elif not baked:                           # this rank does not hold the tail: nothing to append
            rotate_q(lt, gq[:, :, 0], out=self._q_rot)
        decode(lt, q_rot, self._k_packed[li], self._k_norms[li], self._v_packed[li], self._v_norms[li],
               0, self.max_T, n_splits=self._n_splits, scale=self.scale, status=self._status,
               part_o=self._part_o, part_lse=self._part_lse, pos_dev=self._pos,
               pos_add=1 if (ex is None or ex.is_owner) else 0,
               flags=self._dec_flags | (_lib.DEC_PROGRAMMATIC if pd else 0))
        if ex is None:
            combine(self._part_o, self._part_lse, self.n_kv, v_rot=lt.v_rot, out=self._g_out[li], programmatic=pd)
        elif ex.transport == "p2p":     # combine + peer stores in one launch, then the bounded wait + merge
            ex.combine_publish(self._part_o, self._part_lse, self.n_kv, lt.v_rot, programmatic=pd)
            ex.exchange_and_merge(self._g_out[li])
        else:       # local result straight into the message, one all-gather, merge of the messages
            combine(self._part_o, self._part_lse, self.n_kv, v_rot=lt.v_rot, out=self._g_out[li], programmatic=pd,
                    o32_out=ex.msg_o, lse_out=ex.msg_lse)
            ex.exchange_and_merge(self._g_out[li])

    def layer_step(self, layer_idx: int, rope: bool = False):
        """Launch one layer's decode step (append the token in ``static_inputs(layer_idx)`` at the current
        position, attend, leave the result in ``static_outputs()[layer_idx]``) as plain kernel launches on the
        current stream: no allocation, no synchronisation, position read on the device.  This is the form to
        call inside a caller's own CUDA-graph capture of a whole decode step (a serving engine capturing its
        model forward); :meth:`append_and_attend` wraps the same launches in one graph per layer.  Call
        :meth:`increment_seq_len` once per step, outside the captured region or after the replay.

        The host-side length is checked here; a captured step replayed past the capacity is caught on the
        device instead (the append kernel stores nothing and :meth:`check_status` raises)."""
        self._ensure_storage()
        if self._seq_len + 1 > self.max_T and (self._exchange is None or self._exchange.is_owner):
            raise ValueError("cache overflow")
        self._sync_pos()
        self._layer_step(layer_idx, rope)

    def _replay_layer(self, li: int, q, k_new, v_new, rope=None) -> torch.Tensor:
        self._ensure_storage()
        if self._seq_len + 1 > self.max_T:
            raise ValueError("cache overflow")
        self._sync_pos()
        gq, gk, gv = self.static_inputs(li)
        if q.data_ptr() != gq.data_ptr():
            gq.copy_(q.reshape(gq.shape))
        if k_new.data_ptr() != gk.data_ptr():
            gk.copy_(k_new)
        if v_new.data_ptr() != gv.data_ptr():
            gv.copy_(v_new)
        use_rope = rope is not None
        if use_rope:
            self._g_rope[0].copy_(rope[0].reshape(self.B, self.hd))
            self._g_rope[1].copy_(rope[1].reshape(self.B, self.hd))
        g = self._graphs[li].get(use_rope)
        if g is None:
            self._layer_step(li, use_rope)            # eager once: sets kernel attributes, validates shapes
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._layer_step(li, use_rope)
            self._graphs[li][use_rope] = g
        else:
            g.replay()
            _lib.count_launch(4 if self._buffered else
                              ((4 if self._exchange.transport == "p2p" else 5) if self._exchange else 3))
        return self._g_out[li]

    # -- decode ----------------------------------------------------------------------------
    @torch.no_grad()
    def append_and_attend(self, layer_idx: int, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                          n_splits: int = None, rope=None) -> torch.Tensor:
        """Quantise and append (B, n_kv, S, hd) K/V, then attend the (B, n_q, 1, hd) query over the
        whole cache.  Returns (B, n_q, 1, hd) fp16 (packed_kv_manager.py:268-348).
        ``rope=(cos, sin)`` (fp16, (B, [1,] hd), single-token steps): q and k_new are pre-RoPE and the append
        kernel applies the rotary embedding itself (an extension; the reference's callers rotate first)."""
        t, S = self.seq_len, k_new.shape[2]
        if self._use_graph and S == 1 and n_splits is None and q.is_cuda:
            return self._replay_layer(layer_idx, q, k_new, v_new, rope).unsqueeze(2)
        if rope is not None:
            raise NotImplementedError("fused RoPE is available on the single-token graph path only")
        defer = self._buffered and S == 1
        f0, f1 = self._append_tokens(layer_idx, k_new, v_new, t, defer_flush=defer)
        out, _, _ = self.attend(layer_idx, q, t + S, n_splits=n_splits, flushed=f0 if defer else None)
        if defer:
            self._flush(layer_idx, f0, f1)
        return out.unsqueeze(2)

    @torch.no_grad()
    def attend(self, layer_idx: int, q: torch.Tensor, seq_len: int = None, *, n_splits: int = None,
               token_range=None, want_partial: bool = False, flushed: int = None, with_buffers: bool = True):
        """Attention of q (B, n_q, [1,] hd) over the first ``seq_len`` cached tokens.

        ``token_range=(lo, hi)`` restricts the packed region to rows [lo, hi) and ``with_buffers``
        says whether this call also covers the fp16 region (sequence sharding: one rank does).
        Returns (out fp16 (B, n_q, hd), out_f32 | None, lse | None); the last two when ``want_partial``."""
        li = layer_idx
        lt: LayerTables = self._layers[li]
        seq_len = self.seq_len if seq_len is None else seq_len
        n_sink_tok, n_packed, n_recent = self._region_sizes(seq_len, flushed)
        if q.dim() == 4:
            q = q[:, :, 0]
        q = q.to(torch.float16)
        lo, hi = (0, n_packed) if token_range is None else token_range
        lo = max(0, min(lo, n_packed))
        hi = max(lo, min(hi, n_packed))
        baked = all(self.quantizers[li][h]._q_perm_baked for h in range(self.n_kv))
        q_rot = q.contiguous() if baked else rotate_q(lt, q)
        part_o, part_lse = decode(lt, q_rot, self._k_packed[li], self._k_norms[li], self._v_packed[li],
                                  self._v_norms[li], lo, hi, n_splits=n_splits, scale=self.scale,
                                  status=self._status, flags=self._dec_flags)
        buf_o = buf_lse = None
        if self._buffered and with_buffers:
            buf_o, buf_lse = self._buffer_partial(li, q, n_sink_tok, n_packed, n_recent)
        return combine(part_o, part_lse, self.n_kv, v_rot=lt.v_rot, buf_o=buf_o, buf_lse=buf_lse,
                       want_f32=want_partial, want_lse=want_partial)

    def _buffer_partial(self, li, q, n_sink_tok, n_packed, n_recent):
        """(O, LSE) of the fp16 region: sink slots [0, n_sink_tok) + ring slots of the recent tokens."""
        ring = self._buf_cap - self.n_sink
        return buffer_attn(q, self._k_buf[li], self._v_buf[li], self.n_kv, self.scale,
                           n_sink_tokens=n_sink_tok, n_ring_tokens=n_recent, sink_cap=self.n_sink,
                           ring_first=n_packed % ring, ring_size=ring)

    def increment_seq_len(self, by: int = 1):
        """Call after all layers processed the new token(s) (packed_kv_manager.py:350-352)."""
        if self._exchange is not None and not self._exchange.is_owner:
            return                                # appended tokens live on the owner rank
        self._seq_len += by
        if self._pos is not None and not self._pos_dirty:
            self._pos.add_(by)
        _, self.n_packed, _ = self._region_sizes(self._seq_len)
        if self._k_packed is not None:
            self._refresh_partition()

    def release_graphs(self):
        """Drop the captured per-layer CUDA graphs (they are re-captured on the next step).  Call this before
        destroying a process group whose collectives the graphs captured (sequence sharding)."""
        torch.cuda.synchronize(self.device)
        self._graphs = [dict() for _ in range(self.n_layers)]

    def check_status(self):
        """Synchronise and raise if a kernel reported a timed-out wait (1: the outputs of that launch are
        invalid) or an append past the end of the cache (2: nothing was stored).  Covers the decode / append
        status word and the bulk tcgen05 encoder's own sticky status."""
        if self._status is not None and int(self._status.item()) != 0:
            code = int(self._status.item())
            what = {1: "a bounded wait inside a kernel gave up", 2: "an append past the end of the cache was refused"}
            raise RuntimeError(f"kernel status {code}: {what.get(code, 'unknown')}")
        if self.device.type == "cuda" and _lib.lib().bgtq_encode_tcgen05_status() != 0:
            raise RuntimeError("the tcgen05 bulk encoder reported a timed-out wait: the rows of that launch are incomplete")
        if self.device.type == "cuda" and _lib.lib().bgtq_prefill_tcgen05_status() != 0:
            raise RuntimeError("the tcgen05 prefill attention reported a timed-out wait: the output of that launch is invalid")

    def bake_q_permutations(self, model, n_kv_heads: int, n_q_heads: int):
        """Bake each head's permutation + rotation into q_proj (packed_kv_manager.py:354-373)."""
        layers = _get_model_layers(model)
        for li in range(self.n_layers):
            attn = layers[li].self_attn
            for hi in range(self.n_kv):
                self.quantizers[li][hi].bake_permutation_into_qproj(
                    attn.q_proj.weight.data, kv_head_idx=hi, n_kv_heads=n_kv_heads, n_q_heads=n_q_heads,
                    q_proj_bias=getattr(attn.q_proj, "bias", None))

    def cache_memory_bytes(self) -> int:
        """Compressed cache bytes for the current length, padding included (packed_kv_manager.py:375-382)."""
        _, T, n_rec = self._region_sizes(self.seq_len)
        per_tok = self._max_k_packed_bytes + packed_v_bytes(self.hd, self.v_bits) + self._norm_row_groups() * 2 + 2
        packed = per_tok * T * self.n_kv * self.B * self.n_layers
        fp16 = (min(self.seq_len, self.n_sink) + n_rec) * self.hd * 2 * 2 * self.n_kv * self.B * self.n_layers
        return packed + fp16

    def live_bytes_per_step(self) -> int:
        """Bytes one decode step must read: per head its own packed K size and group count
        (not the padded strides), V bytes, norms, plus the fp16 buffer tokens."""
        sink, T, n_rec = self._region_sizes(self.seq_len)
        vpb = packed_v_bytes(self.hd, self.v_bits)
        tot = 0
        for li in range(self.n_layers):
            for hi in range(self.n_kv):
                qz = self.quantizers[li][hi]
                tot += T * (qz._total_packed_bytes + 2 * qz._n_groups + vpb + 2)
        tot *= self.B
        tot += (sink + n_rec) * self.hd * 2 * 2 * self.n_kv * self.B * self.n_layers
        return tot

    def fp16_cache_bytes(self) -> int:
        return self.n_layers * self.B * self.n_kv * self.seq_len * self.hd * 2 * 2


def _layer_kv(pkv, li):
    if hasattr(pkv, "key_cache"):
        return pkv.key_cache[li], pkv.value_cache[li]
    if hasattr(pkv, "layers"):
        lay = pkv.layers[li]
        return lay.keys, lay.values
    return pkv[li][0], pkv[li][1]


def _get_model_layers(model):
    if hasattr(model, "model") and hasattr(model.model, "layers"):
        return list(model.model.layers)
    raise ValueError("Cannot find model layers - expected model.model.layers")


def decode_step(model, input_ids, position_ids, kv_manager: BlockGTQKVManager):
    """One decode step of an HF Llama-style model through the packed cache
    (packed_kv_manager.py:401-453).  input_ids/position_ids (B, 1) -> logits (B, 1, vocab)."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    hidden = model.model.embed_tokens(input_ids)
    n_q, n_kv, hd = kv_manager.n_q, kv_manager.n_kv, kv_manager.hd
    for li, layer in enumerate(_get_model_layers(model)):
        resid = hidden
        hidden = layer.input_layernorm(hidden)
        attn = layer.self_attn
        B, S, _ = hidden.shape
        q = attn.q_proj(hidden).view(B, S, n_q, hd).transpose(1, 2)
        k = attn.k_proj(hidden).view(B, S, n_kv, hd).transpose(1, 2)
        v = attn.v_proj(hidden).view(B, S, n_kv, hd).transpose(1, 2)
        rope = getattr(attn, "rotary_emb", None) or model.model.rotary_emb
        cos, sin = rope(v, position_ids)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        out = kv_manager.append_and_attend(li, q, k, v)
        hidden = resid + attn.o_proj(out.transpose(1, 2).reshape(B, S, n_q * hd).to(hidden.dtype))
        resid = hidden
        hidden = resid + layer.mlp(layer.post_attention_layernorm(hidden))
    kv_manager.increment_seq_len()
    return model.lm_head(model.model.norm(hidden))
