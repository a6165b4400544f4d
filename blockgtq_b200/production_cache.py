"""``BlockGTQProductionCache``: the reference's production decode cache (blockgtq/production_cache.py:34-283)
on the CUDA library.  K rows use the nibble/raw "mixed" layout with corrected norms, V rows 4-bit nibbles
(or the bit-packed layouts with ``k_nibble=False`` / ``v_nibble=False``).  Calibration is owned by the
caller, as in the reference: pass the per-(layer, head) quantizers, the per-layer batched args and the
per-head kernel args.  A batch dimension other than 1 is an extension (``batch_size``)."""
from __future__ import annotations

import math

import torch

from .packed_kv_manager import BlockGTQKVManager

__all__ = ["BlockGTQProductionCache"]


class BlockGTQProductionCache:
    def __init__(self, quantizers, batched_args, kernel_args, n_layers, nkv, nq, hd, max_T, v_bits=3,
                 k_nibble=True, v_nibble=True, device="cuda", batch_size=1, use_cuda_graph=None):
        self.quantizers, self.batched_args, self.kernel_args = quantizers, batched_args, kernel_args
        self.n_layers, self.nkv, self.nq, self.hd = n_layers, nkv, nq, hd
        self.gqa = nq // nkv
        self.v_bits, self.k_nibble, self.v_nibble = v_bits, k_nibble, v_nibble
        self.device = device
        self.scale = 1.0 / math.sqrt(hd)
        q0 = quantizers[0][0]
        self._mgr = BlockGTQKVManager(n_layers, nq, nkv, hd, max_T, batch_size=batch_size, k_avg_bits=q0.avg_bits,
                                      v_bits=v_bits, device=device, k_mixed=k_nibble, v_nibble=v_nibble,
                                      use_cuda_graph=use_cuda_graph)
        for li in range(n_layers):
            m = self._mgr
            for hi, qz in enumerate(quantizers[li]):
                m.quantizers[li][hi] = qz
                m._kernel_args[li][hi] = kernel_args[li][hi]
                m._max_k_packed_bytes = max(m._max_k_packed_bytes, qz._total_packed_bytes)
                m._max_n_groups = max(m._max_n_groups, qz._n_groups)
            m._batched_args[li] = batched_args[li]
            m._layers[li] = batched_args[li]["_layer"]
        self.max_ng = self._mgr._max_n_groups
        self.k_bytes_per_tok = (max(ba["max_mixed_bytes"] for ba in batched_args) if k_nibble
                                else max(ba["max_tpb"] for ba in batched_args))
        self.vpb = hd // 2 if v_nibble else batched_args[0]["v_packed_bytes"]
        self._mgr._ensure_storage()

    # storage tensors, (n_layers, B, nkv, max_T, bytes) as in production_cache.py:69-86
    k_packed = property(lambda self: self._mgr._k_packed)
    k_norms = property(lambda self: self._mgr._k_norms)
    v_packed = property(lambda self: self._mgr._v_packed)
    v_norms = property(lambda self: self._mgr._v_norms)

    @property
    def seq_len(self):
        return self._mgr.seq_len

    @seq_len.setter
    def seq_len(self, v):
        self._mgr.seq_len = v

    def _encode_batched(self, layer_idx, k, v, t_pos):
        """Multi-token encode into rows [t_pos, t_pos + S) (production_cache.py:174-201)."""
        self._mgr._encode_kv(layer_idx, k, v, t_pos, t_pos + k.shape[2])

    def _encode_graphed(self, layer_idx, k, v, t_pos):
        self._mgr._encode_kv(layer_idx, k, v, t_pos, t_pos + 1)

    @torch.no_grad()
    def encode_and_attend(self, layer_idx, q, k, v, rope=None):
        """Encode the new (B, n_kv, S, hd) K/V and attend the (B, n_q, 1, hd) query: -> (B, n_q, 1, hd) fp16
        (production_cache.py:207-264).  ``rope=(cos, sin)``: q and k are pre-RoPE, see
        :meth:`BlockGTQKVManager.append_and_attend`."""
        return self._mgr.append_and_attend(layer_idx, q, k, v, rope=rope)

    @property
    def can_fuse_rope(self) -> bool:
        """Single-token steps can take pre-RoPE q/k (graph path, rotations not baked into q_proj)."""
        m = self._mgr
        return m._use_graph and not any(qz._q_perm_baked for row in m.quantizers for qz in row if qz is not None)

    def increment_seq_len(self, by=1):
        self._mgr.increment_seq_len(by)

    def static_qkv(self, layer_idx=0):
        return self._mgr.static_qkv(layer_idx)

    def static_inputs(self, layer_idx=0):
        return self._mgr.static_inputs(layer_idx)

    def cache_memory_bytes(self) -> int:
        T = self.seq_len
        per_tok = self.k_bytes_per_tok + self.vpb + self.max_ng * 2 + 2
        return per_tok * T * self.nkv * self.n_layers * self._mgr.B

    def fp16_cache_bytes(self) -> int:
        return self.n_layers * self.nkv * self.seq_len * self.hd * 2 * 2 * self._mgr.B
