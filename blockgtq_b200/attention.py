"""Operator-level decode attention with the reference's signature
(blockgtq/kernels/fused_packed_attention.py:1541-1861).

The reference specialises its Triton kernel on one head's segment tuple and is
called once per KV head.  This wrapper accepts the same arguments, turns the
segment tuple / codebook / V LUT into a head descriptor (cached) and runs the
CUDA decode + combine kernels.  Callers that hold a whole layer should use
:mod:`blockgtq_b200.layer` directly (one launch for all heads).
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from .layer import HD, combine, decode, make_decode_plan

_cache = {}


class _AdHocLayer:
    """Minimal stand-in for LayerTables built from operator arguments."""

    def __init__(self, segments, codebook_flat, v_lut, v_bits, n_kv, nopack, device):
        self.n_kv = n_kv
        self.device = device
        self.desc_host = (_lib.HeadDesc * n_kv)()
        cb = codebook_flat.detach().to(torch.float16).cpu().view(torch.int16).numpy().astype(np.uint16)
        vl = v_lut.detach().to(torch.float16).cpu().view(torch.int16).numpy().astype(np.uint16)
        for h in range(n_kv):
            d = self.desc_host[h]
            d.n_seg = len(segments)
            d.v_bits = v_bits
            d.nopack_start, d.nopack_len = nopack
            for s, (bw, start, length, pack_off, lut_off, _ni) in enumerate(segments):
                d.seg_bw[s], d.seg_start[s], d.seg_len[s] = bw, start, length
                d.seg_pack_off[s], d.seg_lut_off[s] = pack_off, lut_off
            for i, x in enumerate(cb[:512]):
                d.codebook[i] = int(x)
            for i, x in enumerate(vl[:16]):
                d.v_lut[i] = int(x)
        self.desc_dev = torch.from_numpy(np.frombuffer(self.desc_host, dtype=np.uint8).copy()).to(device)
        self._plans = {}

    def plan(self, flags=0):
        p = self._plans.get(flags)
        if p is None:
            p = make_decode_plan(self.desc_host, self.n_kv, flags, self.device)
            self._plans[flags] = p
        return p[0]


def _layer_for(segments, codebook_flat, v_lut, v_bits, n_kv, device):
    segs = tuple(tuple(int(x) for x in s) for s in segments)
    key = (segs, codebook_flat.data_ptr(), v_lut.data_ptr(), int(v_bits), n_kv, str(device))
    lt = _cache.get(key)
    if lt is None:
        raw = [s for s in segs if s[0] > 4 and s[2] > 0]
        nopack = (min(s[1] for s in raw), sum(s[2] for s in raw)) if raw else (HD, 0)
        lt = _AdHocLayer(segs, codebook_flat, v_lut, v_bits, n_kv, nopack, device)
        if len(_cache) > 4096:
            _cache.clear()
        _cache[key] = lt
    return lt


@torch.no_grad()
def fused_blockgtq_decode_attention(
        q, k_packed, k_norms, codebook_flat, lut_offset, norm_group, segments,
        v_codes, v_norms, v_lut, scale=None, block_t=64, block_m=16, t_splits=32,
        v_skip_thresh=0.0, v_norm_scale=None, onebit_fast="auto", q_pack_perm=None,
        v_bits=0, v_rotation=None, k_nibble=False, v_nibble=False, v_paired_2b=False,
        k_paired_2b=False, k_paired_4b=False, k_paired_8b=False, k_paired_1b=False,
        return_lse=False):
    """q (B, n_q, 1, 128) fp16 (already rotated for packed K) x packed cache -> (B, n_q, 1, 128) fp16.

    ``t_splits`` is honoured as the number of token splits.  Tile-shape and fast-path
    switches of the Triton kernel (``block_t``, ``block_m``, ``onebit_fast``, ``*_paired_*``,
    ``v_skip_thresh``) select between mathematically equal code paths there and are accepted and
    ignored here.  ``lut_offset`` / ``norm_group`` are unused by the reference kernel as well.
    Raw (unpacked) V codes (``v_bits=0`` without ``v_nibble``) and int4 V norms are not supported."""
    assert q.dim() == 4 and q.shape[2] == 1
    assert len(segments) <= 8
    if v_nibble:
        vb_codebook = int(round(math.log2(v_lut.numel())))
    elif v_bits and v_bits > 0:
        vb_codebook = int(v_bits)
    else:
        raise NotImplementedError("raw uint8 V codes are not supported; pack V (v_bits=1..4) or use v_nibble")
    if v_norms.dtype != torch.float16:
        raise NotImplementedError("int4 V norms are not supported")
    B, n_q, _, D = q.shape
    n_kv, T = k_packed.shape[1], k_packed.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q_pack_perm is not None:
        q = q[:, :, :, q_pack_perm]
    q2 = q.reshape(B, n_q, D).to(torch.float16).contiguous()
    if v_norms.dim() == 4:
        v_norms = v_norms[..., 0]
    lt = _layer_for(segments, codebook_flat, v_lut, vb_codebook, n_kv, q.device)
    flags = (_lib.DEC_K_MIXED if k_nibble else 0) | (_lib.DEC_V_NIBBLE if v_nibble else 0)
    part_o, part_lse = decode(lt, q2, k_packed, k_norms.to(torch.float16), v_codes, v_norms, 0, T,
                              n_splits=max(1, int(t_splits)), scale=scale, flags=flags)
    rot = None
    if v_rotation is not None:
        rot = v_rotation.to(torch.float32).contiguous()
        rot = rot.unsqueeze(0).expand(n_kv, -1, -1).contiguous() if rot.dim() == 2 else rot
    out, _o32, lse = combine(part_o, part_lse, n_kv, v_rot=rot, want_lse=return_lse)
    if return_lse:
        return out.unsqueeze(2), lse
    return out.unsqueeze(2)


@torch.no_grad()
def fused_blockgtq_prefill_attention(
        q, k_packed, k_norms, codebook_flat, lut_offset, norm_group, segments,
        v_codes, v_norms, v_lut, scale=None, block_q=64, block_t=64, v_skip_thresh=0.0,
        v_norm_scale=None, v_bits=0, v_rotation=None, is_causal=True, q_pos_offset=0,
        k_nibble=False, v_nibble=False, min_seg_for_dot=16):
    """q (B, n_q, S_q, 128) fp16 (already rotated for packed K) x packed cache -> (B, n_q, S_q, 128) fp16
    (blockgtq/kernels/fused_packed_attention.py:2597-2760).  Query i has position ``q_pos_offset + i``
    and, when ``is_causal``, attends cache tokens up to and including it.  ``block_q`` / ``block_t`` /
    ``v_skip_thresh`` / ``min_seg_for_dot`` select tile shapes and equal-valued code paths in the
    Triton kernel and are accepted and ignored; raw V codes and int4 V norms are not supported."""
    from .layer import prefill_attention
    assert q.dim() == 4 and len(segments) <= 8
    if v_nibble:
        vb_codebook = int(round(math.log2(v_lut.numel())))
    elif v_bits and v_bits > 0:
        vb_codebook = int(v_bits)
    else:
        raise NotImplementedError("raw uint8 V codes are not supported; pack V (v_bits=1..4) or use v_nibble")
    if v_norms.dtype != torch.float16:
        raise NotImplementedError("int4 V norms are not supported")
    n_kv, T = k_packed.shape[1], k_packed.shape[2]
    if v_norms.dim() == 4:
        v_norms = v_norms[..., 0]
    lt = _layer_for(segments, codebook_flat, v_lut, vb_codebook, n_kv, q.device)
    flags = (_lib.DEC_K_MIXED if k_nibble else 0) | (_lib.DEC_V_NIBBLE if v_nibble else 0)
    rot = None
    if v_rotation is not None:
        rot = v_rotation.to(torch.float32).contiguous()
        rot = rot.unsqueeze(0).expand(n_kv, -1, -1).contiguous() if rot.dim() == 2 else rot
    q16 = q.to(torch.float16)
    if q16.stride(3) != 1:
        q16 = q16.contiguous()
    return prefill_attention(lt, q16, k_packed, k_norms.to(torch.float16), v_codes, v_norms, T,
                             q_pos_offset=int(q_pos_offset), causal=bool(is_causal), scale=scale, flags=flags,
                             v_rot=rot)
