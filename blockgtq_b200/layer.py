"""Per-layer device tables and thin operator wrappers over the C ABI.

A :class:`LayerTables` owns, for the KV heads of one layer, the uploaded array
of ``BgtqHeadDesc`` records, the rotation matrices and the cached decode plans.
The functions below take torch tensors, pass raw pointers and strides to
``libbgtq.so`` and return torch tensors; they enqueue on the current stream
and never synchronise.
"""
from __future__ import annotations

import os

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from .calib import KHeadTables, VHeadTables, packed_v_bytes

HD = _lib.HD


def _fill_desc(d: _lib.HeadDesc, kt: KHeadTables, vt: VHeadTables):
    if kt.head_dim != HD:
        raise ValueError("the CUDA kernels support head_dim 128 only")
    pm = kt.pack_meta
    d.n_seg = kt.n_groups
    d.k_row_bytes = kt.total_packed_bytes
    d.v_bits = vt.bits
    d.v_row_bytes = vt.packed_bytes
    d.nopack_start, d.nopack_len = pm["nopack_start"], pm["nopack_len"]
    d.k_mixed_bytes = pm["nopack_start"] // 2 + pm["nopack_len"]
    cb16 = kt.codebook_flat.view(torch.int16).numpy().astype(np.uint16)
    for s, (bw, start, length, pack_off, lut_off, _ni) in enumerate(kt.segments):
        d.seg_bw[s], d.seg_start[s], d.seg_len[s] = bw, start, length
        d.seg_pack_off[s], d.seg_lut_off[s] = pack_off, lut_off
        d.lut_off[s] = float(kt.lut_offsets[start])
        d.lut_inv[s] = float(kt.lut_inv_scales[start])
        cents = kt.pos_centroids[start, :1 << bw]
        for i in range(1 << bw):
            d.codebook[lut_off + i] = int(cb16[lut_off + i])
            d.k_cents[lut_off + i] = float(cents[i])
        row = kt.code_lut[s].numpy()
        C.memmove(d.code_lut[s], row.ctypes.data, _lib.N_BINS)
    nc = 1 << vt.bits
    vl16 = vt.lut_f16.view(torch.int16).numpy().astype(np.uint16)
    for i in range(16):
        d.v_cents[i] = float(vt.centroids[i]) if i < nc else 0.0
        d.v_bounds[i] = float(vt.boundaries[i]) if i < nc - 1 else float("inf")
        d.v_lut[i] = int(vl16[i]) if i < nc else 0
    hp = kt.head_perm.numpy().astype(np.uint8)
    go = kt.group_of.numpy().astype(np.uint8)
    C.memmove(d.head_perm, hp.ctypes.data, HD)
    C.memmove(d.group_of, go.ctypes.data, HD)


def make_decode_plan(desc_host, n_kv: int, flags: int, device, row_strides=None):
    """Decode plan of a layer's KV heads with its lookup-table image uploaded to ``device``.
    Returns (plan, image tensor); the caller keeps the image alive as long as the plan is used.
    ``row_strides`` = (packed-K bytes, K-norm values, packed-V bytes, V-norm values) per token fixes them in
    the specialised kernel (launches with other strides or unaligned slices then run the general kernel)."""
    L = _lib.lib()
    p = _lib.DecodePlan()
    _lib.check(L.bgtq_decode_plan(C.byref(desc_host), n_kv, flags, C.byref(p)), "bgtq_decode_plan")
    n = int(L.bgtq_decode_image_bytes(C.byref(p)))
    if n <= 0:
        raise RuntimeError("bgtq_decode_image_bytes failed")
    host = np.zeros(n, dtype=np.uint8)
    _lib.check(L.bgtq_decode_build_image(C.byref(p), C.byref(desc_host), host.ctypes.data, n),
               "bgtq_decode_build_image")
    image = torch.from_numpy(host).to(device)
    _lib.check(L.bgtq_decode_plan_set_image(C.byref(p), image.data_ptr()), "bgtq_decode_plan_set_image")
    if not (flags & _lib.DEC_GENERIC) and not os.environ.get("BGTQ_DEC_NO_JIT") and torch.device(device).type == "cuda":
        if row_strides is not None:
            _lib.check(L.bgtq_decode_plan_set_row_strides(C.byref(p), *[int(x) for x in row_strides]),
                       "bgtq_decode_plan_set_row_strides")
        _specialize(p)
    return p, image


_jit_warned = False


def _specialize(plan):
    """Compile (NVRTC) and attach the decode kernel specialised for the plan's heads.  Without NVRTC the
    plan keeps using the general kernel; a compile or load failure is an error."""
    global _jit_warned
    log = C.create_string_buffer(1 << 16)
    rc = _lib.lib().bgtq_decode_plan_specialize(C.byref(plan), 0, log, len(log))
    if rc == -2:
        if not _jit_warned:
            import warnings
            warnings.warn("NVRTC not found: the packed decode runs its general kernel (" + log.value.decode() + ")")
            _jit_warned = True
        return
    if rc != 0:
        raise RuntimeError("specialising the decode kernel failed:\n" + log.value.decode(errors="replace"))


class LayerTables:
    """Device-resident static tables for the KV heads of one layer."""

    def __init__(self, k_tables, v_tables, device):
        self.n_kv = len(k_tables)
        self.device = torch.device(device)
        self.k_tables, self.v_tables = list(k_tables), list(v_tables)
        self.desc_host = (_lib.HeadDesc * self.n_kv)()
        for h in range(self.n_kv):
            _fill_desc(self.desc_host[h], k_tables[h], v_tables[h])
        raw = np.frombuffer(self.desc_host, dtype=np.uint8).copy()
        self.desc_dev = torch.from_numpy(raw).to(self.device)
        self.rot_k = torch.stack([t.block_rot.T.contiguous() for t in k_tables]).contiguous().to(self.device)
        self.v_rot = torch.stack([t.rotation for t in v_tables]).contiguous().to(self.device)       # R
        self.rot_v = torch.stack([t.rotation.T.contiguous() for t in v_tables]).contiguous().to(self.device)
        self.v_bits = v_tables[0].bits
        self.vpb = packed_v_bytes(HD, self.v_bits)
        self.max_tpb = max(t.total_packed_bytes for t in k_tables)
        self.max_ng = max(t.n_groups for t in k_tables)
        self.max_mixed_bytes = max(t.pack_meta["nopack_start"] // 2 + t.pack_meta["nopack_len"] for t in k_tables)
        self.head_perm = torch.stack([t.head_perm for t in k_tables]).long().to(self.device)   # (n_kv, 128)
        self._plans = {}
        self._partition = None
        self._row_strides = {}
        self._early_fresh = 0

    def plan(self, flags: int = 0) -> _lib.DecodePlan:
        p = self._plans.get(flags)
        if p is None:
            p = make_decode_plan(self.desc_host, self.n_kv, flags, self.device,
                                 row_strides=self._row_strides.get(bool(flags & _lib.DEC_K_MIXED)))
            if self._partition is not None:
                _lib.check(_lib.lib().bgtq_decode_plan_set_partition(C.byref(p[0]), self._partition.data_ptr()),
                           "bgtq_decode_plan_set_partition")
            if self._early_fresh:
                _lib.check(_lib.lib().bgtq_decode_plan_set_early_fetch(C.byref(p[0]), self._early_fresh),
                           "bgtq_decode_plan_set_early_fetch")
            self._plans[flags] = p
        return p[0]

    def set_row_strides(self, kp_st: int, kn_st: int, vp_st: int, vn_st: int, mixed: bool = False) -> None:
        """Row strides (packed-K bytes, K-norm values, packed-V bytes, V-norm values per token) of the cache
        this layer's decode launches will read, for plans made after this call: their specialised kernel is
        compiled for exactly these (see ``bgtq_decode_plan_set_row_strides``)."""
        self._row_strides[bool(mixed)] = (kp_st, kn_st, vp_st, vn_st)

    def set_early_fetch(self, fresh_rows: int) -> None:
        """Let programmatic decode launches of this layer stream the cache before their dependency wait; the
        caller promises what ``bgtq_decode_plan_set_early_fetch`` asks for (0 turns it off again)."""
        self._early_fresh = int(fresh_rows)
        for p in self._plans.values():
            _lib.check(_lib.lib().bgtq_decode_plan_set_early_fetch(C.byref(p[0]), self._early_fresh),
                       "bgtq_decode_plan_set_early_fetch")

    def set_partition(self, table_dev) -> None:
        """Attach (or, with None, detach) a device copy of a ``decode_partition`` table to this layer's decode
        plans; the kernel uses it for launches it was made for and ignores it otherwise."""
        if table_dev is not None and (table_dev.dtype != torch.int32 or not table_dev.is_contiguous()
                                      or table_dev.device != self.device):
            raise ValueError("partition table must be a contiguous int32 tensor on the layer's device")
        self._partition = table_dev
        ptr = table_dev.data_ptr() if table_dev is not None else None
        for p in self._plans.values():
            _lib.check(_lib.lib().bgtq_decode_plan_set_partition(C.byref(p[0]), ptr), "bgtq_decode_plan_set_partition")


def _strides3(t: torch.Tensor):
    """(batch, head, token) element strides of a (B, H, T, X) tensor with unit last stride."""
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError(f"expected a (B, H, T, X) tensor with contiguous last dim, got {tuple(t.shape)} "
                         f"strides {t.stride()}")
    return t.stride(0), t.stride(1), t.stride(2)


def encode(layer: LayerTables, k, v, t0, k_packed, k_norms, v_packed, v_norms, *, flags=0,
           k_codes=None, v_codes=None, pos_dev=None, status=None):
    """Encode ``k``/``v`` (B, n_kv, S, 128) fp16 into rows ``t0 .. t0+S`` of the cache tensors
    ``k_packed`` (B, n_kv, T, bytes) u8, ``k_norms`` (B, n_kv, T, groups) f16|f32,
    ``v_packed`` (B, n_kv, T, bytes) u8 and ``v_norms`` (B, n_kv, T) f16.  Either side may be None.
    Bulk row counts (>= 128 rows) run the tcgen05 / tensor-memory encoder; ``_lib.ENC_NO_TCGEN05`` in ``flags``
    (or the environment variable ``BGTQ_ENC_NO_TCGEN05``) keeps them on the warp-MMA one."""
    L = _lib.lib()
    ref = k if k is not None else v
    _lib.require_cuda(ref, "k/v")
    B, H, S, D = ref.shape
    if H != layer.n_kv or D != HD:
        raise ValueError("shape does not match the layer tables")
    if k is None:
        flags |= _lib.ENC_SKIP_K
    if v is None:
        flags |= _lib.ENC_SKIP_V
    if os.environ.get("BGTQ_ENC_NO_TCGEN05"):
        flags |= _lib.ENC_NO_TCGEN05
    ks = _strides3(k) if k is not None else (0, 0, 0)
    vs = _strides3(v) if v is not None else (0, 0, 0)
    if k is not None:
        if k.dtype != torch.float16 or k_packed.dtype != torch.uint8:
            raise TypeError("k must be float16 and k_packed uint8")
        if k_norms.dtype == torch.float16:
            flags |= _lib.ENC_K_NORMS_F16
        elif k_norms.dtype != torch.float32:
            raise TypeError("k_norms must be float16 or float32")
        kps, kns = _strides3(k_packed), _strides3(k_norms)
        if t0 + S > k_packed.shape[2]:
            raise ValueError("cache overflow")
        kp_bytes, kn_count = k_packed.shape[3], k_norms.shape[3]
    else:
        kps = kns = (0, 0, 0)
        kp_bytes = kn_count = 1
    if v is not None:
        if v.dtype != torch.float16 or v_packed.dtype != torch.uint8 or v_norms.dtype != torch.float16:
            raise TypeError("v must be float16, v_packed uint8, v_norms float16")
        vps = _strides3(v_packed)
        need = HD // 2 if flags & _lib.ENC_V_NIBBLE else layer.vpb
        if v_packed.shape[3] < need:
            raise ValueError("v_packed rows are too short")
        vns = (v_norms.stride(0), v_norms.stride(1), v_norms.stride(2))
    else:
        vps = vns = (0, 0, 0)
    _lib.check(L.bgtq_encode(
        _lib.ptr(layer.desc_dev), _lib.ptr(layer.rot_k), _lib.ptr(layer.rot_v),
        _lib.ptr(k), *ks, _lib.ptr(v), *vs, B, H, S, int(t0),
        _lib.ptr(k_packed), *kps, kp_bytes, _lib.ptr(k_norms), *kns, kn_count,
        _lib.ptr(v_packed), *vps, _lib.ptr(v_norms), *vns,
        _lib.ptr(k_codes), _lib.ptr(v_codes), flags, _lib.ptr(pos_dev),
        int((k_packed if k is not None else v_packed).shape[2]), _lib.ptr(status),
        _lib.stream_ptr(ref.device)), "bgtq_encode")
    _lib.count_launch()


def rotate_q(layer: LayerTables, q: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """q (B, n_q, 128) or (B, n_q, 1, 128) fp16 -> (B, n_q, 128) fp16 in the packed-K basis."""
    _lib.require_cuda(q, "q")
    if q.dim() == 4:
        q = q[:, :, 0]
    if q.stride(2) != 1 or q.dtype != torch.float16:
        q = q.contiguous().to(torch.float16)
    B, n_q, _ = q.shape
    if out is None:
        out = torch.empty(B, n_q, HD, dtype=torch.float16, device=q.device)
    _lib.check(_lib.lib().bgtq_rotate_q(_lib.ptr(layer.desc_dev), _lib.ptr(layer.rot_k), _lib.ptr(q),
                                        q.stride(0), q.stride(1), _lib.ptr(out), B, n_q, layer.n_kv,
                                        _lib.stream_ptr(q.device)), "bgtq_rotate_q")
    _lib.count_launch()
    return out


def rotate_q_bulk(layer: LayerTables, q: torch.Tensor) -> torch.Tensor:
    """Many positions at once: q (B, n_q, S, 128) fp16 -> same shape in the packed-K basis, as one
    gather + fp32 GEMM per KV head group (the per-row kernel behind :func:`rotate_q` is meant for the
    handful of rows of a decode step)."""
    _lib.require_cuda(q, "q")
    B, n_q, S, D = q.shape
    gqa = n_q // layer.n_kv
    qg = q.reshape(B, layer.n_kv, gqa * S, D).float()
    idx = layer.head_perm.view(1, layer.n_kv, 1, D).expand(B, layer.n_kv, gqa * S, D)
    out = torch.matmul(torch.gather(qg, 3, idx), layer.rot_k.view(1, layer.n_kv, D, D))
    return out.to(torch.float16).view(B, n_q, S, D)


def step_prepare(layer: LayerTables, q, k, v, t0, k_packed, k_norms, v_packed, v_norms, *, q_rot=None,
                 flags=0, pos_dev=None, rope=None, ring=None, status=None):
    """``ring=(k_buf, v_buf, n_sink, window)``: three-region mode (``bgtq_step_prepare_ring``), see bgtq.h.
    Rotate q (B, n_q, [1,] 128) into ``q_rot`` and append one token k/v (B, n_kv, 1, 128) at slot
    ``t0`` (or ``*pos_dev``) of the cache tensors, in one launch.  ``q=None`` skips the rotation.
    ``rope=(cos, sin)``, each fp16 (B, 128) (or (B, 1, 128)): q and k are pre-RoPE and the kernel applies
    the rotary embedding of the step's position first (``bgtq_step_prepare_rope``)."""
    _lib.require_cuda(k, "k")
    B, H, S, D = k.shape
    if S != 1 or H != layer.n_kv or D != HD or v.shape != k.shape:
        raise ValueError("step_prepare appends exactly one token per (batch, KV head)")
    if k.dtype != torch.float16 or v.dtype != torch.float16 or k.stride(3) != 1 or v.stride(3) != 1:
        raise TypeError("k and v must be float16 with contiguous last dim")
    if k_norms.dtype == torch.float16:
        flags |= _lib.ENC_K_NORMS_F16
    n_q = 0
    qa = (0, 0, 0)
    if q is not None:
        if q.dim() == 4:
            q = q[:, :, 0]
        if q.dtype != torch.float16 or q.stride(2) != 1:
            q = q.to(torch.float16).contiguous()
        n_q = q.shape[1]
        if q_rot is None:
            q_rot = torch.empty(B, n_q, HD, dtype=torch.float16, device=k.device)
        qa = (_lib.ptr(q), q.stride(0), q.stride(1))
    kps, kns, vps = _strides3(k_packed), _strides3(k_norms), _strides3(v_packed)
    vns = (v_norms.stride(0), v_norms.stride(1), v_norms.stride(2))
    common = (_lib.ptr(layer.desc_dev), _lib.ptr(layer.rot_k), _lib.ptr(layer.rot_v), *qa,
              _lib.ptr(q_rot) if q is not None else 0, n_q,
              _lib.ptr(k), k.stride(0), k.stride(1), _lib.ptr(v), v.stride(0), v.stride(1), B, H, int(t0),
              _lib.ptr(k_packed), *kps, k_packed.shape[3], _lib.ptr(k_norms), *kns, k_norms.shape[3],
              _lib.ptr(v_packed), *vps, _lib.ptr(v_norms), *vns, flags, _lib.ptr(pos_dev),
              int(k_packed.shape[2]), _lib.ptr(status))
    if ring is not None:
        if rope is not None:
            raise NotImplementedError("fused RoPE and the three-region mode cannot be combined")
        k_buf, v_buf, n_sink, window = ring
        if k_buf.stride(2) != HD or k_buf.stride(3) != 1 or v_buf.stride() != k_buf.stride():
            raise ValueError("buffer tensors must be (B, n_kv, cap, 128) with contiguous token rows")
        _lib.check(_lib.lib().bgtq_step_prepare_ring(*common, _lib.ptr(k_buf), _lib.ptr(v_buf), k_buf.stride(0),
                                                     k_buf.stride(1), int(n_sink), int(window),
                                                     _lib.stream_ptr(k.device)), "bgtq_step_prepare_ring")
    elif rope is not None:
        cos, sin = (t.reshape(B, HD) for t in rope)
        if cos.dtype != torch.float16 or sin.dtype != torch.float16 or cos.stride(1) != 1 or sin.stride(1) != 1 \
                or cos.stride(0) != sin.stride(0):
            raise TypeError("rope tables must be float16 (B, 128) with equal row strides")
        _lib.check(_lib.lib().bgtq_step_prepare_rope(*common, _lib.ptr(cos), _lib.ptr(sin), cos.stride(0),
                                                     _lib.stream_ptr(k.device)), "bgtq_step_prepare_rope")
    else:
        _lib.check(_lib.lib().bgtq_step_prepare(*common, _lib.stream_ptr(k.device)), "bgtq_step_prepare")
    _lib.count_launch()
    return q_rot


def default_splits(n_batch: int, n_kv: int, n_tokens: int) -> int:
    return _lib.lib().bgtq_decode_default_splits(n_batch, n_kv, n_tokens)


def decode_grid_size(n_batch: int, n_kv: int, n_splits: int) -> int:
    """CTAs ``decode`` launches for this shape on the current device."""
    n = _lib.lib().bgtq_decode_grid_size(n_batch, n_kv, n_splits)
    if n < 1:
        _lib.check(n, "bgtq_decode_grid_size")
    return n


def decode_partition(n_batch: int, n_kv: int, n_tokens: int, n_splits: int, n_cta: int = None, out=None):
    """Item-range table (host int32 tensor, ``n_cta + 5`` words) that gives CTAs whose range straddles two
    (batch, head) pairs fewer items; copy it to the device and attach it with ``LayerTables.set_partition``."""
    if n_cta is None:
        n_cta = decode_grid_size(n_batch, n_kv, n_splits)
    if out is None:
        out = torch.empty(n_cta + 5, dtype=torch.int32)
    _lib.check(_lib.lib().bgtq_decode_partition(n_batch, n_kv, n_tokens, n_splits, n_cta, out.data_ptr(), out.numel()),
               "bgtq_decode_partition")
    return out


def decode(layer: LayerTables, q_rot, k_packed, k_norms, v_packed, v_norms, t_begin, t_end, *,
           n_splits=None, scale=None, flags=0, part_o=None, part_lse=None, status=None, pos_dev=None, pos_add=0):
    """Split-KV attention partials over cache rows [t_begin, t_end).

    Returns (part_o (B, n_q, n_splits, 128) f32, part_lse (B, n_q, n_splits) f32); slots that hold no
    partial have ``part_lse = -inf`` and an undefined ``part_o`` row (see ``bgtq_decode``)."""
    _lib.require_cuda(q_rot, "q_rot")
    B, n_q, _ = q_rot.shape
    if not q_rot.is_contiguous() or q_rot.dtype != torch.float16:
        raise ValueError("q_rot must be contiguous float16 (B, n_q, 128)")
    if k_norms.dtype != torch.float16 or v_norms.dtype != torch.float16:
        raise TypeError("cache norms must be float16")
    n_tok = t_end - t_begin
    if n_splits is None:
        n_splits = default_splits(B, layer.n_kv, n_tok)
    if scale is None:
        scale = 1.0 / math.sqrt(HD)
    if part_o is None:
        part_o = torch.empty(B, n_q, n_splits, HD, dtype=torch.float32, device=q_rot.device)
        part_lse = torch.empty(B, n_q, n_splits, dtype=torch.float32, device=q_rot.device)
    kps, kns, vps = _strides3(k_packed), _strides3(k_norms), _strides3(v_packed)
    vns = (v_norms.stride(0), v_norms.stride(1), v_norms.stride(2))
    plan = layer.plan(flags)
    _lib.check(_lib.lib().bgtq_decode(
        C.addressof(plan), _lib.ptr(layer.desc_dev), _lib.ptr(q_rot),
        _lib.ptr(k_packed), *kps, _lib.ptr(k_norms), *kns, _lib.ptr(v_packed), *vps, _lib.ptr(v_norms), *vns,
        B, n_q, layer.n_kv, int(t_begin), int(t_end), int(n_splits), float(scale),
        _lib.ptr(part_o), _lib.ptr(part_lse), _lib.ptr(status), _lib.ptr(pos_dev), int(pos_add),
        _lib.stream_ptr(q_rot.device)), "bgtq_decode")
    _lib.count_launch()
    return part_o, part_lse


def prefill_attention(layer: LayerTables, q_rot, k_packed, k_norms, v_packed, v_norms, n_tokens, *,
                      q_pos_offset=0, causal=True, scale=None, flags=0, v_rot=None):
    """Attention of q_rot (B, n_q, S_q, 128) fp16 (packed-K basis) over the first ``n_tokens`` cache rows;
    query i has absolute position ``q_pos_offset + i`` and, when ``causal``, sees tokens up to it.
    ``v_rot`` (n_kv, 128, 128) fp32 = R finishes V's rotation with one batched fp32 GEMM.
    Returns (B, n_q, S_q, 128) fp16.  ``_lib.PF_NO_TCGEN05`` in ``flags`` (or the environment variable
    ``BGTQ_PF_NO_TCGEN05``) keeps the products on mma.sync instead of tcgen05 / tensor memory."""
    _lib.require_cuda(q_rot, "q_rot")
    if os.environ.get("BGTQ_PF_NO_TCGEN05"):
        flags |= _lib.PF_NO_TCGEN05
    B, n_q, S_q, D = q_rot.shape
    if D != HD or q_rot.dtype != torch.float16 or q_rot.stride(3) != 1:
        raise ValueError("q_rot must be float16 (B, n_q, S_q, 128) with contiguous rows")
    if k_norms.dtype != torch.float16 or v_norms.dtype != torch.float16:
        raise TypeError("cache norms must be float16")
    if scale is None:
        scale = 1.0 / math.sqrt(HD)
    out_rot = torch.empty(B, n_q, S_q, HD, dtype=torch.float32, device=q_rot.device)
    kps, kns, vps = _strides3(k_packed), _strides3(k_norms), _strides3(v_packed)
    vns = (v_norms.stride(0), v_norms.stride(1), v_norms.stride(2))
    _lib.check(_lib.lib().bgtq_prefill_attention(
        _lib.ptr(layer.desc_dev), _lib.ptr(q_rot), q_rot.stride(0), q_rot.stride(1), q_rot.stride(2),
        _lib.ptr(k_packed), *kps, _lib.ptr(k_norms), *kns, _lib.ptr(v_packed), *vps, _lib.ptr(v_norms), *vns,
        B, n_q, layer.n_kv, S_q, int(n_tokens), int(q_pos_offset), 1 if causal else 0, float(scale), int(flags),
        _lib.ptr(out_rot), _lib.stream_ptr(q_rot.device)), "bgtq_prefill_attention")
    _lib.count_launch()
    if v_rot is None:
        return out_rot.to(torch.float16)
    gqa = n_q // layer.n_kv
    o = torch.matmul(out_rot.view(B, layer.n_kv, gqa * S_q, HD), v_rot.view(1, layer.n_kv, HD, HD))
    return o.view(B, n_q, S_q, HD).to(torch.float16)


def combine_ranks(gathered, n_batch, n_q, *, out=None):
    """Merge the all-gathered per-rank messages ``gathered`` (W, n_batch*n_q*129) fp32, each
    [O (B, n_q, 128) | LSE (B, n_q)], into fp16 (B, n_q, 128)."""
    _lib.require_cuda(gathered, "gathered")
    W = gathered.shape[0]
    if out is None:
        out = torch.empty(n_batch, n_q, HD, dtype=torch.float16, device=gathered.device)
    _lib.check(_lib.lib().bgtq_combine_ranks(
        _lib.ptr(gathered), W, gathered.stride(0), n_batch, n_q, _lib.ptr(out), out.stride(0), out.stride(1),
        0, _lib.stream_ptr(gathered.device)), "bgtq_combine_ranks")
    _lib.count_launch()
    return out


def combine(part_o, part_lse, n_kv, *, v_rot=None, buf_o=None, buf_lse=None, out=None,
            want_f32=False, want_lse=False, programmatic=False, o32_out=None, lse_out=None):
    """Merge (B, n_q, S, 128)/(B, n_q, S) partials -> fp16 (B, n_q, 128) [+ f32 copy, total LSE].
    ``programmatic``: launch as a programmatic dependent of the preceding kernel (see bgtq.h)."""
    B, n_q, S, _ = part_o.shape
    dev = part_o.device
    if out is None:
        out = torch.empty(B, n_q, HD, dtype=torch.float16, device=dev)
    o32 = o32_out if o32_out is not None else (
        torch.empty(B, n_q, HD, dtype=torch.float32, device=dev) if want_f32 else None)
    lse = lse_out if lse_out is not None else (
        torch.empty(B, n_q, dtype=torch.float32, device=dev) if want_lse else None)
    _lib.check(_lib.lib().bgtq_combine(
        _lib.ptr(part_o), _lib.ptr(part_lse), S, _lib.ptr(v_rot), _lib.ptr(buf_o), _lib.ptr(buf_lse),
        B, n_q, n_kv, _lib.ptr(out), out.stride(0), out.stride(1), _lib.ptr(o32), _lib.ptr(lse),
        _lib.COMBINE_PROGRAMMATIC if programmatic else 0, _lib.stream_ptr(dev)), "bgtq_combine")
    _lib.count_launch()
    return out, o32, lse


def buffer_attn(q, k_buf, v_buf, n_kv, scale, *, n_sink_tokens=0, n_ring_tokens=0, sink_cap, ring_first=0, ring_size,
                pos_dev=None, out=None):
    """Attention over unquantised fp16 tokens.  q (B, n_q, 128) fp16 (original basis);
    k_buf/v_buf (B, n_kv, cap, 128) fp16 with contiguous token rows: a sink prefix and a ring
    of ``ring_size`` slots starting at slot ``sink_cap`` (see ``bgtq_buffer_attn``)."""
    _lib.require_cuda(q, "q")
    if q.dim() == 4:
        q = q[:, :, 0]
    B, n_q, _ = q.shape
    if out is not None:
        o, lse = out
    else:
        o = torch.empty(B, n_q, HD, dtype=torch.float32, device=q.device)
        lse = torch.empty(B, n_q, dtype=torch.float32, device=q.device)
    if k_buf.stride(2) != HD or k_buf.stride(3) != 1 or v_buf.stride() != k_buf.stride():
        raise ValueError("buffer tensors must be (B, n_kv, cap, 128) with contiguous token rows")
    _lib.check(_lib.lib().bgtq_buffer_attn_pos(
        _lib.ptr(q), q.stride(0), q.stride(1), _lib.ptr(k_buf), _lib.ptr(v_buf), k_buf.stride(0), k_buf.stride(1),
        int(n_sink_tokens), int(n_ring_tokens), int(sink_cap), int(ring_first), int(ring_size),
        B, n_q, n_kv, float(scale), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(pos_dev), _lib.stream_ptr(q.device)),
        "bgtq_buffer_attn_pos")
    _lib.count_launch()
    return o, lse
