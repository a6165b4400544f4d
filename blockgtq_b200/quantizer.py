"""Host mirror of the reference's quantizer module (blockgtq/quantizer.py):
same class, function and argument names, same return shapes and dtypes, with
every GPU step executed by ``libbgtq.so``.

``BlockGTQQuantizer`` holds the static tables of one (layer, KV head).
``build_batched_encode_args`` stacks the heads of a layer and uploads them once;
the ``compress_*_batched`` operators then encode all heads in one launch.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib, calib
from .layer import LayerTables, encode as _encode

HD = _lib.HD

__all__ = [
    "BlockGTQQuantizer", "build_pack_meta", "build_batched_encode_args",
    "compress_k_packed_batched", "compress_v_packed_batched",
    "compress_k_mixed_batched", "compress_v_nibble4_batched",
]


def build_pack_meta(bit_allocation: torch.Tensor, head_perm: torch.Tensor) -> dict:
    """Per-width run table of a packed K row (quantizer.py:34-102)."""
    return calib._pack_meta(bit_allocation.detach().cpu().long(), head_perm.detach().cpu().long())


class _VQuantView:
    """The handful of ``PolarQuantGPU`` attributes callers read (v_quantize_gpu.py:57-81)."""

    def __init__(self, vt: calib.VHeadTables, device):
        self.d, self.bit_width, self.n_centroids = vt.head_dim, vt.bits, 1 << vt.bits
        self.device = device
        self.rotation = vt.rotation.to(device)
        self.centroids = vt.centroids.to(device)
        self.boundaries = vt.boundaries.to(device)

    @property
    def v_lut(self):
        return self.centroids.to(torch.float16)


class BlockGTQQuantizer:
    """Per-head K (mixed-rate) and V (uniform) quantiser tables + single-head operators.

    Constructor arguments and defaults follow quantizer.py:1007-1022."""

    def __init__(self, head_dim: int, avg_bits: float = 3.0, rotation_threshold: int = 2,
                 min_bits: int = 1, max_bits: int = 8, rope_base: float = 1e6, n_bins: int = 256,
                 device: torch.device = None):
        if head_dim != HD:
            raise ValueError("blockgtq_b200 supports head_dim=128 only")
        self.head_dim = head_dim
        self.avg_bits = avg_bits
        self.rotation_threshold = rotation_threshold
        self.min_bits, self.max_bits = min_bits, max_bits
        self.rope_base = rope_base
        self.n_bins = n_bins
        self.device = torch.device(device) if device is not None else torch.device("cuda:0")
        self.bit_allocation = None
        self._calibrated = False
        self._layer1 = None

    # -- calibration ---------------------------------------------------------
    def calibrate(self, q_data: torch.Tensor, k_data: torch.Tensor, bit_allocation: torch.Tensor = None):
        """Energies -> greedy bit map -> tables (quantizer.py:1024-1080).  ``q_data`` is
        ``(gqa * N, hd)``, ``k_data`` ``(N, hd)``; both are moved to the host for the (cheap) table build."""
        qd = None if q_data is None else q_data.detach().float().cpu()
        kd = None if k_data is None else k_data.detach().float().cpu()
        kt = calib.build_k_tables(qd, kd, head_dim=self.head_dim, avg_bits=self.avg_bits,
                                  rotation_threshold=self.rotation_threshold, min_bits=self.min_bits,
                                  max_bits=self.max_bits, n_bins=self.n_bins, bit_allocation=bit_allocation)
        self._tables = kt
        dev = self.device
        self.bit_allocation = kt.bit_allocation
        self._head_perm = kt.head_perm.to(dev)
        self._n_groups = kt.n_groups
        self._single_group = kt.n_groups == 1
        self._group_of = None if self._single_group else kt.group_of.to(dev)
        self._block_rot_T = kt.block_rot.T.contiguous().to(dev)
        inv = torch.empty_like(kt.head_perm)
        inv[kt.head_perm] = torch.arange(self.head_dim)
        self._rot_unperm = kt.block_rot[:, inv].contiguous().to(dev)
        self._pos_centroids = kt.pos_centroids.to(dev)
        self._pos_boundaries = kt.pos_boundaries.to(dev)
        self._code_lut = kt.code_lut.to(dev)
        self._pos_to_cb = kt.pos_to_cb.to(dev)
        self._lut_offsets = kt.lut_offsets.to(dev)
        self._lut_inv_scales = kt.lut_inv_scales.to(dev)
        self._n_codebooks = kt.n_groups
        self._pack_meta = kt.pack_meta
        self._pack_perm = kt.pack_meta["pack_perm"].to(dev)
        self._inv_pack_perm = kt.pack_meta["inv_pack_perm"].to(dev)
        self._total_packed_bytes = kt.total_packed_bytes
        self._total_bits = int(kt.bit_allocation.sum().item()) * 2
        self._calibrated = True
        self._q_perm_baked = False
        self._layer1 = None

    @property
    def effective_bits_per_dim(self):
        if self.bit_allocation is None:
            return self.avg_bits
        return self.bit_allocation.float().sum().item() / (self.head_dim // 2)

    @property
    def pack_meta(self):
        return self._pack_meta

    def build_kernel_args(self) -> dict:
        """Decode-side arguments of this head (quantizer.py:1093-1148)."""
        assert self._calibrated
        kt, dev = self._tables, self.device
        lut_offset = torch.zeros(self.head_dim, dtype=torch.int32)
        for bw, start, length, _po, lo, _ni in kt.segments:
            lut_offset[start:start + length] = lo
        return {
            "codebook_flat": kt.codebook_flat.to(dev),
            "lut_offset": lut_offset.to(dev),
            "norm_group": kt.group_of.to(torch.int32).to(dev),
            "segments_b": list(kt.segments),
            "total_packed_bytes": kt.total_packed_bytes,
        }

    @property
    def composite_q_perm(self) -> torch.Tensor:
        assert self._calibrated
        return self._head_perm[self._pack_perm]

    # -- V side ----------------------------------------------------------------
    def init_v_quantizer(self, v_bits: int = 3, seed: int = 42):
        """Seed-deterministic V rotation and codebook (quantizer.py:1478-1497)."""
        self._v_tables = calib.build_v_tables(self.head_dim, v_bits, seed)
        self._v_quantizer = _VQuantView(self._v_tables, self.device)
        self._v_bits = v_bits
        self._v_rot = self._v_quantizer.rotation.contiguous()
        self._v_rot_T = self._v_rot.T.contiguous()
        self._v_boundaries = self._v_quantizer.boundaries.contiguous()
        self._v_centroids_f32 = self._v_quantizer.centroids.contiguous()
        self._layer1 = None

    @property
    def v_bits(self) -> int:
        return getattr(self, "_v_bits", 0)

    @property
    def v_lut(self) -> torch.Tensor:
        assert hasattr(self, "_v_quantizer"), "call init_v_quantizer() first"
        return self._v_quantizer.v_lut

    # -- single-head operators ---------------------------------------------------
    def _single(self) -> LayerTables:
        if self._layer1 is None:
            vt = getattr(self, "_v_tables", None) or calib.build_v_tables(self.head_dim, 3, 42)
            self._layer1 = LayerTables([self._tables], [vt], self.device)
        return self._layer1

    def _rows(self, x):
        flat = x.reshape(-1, self.head_dim).to(torch.float16).contiguous()
        return flat.view(1, 1, flat.shape[0], self.head_dim), x.shape[:-1]

    @torch.no_grad()
    def compress(self, k: torch.Tensor, block_n: int = 32):
        """fp16 keys -> (codes (..., hd) u8 in packed order, norms (..., G) f32) (quantizer.py:1245-1296)."""
        assert self._calibrated
        x, lead = self._rows(k)
        n = x.shape[2]
        lt = self._single()
        kp = torch.empty(1, 1, n, lt.max_tpb, dtype=torch.uint8, device=x.device)
        kn = torch.empty(1, 1, n, self._n_groups, dtype=torch.float32, device=x.device)
        codes = torch.empty(1, 1, n, self.head_dim, dtype=torch.uint8, device=x.device)
        _encode(lt, x, None, 0, kp, kn, None, None, k_codes=codes)
        return codes.reshape(*lead, self.head_dim), kn.reshape(*lead, self._n_groups)

    @torch.no_grad()
    def correct_norms(self, k, raw_norms, block_n: int = 32):
        """raw_norms / ||centroid[codes]|| per group (quantizer.py:1298-1345)."""
        codes, _ = self.compress(k)
        cf = codes.reshape(-1, self.head_dim).long()
        cents = self._pos_centroids[torch.arange(self.head_dim, device=cf.device)[None, :], cf]
        out = raw_norms.reshape(-1, self._n_groups).float().clone()
        go = self._tables.group_of.to(cf.device)
        for g in range(self._n_groups):
            out[:, g] /= cents[:, go == g].norm(dim=-1).clamp(min=1e-10)
        return out.reshape(*k.shape[:-1], self._n_groups)

    @torch.no_grad()
    def compress_packed(self, k, block_n: int = 32, norm_correct: bool = False):
        """-> (packed (..., bytes) u8, norms (..., G) f32, information bits) (quantizer.py:1347-1430)."""
        assert self._calibrated
        x, lead = self._rows(k)
        n = x.shape[2]
        lt = self._single()
        kp = torch.empty(1, 1, n, self._total_packed_bytes, dtype=torch.uint8, device=x.device)
        kn = torch.empty(1, 1, n, self._n_groups, dtype=torch.float32, device=x.device)
        _encode(lt, x, None, 0, kp, kn, None, None)
        norms = kn.reshape(*lead, self._n_groups)
        if norm_correct:
            norms = self.correct_norms(k, norms)
        return kp.reshape(*lead, self._total_packed_bytes), norms, self._total_bits

    @torch.no_grad()
    def compress_v(self, v):
        """-> (codes (..., hd) u8, corrected norms (...,) f16) (quantizer.py:1523-1541)."""
        x, lead = self._rows(v)
        n = x.shape[2]
        lt = self._single()
        vp = torch.empty(1, 1, n, lt.vpb, dtype=torch.uint8, device=x.device)
        vn = torch.empty(1, 1, n, dtype=torch.float16, device=x.device)
        codes = torch.empty(1, 1, n, self.head_dim, dtype=torch.uint8, device=x.device)
        _encode(lt, None, x, 0, None, None, vp, vn, v_codes=codes)
        return codes.reshape(*lead, self.head_dim), vn.reshape(*lead)

    @torch.no_grad()
    def compress_v_packed(self, v, block_n: int = 32):
        """-> (packed (..., bytes) u8, corrected norms (...,) f16) (quantizer.py:1543-1591)."""
        x, lead = self._rows(v)
        n = x.shape[2]
        lt = self._single()
        vp = torch.empty(1, 1, n, lt.vpb, dtype=torch.uint8, device=x.device)
        vn = torch.empty(1, 1, n, dtype=torch.float16, device=x.device)
        _encode(lt, None, x, 0, None, None, vp, vn)
        return vp.reshape(*lead, lt.vpb), vn.reshape(*lead)

    # -- query side ----------------------------------------------------------------
    def rotate_q_for_packed_kernel(self, q: torch.Tensor) -> torch.Tensor:
        """q (..., hd) -> same shape/dtype, permuted and rotated like K (quantizer.py:1160-1187)."""
        assert self._calibrated
        from .layer import rotate_q
        if q.dtype != torch.float16:
            flat = q.reshape(-1, self.head_dim).float()
            return ((flat[:, self._head_perm] @ self._block_rot_T)[:, self._pack_perm]).to(q.dtype).reshape(q.shape)
        flat = q.reshape(1, -1, self.head_dim)
        # one "KV head" with every row as a query head of its group
        lt = self._single()
        out = rotate_q(_GroupView(lt, flat.shape[1]), flat)
        return out.reshape(q.shape)

    @torch.no_grad()
    def bake_permutation_into_qproj(self, q_proj_weight, kv_head_idx: int, n_kv_heads: int, n_q_heads: int,
                                    q_proj_bias: Optional[torch.Tensor] = None) -> None:
        """Fold permutation + rotation into the q_proj rows of this KV head's query group, in place, so
        that the projection's output already is ``rotate_q_for_packed_kernel`` of the original output and
        the decode step can skip the rotation (quantizer.py:1189-1243).

        With ``rot_T = block_rot_T`` the rotation of a query row is ``q[head_perm] @ rot_T``, i.e. the
        baked weight is ``(rot_T.T @ W[head_perm])[pack_perm]``.  The reference's function multiplies by
        ``rot_T`` itself (quantizer.py:1232), which equals the rotation only for a symmetric matrix: on
        random data its baked projection differs from its own ``rotate_q_for_packed_kernel`` by more than
        the values themselves.  This implementation follows the documented intent, and a test holds it to
        the rotation."""
        assert self._calibrated and kv_head_idx < n_kv_heads
        hd, gqa = self.head_dim, n_q_heads // n_kv_heads
        assert q_proj_weight.shape[0] == n_q_heads * hd
        hp = self._head_perm.detach().cpu()
        pp = self._pack_perm.detach().cpu()
        rt = self._block_rot_T.detach().cpu().float()
        for g in range(gqa):
            s = (kv_head_idx * gqa + g) * hd
            w = q_proj_weight[s:s + hd].detach().clone().cpu()[hp].float()
            q_proj_weight[s:s + hd] = (rt.T @ w).to(q_proj_weight.dtype)[pp].to(q_proj_weight.device)
            if q_proj_bias is not None:
                bv = q_proj_bias[s:s + hd].detach().clone().cpu()[hp].float()
                q_proj_bias[s:s + hd] = (rt.T @ bv.unsqueeze(1)).squeeze(1)[pp].to(q_proj_bias.dtype).to(
                    q_proj_bias.device)
        self._q_perm_baked = True


class _GroupView:
    """Presents single-head tables to rotate_q with n_kv = 1 (all rows share the head)."""

    def __init__(self, lt: LayerTables, n_rows: int):
        self.desc_dev, self.rot_k, self.n_kv = lt.desc_dev, lt.rot_k, 1


# ---------------------------------------------------------------------------
# batched (all KV heads of a layer) operators
# ---------------------------------------------------------------------------

def build_batched_encode_args(quantizers: list, device="cuda") -> dict:
    """Stack the heads of one layer and upload their tables once.

    Returns the reference's dictionary keys that callers read
    (quantizer.py:1710-1747) plus ``'_layer'``, the device tables."""
    q0 = quantizers[0]
    lt = LayerTables([q._tables for q in quantizers], [q._v_tables for q in quantizers], device)
    n_kv, hd = len(quantizers), q0.head_dim
    pms = [q._pack_meta for q in quantizers]

    def mx(bw):
        return max((pm[bw]["length"] if bw in pm else 0) for pm in pms)

    # Tables the reference's Triton kernels index directly (quantizer.py:1722-1730).  The CUDA kernels read the
    # same values from the uploaded head descriptors; the stacks are kept for callers that inspect them.
    dev = torch.device(device)
    max_ncb = max(q._n_codebooks for q in quantizers)
    max_ng = max(q._n_groups for q in quantizers)
    clut_stride = q0._code_lut.stride(0)
    clut = torch.zeros(n_kv, max_ncb, clut_stride, dtype=q0._code_lut.dtype, device=dev)
    max_nc = max(q._pos_centroids.shape[1] for q in quantizers)
    pos_cents = torch.zeros(n_kv, hd, max_nc, dtype=torch.float32, device=dev)
    grp = torch.zeros(n_kv, hd, dtype=torch.long, device=dev)
    gmask = torch.zeros(n_kv, max_ng, hd, dtype=torch.float32, device=dev)
    pack_params = torch.zeros(n_kv, 16, dtype=torch.int32, device=dev)
    for i, q in enumerate(quantizers):
        clut[i, :q._n_codebooks] = q._code_lut.to(dev)
        pos_cents[i, :, :q._pos_centroids.shape[1]] = q._pos_centroids.to(dev)
        if q._group_of is not None:
            grp[i] = q._group_of.to(dev)
        ipp = q._inv_pack_perm.to(dev)
        for g in range(q._n_groups):
            in_g = (q._group_of.to(dev) == g) if q._group_of is not None else torch.ones(hd, dtype=torch.bool, device=dev)
            gmask[i, g] = in_g[ipp].float()
        m = q._pack_meta
        row = []
        for bw in (1, 2, 3, 4):
            row += [m[bw]["start"], m[bw]["length"], m[bw]["pack_offset"]] if bw in m else [0, 0, 0]
        row += [m["nopack_start"], m["nopack_len"], m["nopack_off"], q._n_groups]
        pack_params[i] = torch.tensor(row, dtype=torch.int32)

    return {
        "_layer": lt,
        "k_clut_stack": clut, "k_pos_cents_stack": pos_cents,
        "k_ptcb_stack": torch.stack([q._pos_to_cb.to(dev) for q in quantizers]),
        "k_loff_stack": torch.stack([q._lut_offsets.to(dev) for q in quantizers]),
        "k_linv_stack": torch.stack([q._lut_inv_scales.to(dev) for q in quantizers]),
        "k_grp_stack": grp, "k_group_mask_stack": gmask, "k_pack_params": pack_params, "k_clut_stride": clut_stride,
        "v_rot_T_stack": lt.rot_v, "v_bound_stack": torch.stack([q._v_boundaries for q in quantizers]),
        "v_cent_stack": torch.stack([q._v_centroids_f32 for q in quantizers]),
        "v_bits": lt.v_bits, "v_n_cents": 1 << lt.v_bits, "v_packed_bytes": lt.vpb, "v_nibble_bytes": hd // 2,
        "k_perm_stack": torch.stack([q._head_perm for q in quantizers]),
        "k_inv_pp_stack": torch.stack([q._inv_pack_perm for q in quantizers]),
        "k_rot_stack": lt.rot_k,
        "n_kv": n_kv, "hd": hd, "n_bins": q0.n_bins,
        "max_n_groups": lt.max_ng, "max_n_codebooks": max(q._n_codebooks for q in quantizers),
        "max_tpb": lt.max_tpb,
        "max_bw1_len": mx(1), "max_bw2_len": mx(2), "max_bw3_len": mx(3), "max_bw4_len": mx(4),
        "max_np_len": max(pm["nopack_len"] for pm in pms),
        "max_mixed_bytes": lt.max_mixed_bytes,
        "mixed_nopack_starts": [pm["nopack_start"] for pm in pms],
        "mixed_nopack_lens": [pm["nopack_len"] for pm in pms],
    }


def _flat4(x: torch.Tensor):
    """(n_kv, N, hd) -> (1, n_kv, N, hd) view for the encoder's (B, H, S, D) grid."""
    if x.dim() != 3 or x.shape[2] != HD:
        raise ValueError("expected (n_kv, N, 128)")
    return x.to(torch.float16).contiguous().unsqueeze(0)


@torch.no_grad()
def compress_k_packed_batched(k_flat, args, block_n: int = 32):
    """(n_kv, N, hd) fp16 -> (packed (n_kv, N, max_tpb) u8, norms (n_kv, N, max_ng) f32)
    (quantizer.py:2104-2172)."""
    lt = args["_layer"]
    n_kv, n, _ = k_flat.shape
    kp = torch.empty(1, n_kv, n, lt.max_tpb, dtype=torch.uint8, device=k_flat.device)
    kn = torch.empty(1, n_kv, n, lt.max_ng, dtype=torch.float32, device=k_flat.device)
    _encode(lt, _flat4(k_flat), None, 0, kp, kn, None, None)
    return kp[0], kn[0]


@torch.no_grad()
def compress_v_packed_batched(v_flat, args, block_n: int = 32):
    """(n_kv, N, hd) fp16 -> (packed (n_kv, N, vpb) u8, norms (n_kv, N) f16) (quantizer.py:1979-2029)."""
    lt = args["_layer"]
    n_kv, n, _ = v_flat.shape
    vp = torch.empty(1, n_kv, n, lt.vpb, dtype=torch.uint8, device=v_flat.device)
    vn = torch.empty(1, n_kv, n, dtype=torch.float16, device=v_flat.device)
    _encode(lt, None, _flat4(v_flat), 0, None, None, vp, vn)
    return vp[0], vn[0]


@torch.no_grad()
def compress_k_mixed_batched(k_flat, args, block_n: int = 32, norm_correct: bool = True):
    """-> (k_mixed (n_kv, N, max_mixed_bytes) u8: nibble pairs then raw bytes, norms f32)
    (quantizer.py:1843-1976)."""
    lt = args["_layer"]
    n_kv, n, _ = k_flat.shape
    kp = torch.empty(1, n_kv, n, lt.max_mixed_bytes, dtype=torch.uint8, device=k_flat.device)
    kn = torch.empty(1, n_kv, n, lt.max_ng, dtype=torch.float32, device=k_flat.device)
    if norm_correct:
        _encode(lt, _flat4(k_flat), None, 0, kp, kn, None, None, flags=_lib.ENC_K_MIXED)
    else:
        # layout from the mixed mode, norms from the plain mode
        _encode(lt, _flat4(k_flat), None, 0, kp, kn.clone(), None, None, flags=_lib.ENC_K_MIXED)
        tmp = torch.empty(1, n_kv, n, lt.max_tpb, dtype=torch.uint8, device=k_flat.device)
        _encode(lt, _flat4(k_flat), None, 0, tmp, kn, None, None)
    return kp[0], kn[0]


@torch.no_grad()
def compress_v_nibble4_batched(v_flat, args, block_n: int = 32):
    """-> (nibble4 (n_kv, N, hd/2) u8, norms (n_kv, N) f16) (quantizer.py:2032-2101)."""
    lt = args["_layer"]
    n_kv, n, _ = v_flat.shape
    vp = torch.empty(1, n_kv, n, HD // 2, dtype=torch.uint8, device=v_flat.device)
    vn = torch.empty(1, n_kv, n, dtype=torch.float16, device=v_flat.device)
    _encode(lt, None, _flat4(v_flat), 0, None, None, vp, vn, flags=_lib.ENC_V_NIBBLE)
    return vp[0], vn[0]
