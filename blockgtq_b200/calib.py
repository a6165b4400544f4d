"""Host-side metadata for one (layer, KV-head): everything the CUDA kernels
need that is fixed after calibration.

The tables built here must equal the reference's tensor for tensor, because
they define both the packed byte layout and the code values:

* block energies and the greedy bit map     (blockgtq/freq_analysis.py:18-35,
                                              blockgtq/allocator.py:20-55)
* ``head_perm``, width groups, block-diagonal Haar rotation, per-group
  Lloyd-Max codebooks                        (blockgtq/block_gtq_pipeline.py:151-246)
* the 256-bin uniform LUT that maps a rotated coordinate to a code
                                             (blockgtq/kernels/quant_kernels.py:276-364)
* packed-segment table                       (blockgtq/quantizer.py:34-102)
* flat fp16 codebook + segment tuples        (blockgtq/quantizer.py:1093-1148)
* V rotation, Monte-Carlo Lloyd codebook     (blockgtq/v_quantize_gpu.py:19-81)

Where the reference's result depends on a library routine (``torch.argsort``
tie order, ``torch.linspace`` rounding, NumPy's ``default_rng`` stream, LAPACK
QR, SciPy's normal CDF) the same routine is called here so the outputs agree
bit for bit; the arithmetic around those calls is written independently and
vectorised (the reference spends about 3 s per head in Python loops, this
takes a few milliseconds).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from functools import lru_cache

import numpy as np
import torch

from .allocator import greedy_bit_allocation

__all__ = [
    "block_energy", "haar_rotation", "lloyd_max_gaussian", "v_codebook",
    "v_rotation", "packed_v_bytes", "segment_bytes", "KHeadTables",
    "VHeadTables", "build_k_tables", "build_v_tables",
]


# ---------------------------------------------------------------------------
# scores
# ---------------------------------------------------------------------------

def block_energy(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """``s_i = (E||q_i||^2 + E||k_i||^2) / 2`` per RoPE block.

    ``q`` is ``(n_q_samples, hd)``, ``k`` is ``(n_k_samples, hd)``; block ``i``
    is the split-half pair of dims ``(i, i + hd/2)``
    (blockgtq/rope_utils.py:23-32).
    """
    half = q.shape[-1] // 2

    def _e(x):
        sq = x * x
        return (sq[..., :half] + sq[..., half:]).mean(dim=0)

    return (_e(q) + _e(k)) / 2


# ---------------------------------------------------------------------------
# rotations and codebooks
# ---------------------------------------------------------------------------

def haar_rotation(d: int, seed: int, *, fix_zero_sign: bool) -> np.ndarray:
    """Seeded Haar rotation (float64): QR of a Gaussian matrix, columns
    multiplied by ``sign(diag R)``, first column flipped if ``det < 0``.

    K-side group rotations treat ``sign == 0`` as ``+1`` and test the
    determinant with ``slogdet`` (block_gtq_pipeline.py:81-92); the V-side
    rotation uses the raw sign and ``det`` (v_quantize_gpu.py:19-29).
    """
    g = np.random.default_rng(seed).standard_normal((d, d))
    qm, rm = np.linalg.qr(g)
    sg = np.sign(np.diag(rm))
    if fix_zero_sign:
        sg[sg == 0] = 1.0
    qm = qm * sg[np.newaxis, :]
    neg = (np.linalg.slogdet(qm)[0] < 0) if fix_zero_sign else (np.linalg.det(qm) < 0)
    if neg:
        qm[:, 0] = -qm[:, 0]
    return qm


def _gauss_cell_mean(sig: float, lo: np.ndarray, hi: np.ndarray) -> np.ndarray:
    """E[x | lo < x <= hi] for x ~ N(0, sig^2); ``lo``/``hi`` may be +-inf."""
    from scipy import stats as st

    a = lo / sig
    b = hi / sig
    prob = np.where(np.isneginf(a), st.norm.cdf(b),
                    np.where(np.isposinf(b), st.norm.sf(a),
                             st.norm.cdf(b) - st.norm.cdf(a)))
    dens = st.norm.pdf(a) - st.norm.pdf(b)
    with np.errstate(divide="ignore", invalid="ignore"):
        out = sig * dens / prob
    tiny = prob < 1e-15
    if tiny.any():
        fa, fb = np.isfinite(lo), np.isfinite(hi)
        fallback = np.where(fa & ~fb, lo + sig,
                            np.where(~fa & fb, hi - sig,
                                     np.where(fa & fb, (lo + hi) / 2.0, 0.0)))
        out = np.where(tiny, fallback, out)
    return out


@lru_cache(maxsize=None)
def _lloyd_max_cached(bits: int, d: int) -> tuple:
    n = 1 << bits
    if bits == 1:
        c = math.sqrt(2.0 / (math.pi * d))
        return (-c, c)
    if bits == 2:
        return tuple((np.array([-1.51, -0.453, 0.453, 1.51]) / math.sqrt(d)).tolist())
    from scipy import stats as st

    sig = 1.0 / math.sqrt(d)
    edges = st.norm.ppf(np.linspace(0, 1, n + 1)[1:-1], scale=sig)
    cents = None
    for _ in range(101):          # one initial pass from the quantile edges + 100 Lloyd steps
        if cents is not None:
            edges = (cents[:-1] + cents[1:]) / 2.0
        lo = np.concatenate([[-np.inf], edges])
        hi = np.concatenate([edges, [np.inf]])
        cents = _gauss_cell_mean(sig, lo, hi)
    return tuple(np.sort(cents).tolist())


def lloyd_max_gaussian(bits: int, d: int) -> np.ndarray:
    """MSE-optimal ``2**bits`` scalar levels for a coordinate of a unit vector
    rotated in ``d`` dims (~N(0, 1/d)); closed forms for 1 and 2 bits,
    analytic Lloyd iteration otherwise (block_gtq_pipeline.py:24-78)."""
    return np.asarray(_lloyd_max_cached(int(bits), int(d)), dtype=np.float64)


@lru_cache(maxsize=None)
def _v_codebook_cached(bits: int, d: int) -> tuple:
    n = 1 << bits
    if bits == 1:
        c = np.sqrt(2.0 / (np.pi * d))
        return (-c, c)
    if bits == 2:
        return tuple((np.array([-1.51, -0.453, 0.453, 1.51]) / np.sqrt(d)).tolist())
    sig = 1.0 / np.sqrt(d)
    cents = np.linspace(-3 * sig, 3 * sig, n)
    draws = np.random.default_rng(0).normal(0, sig, 100000)   # same stream every sweep
    for _ in range(100):
        cell = np.searchsorted((cents[:-1] + cents[1:]) / 2.0, draws)
        nxt = np.array([draws[cell == i].mean() if (cell == i).any() else cents[i]
                        for i in range(n)])
        if np.allclose(cents, nxt, atol=1e-8):
            break
        cents = nxt
    return tuple(np.sort(cents).tolist())


def v_codebook(bits: int, d: int) -> np.ndarray:
    """V-side levels: closed forms for 1/2 bits, otherwise Lloyd on 100 000
    seeded Gaussian draws (v_quantize_gpu.py:32-54)."""
    return np.asarray(_v_codebook_cached(int(bits), int(d)), dtype=np.float64)


def v_rotation(d: int, seed: int) -> np.ndarray:
    return haar_rotation(d, seed, fix_zero_sign=False).astype(np.float32)


# ---------------------------------------------------------------------------
# byte layout
# ---------------------------------------------------------------------------

def segment_bytes(bits: int, n_codes: int) -> int:
    """Bytes one token spends on a run of ``n_codes`` codes of one width.
    Widths 1-4 are an LSB-first bit stream (3-bit runs padded to whole 3-byte
    groups of 8 codes); widths 5-8 are one raw byte per code
    (quantizer.py:63-72)."""
    if bits == 1:
        return (n_codes + 7) // 8
    if bits == 2:
        return (n_codes + 3) // 4
    if bits == 3:
        return ((n_codes + 7) // 8) * 3
    if bits == 4:
        return (n_codes + 1) // 2
    return n_codes


def packed_v_bytes(head_dim: int, bits: int) -> int:
    """Packed V bytes per token (v_packing.py:17-28); widths 1-4 only."""
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"V packing supports 1-4 bits, got {bits}")
    return segment_bytes(bits, head_dim)


# ---------------------------------------------------------------------------
# K tables
# ---------------------------------------------------------------------------

@dataclass
class KHeadTables:
    """Static K-side tables of one head, all on the host (CPU tensors)."""
    head_dim: int
    bit_allocation: torch.Tensor        # (hd/2,) int64
    head_perm: torch.Tensor             # (hd,) int64: packed position -> original dim
    group_bits: list                    # ascending distinct widths
    group_slices: list                  # [(start, end)] in packed order
    group_of: torch.Tensor              # (hd,) int64
    block_rot: torch.Tensor             # (hd, hd) f32 block diagonal
    pos_centroids: torch.Tensor         # (hd, 2**max_bits) f32, zero padded
    pos_boundaries: torch.Tensor        # (hd, 2**max_bits - 1) f32, +inf padded
    code_lut: torch.Tensor              # (n_groups, n_bins) u8
    pos_to_cb: torch.Tensor             # (hd,) int32
    lut_offsets: torch.Tensor           # (hd,) f32
    lut_inv_scales: torch.Tensor        # (hd,) f32
    pack_meta: dict = field(default_factory=dict)
    segments: list = field(default_factory=list)   # (bw, start, len, pack_off, lut_off, norm_idx)
    codebook_flat: torch.Tensor = None  # (sum 2**bw,) f16
    scores: torch.Tensor = None

    @property
    def n_groups(self) -> int:
        return len(self.group_bits)

    @property
    def total_packed_bytes(self) -> int:
        return self.pack_meta["total_packed_bytes"]


def _pack_meta(bit_allocation: torch.Tensor, head_perm: torch.Tensor) -> dict:
    """Per-width run table in packed order (same keys as quantizer.py:34-102).

    ``head_perm`` already orders dims by width, so the stable sort by width is
    the identity; it is still computed so the contiguity check is real."""
    hd = head_perm.shape[0]
    width_of_dim = torch.cat([bit_allocation, bit_allocation])[head_perm]
    order = torch.argsort(width_of_dim, stable=True)
    w = width_of_dim[order].tolist()
    meta, off = {}, 0
    for bw in range(1, 9):
        where = [i for i, x in enumerate(w) if x == bw]
        if not where:
            continue
        s, n = where[0], len(where)
        if where[-1] != s + n - 1:
            raise AssertionError(f"dims of width {bw} are not contiguous in packed order")
        nb = segment_bytes(bw, n)
        meta[bw] = {"start": s, "length": n, "pack_offset": off, "packed_bytes": nb}
        off += nb
    raw = [meta[b] for b in range(5, 9) if b in meta]
    meta["nopack_start"] = raw[0]["start"] if raw else hd
    meta["nopack_off"] = raw[0]["pack_offset"] if raw else 0
    meta["nopack_len"] = sum(r["length"] for r in raw)
    meta["total_packed_bytes"] = off
    meta["pack_perm"] = order
    inv = torch.empty_like(order)
    inv[order] = torch.arange(hd)
    meta["inv_pack_perm"] = inv
    return meta


def _code_lut(cents32: torch.Tensor, n_bins: int):
    """Uniform-bin LUT for one codebook: returns (lut u8 (n_bins,), offset, inv_scale).

    The bin grid spans [c_min - gap/2, c_max + gap/2] with gap the mean level
    spacing; a bin takes the code of the cell its centre falls in
    (quant_kernels.py:334-362).  Scalars are Python floats taken from the
    float32 levels, as in the reference."""
    nc = cents32.numel()
    lo, hi = cents32.min().item(), cents32.max().item()
    half_gap = (hi - lo) / max(nc - 1, 1) * 0.5
    r0, r1 = lo - half_gap, hi + half_gap
    bw = (r1 - r0) / n_bins
    centres = torch.linspace(r0 + bw / 2, r1 - bw / 2, n_bins, dtype=torch.float32)
    edges = (cents32[:-1] + cents32[1:]) / 2.0
    lut = torch.searchsorted(edges.contiguous(), centres).clamp(max=nc - 1).to(torch.uint8)
    return lut, r0, 1.0 / bw


def build_k_tables(q_data: torch.Tensor, k_data: torch.Tensor, *, head_dim: int,
                   avg_bits: float = 3.0, rotation_threshold: int = 2,
                   min_bits: int = 1, max_bits: int = 8, n_bins: int = 256,
                   bit_allocation: torch.Tensor | None = None) -> KHeadTables:
    """Calibrate one head: energies -> bit map -> every K-side table.

    ``bit_allocation`` may be supplied to skip the data-dependent part."""
    hd, nblk = head_dim, head_dim // 2
    scores = None
    if bit_allocation is None:
        scores = block_energy(q_data, k_data)
        bit_allocation = greedy_bit_allocation(scores, int(nblk * avg_bits), min_bits, max_bits)
    bit_allocation = bit_allocation.detach().cpu().long()

    order = bit_allocation.argsort()            # library tie order is part of the format
    sorted_bits = bit_allocation[order]
    head_perm = torch.stack([order, order + nblk], dim=1).reshape(-1)

    group_bits = sorted(set(sorted_bits.tolist()))
    counts = [int((sorted_bits == b).sum()) * 2 for b in group_bits]
    ends = np.cumsum(counts).tolist()
    slices = [(e - c, e) for c, e in zip(counts, ends)]

    nc_max = 1 << max(group_bits)
    rot = torch.zeros(hd, hd, dtype=torch.float32)
    cents = torch.zeros(hd, nc_max, dtype=torch.float32)
    bounds = torch.full((hd, nc_max - 1), float("inf"), dtype=torch.float32)
    group_of = torch.zeros(hd, dtype=torch.long)
    code_lut = torch.zeros(len(group_bits), n_bins, dtype=torch.uint8)
    offs = torch.zeros(hd, dtype=torch.float32)
    invs = torch.zeros(hd, dtype=torch.float32)

    for gi, (bw, (s, e)) in enumerate(zip(group_bits, slices)):
        d = e - s
        if bw < rotation_threshold:
            rot[s:e, s:e] = torch.eye(d)
        else:
            rot[s:e, s:e] = torch.tensor(haar_rotation(d, 42 + bw, fix_zero_sign=True),
                                         dtype=torch.float32)
        c32 = torch.tensor(lloyd_max_gaussian(bw, d), dtype=torch.float32)
        cents[s:e, :c32.numel()] = c32
        bounds[s:e, :c32.numel() - 1] = (c32[:-1] + c32[1:]) / 2.0
        group_of[s:e] = gi
        code_lut[gi], o, iv = _code_lut(c32, n_bins)
        offs[s:e] = o
        invs[s:e] = iv

    t = KHeadTables(
        head_dim=hd, bit_allocation=bit_allocation, head_perm=head_perm,
        group_bits=group_bits, group_slices=slices, group_of=group_of,
        block_rot=rot, pos_centroids=cents, pos_boundaries=bounds,
        code_lut=code_lut, pos_to_cb=group_of.to(torch.int32),
        lut_offsets=offs, lut_inv_scales=invs, scores=scores)
    t.pack_meta = _pack_meta(bit_allocation, head_perm)

    parts, lut_off = [], 0
    for gi, bw in enumerate(group_bits):
        m = t.pack_meta[bw]
        parts.append(cents[m["start"], :1 << bw].to(torch.float16))
        t.segments.append((bw, m["start"], m["length"], m["pack_offset"], lut_off, gi))
        lut_off += 1 << bw
    t.codebook_flat = torch.cat(parts)
    return t


# ---------------------------------------------------------------------------
# V tables
# ---------------------------------------------------------------------------

@dataclass
class VHeadTables:
    head_dim: int
    bits: int
    seed: int
    rotation: torch.Tensor      # (hd, hd) f32: y = R @ v_unit
    centroids: torch.Tensor     # (2**bits,) f32
    boundaries: torch.Tensor    # (2**bits - 1,) f32
    lut_f16: torch.Tensor       # (2**bits,) f16

    @property
    def packed_bytes(self) -> int:
        return packed_v_bytes(self.head_dim, self.bits)


def build_v_tables(head_dim: int, bits: int, seed: int) -> VHeadTables:
    c64 = v_codebook(bits, head_dim)
    cents = torch.from_numpy(c64.astype(np.float32))
    edges = torch.from_numpy(((c64[:-1] + c64[1:]) / 2.0).astype(np.float32))
    return VHeadTables(head_dim=head_dim, bits=bits, seed=seed,
                       rotation=torch.from_numpy(v_rotation(head_dim, seed)),
                       centroids=cents, boundaries=edges,
                       lut_f16=cents.to(torch.float16))
