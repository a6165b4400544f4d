"""CPU restatement of Block-GTQ's packed-cache hot path in NumPy.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module: it is the checker for the CUDA kernels (tests, the smoke check and the
CPU-baseline leg of the benchmark), never a fallback.

Parity pin: the functions below are checked against vectors produced by the
reference's own encoder and decoder (its Triton kernels executed by Triton's
CPU interpreter, where ``tl.dot`` is a float32 ``np.matmul``); the vectors and
the script that generated them live in ``tests/golden/``.  The reference ships
no tests or known-answer vectors of its own.

Every function takes plain NumPy arrays.  ``meta`` is a dict with the static
tables of one KV head:

    head_perm (hd,) int      packed position -> original dim
    group_of  (hd,) int      packed position -> norm group
    n_groups  int
    rot_t     (hd,hd) f32    y = x_unit[perm] @ rot_t
    code_lut  (G,256) u8     uniform bin -> code, per group
    pos_to_cb (hd,) int
    lut_off, lut_inv (hd,) f32
    segments  [(bw, start, len, pack_off, lut_off, norm_idx)]
    row_bytes int            packed K bytes per token of this head
    codebook  (sum 2**bw,) f16
    v_bits int, v_rot (hd,hd) f32 (y = R @ v_unit), v_bounds, v_cents f32
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
F16 = np.float16


# ---------------------------------------------------------------------------
# bit packing (quantizer.py:861-990, v_packing.py:31-109)
# ---------------------------------------------------------------------------

def seg_bytes(bw: int, n: int) -> int:
    if bw == 1:
        return (n + 7) // 8
    if bw == 2:
        return (n + 3) // 4
    if bw == 3:
        return ((n + 7) // 8) * 3
    if bw == 4:
        return (n + 1) // 2
    return n


def pack_run(codes: np.ndarray, bw: int) -> np.ndarray:
    """Pack ``codes`` (N, n) of one width into (N, seg_bytes) bytes.

    Widths 1-4: code ``i`` occupies bits ``[i*bw, (i+1)*bw)`` of an LSB-first
    stream (for 3 bits this is exactly the 8-codes-in-3-bytes group layout of
    quantizer.py:957-959, the last group zero filled).  Widths 5-8: raw bytes.
    """
    n_rows, n = codes.shape
    if bw >= 5:
        return codes.astype(np.uint8)
    nb = seg_bytes(bw, n)
    c = (codes.astype(np.uint64) & np.uint64((1 << bw) - 1))
    out = np.zeros((n_rows, nb), dtype=np.uint8)
    for i in range(n):
        bit = i * bw
        byte, sh = bit >> 3, bit & 7
        v = c[:, i] << np.uint64(sh)
        out[:, byte] |= (v & np.uint64(0xFF)).astype(np.uint8)
        if sh + bw > 8:
            out[:, byte + 1] |= ((v >> np.uint64(8)) & np.uint64(0xFF)).astype(np.uint8)
    return out


def unpack_run(packed: np.ndarray, bw: int, n: int) -> np.ndarray:
    """Inverse of :func:`pack_run` (decode side: fused_packed_attention.py:1170-1372)."""
    if bw >= 5:
        return packed[:, :n].astype(np.uint8)
    p = packed.astype(np.uint32)
    p = np.concatenate([p, np.zeros((p.shape[0], 1), np.uint32)], axis=1)
    out = np.empty((packed.shape[0], n), dtype=np.uint8)
    for i in range(n):
        bit = i * bw
        byte, sh = bit >> 3, bit & 7
        word = p[:, byte] | (p[:, byte + 1] << 8)
        out[:, i] = ((word >> sh) & ((1 << bw) - 1)).astype(np.uint8)
    return out


def pack_k(codes: np.ndarray, segments, row_bytes: int) -> np.ndarray:
    """codes (N, hd) in packed-dim order -> (N, row_bytes); unused tail bytes 0."""
    out = np.zeros((codes.shape[0], row_bytes), dtype=np.uint8)
    for bw, start, length, off, _lo, _ni in segments:
        out[:, off:off + seg_bytes(bw, length)] = pack_run(codes[:, start:start + length], bw)
    return out


def unpack_k(packed: np.ndarray, segments, hd: int) -> np.ndarray:
    out = np.zeros((packed.shape[0], hd), dtype=np.uint8)
    for bw, start, length, off, _lo, _ni in segments:
        out[:, start:start + length] = unpack_run(packed[:, off:off + seg_bytes(bw, length)], bw, length)
    return out


def pack_v(codes: np.ndarray, bits: int) -> np.ndarray:
    return pack_run(codes, bits)


def unpack_v(packed: np.ndarray, bits: int, hd: int) -> np.ndarray:
    return unpack_run(packed, bits, hd)


def pack_k_mixed(codes: np.ndarray, nopack_start: int, nopack_len: int, row_bytes: int) -> np.ndarray:
    """Production layout (quantizer.py:1930-1951): nibble pairs for the dims
    before ``nopack_start`` then one raw byte per 5-8-bit dim."""
    out = np.zeros((codes.shape[0], row_bytes), dtype=np.uint8)
    nb = nopack_start // 2
    if nopack_start > 0:
        lo = codes[:, 0:nopack_start:2] & 0xF
        hi = codes[:, 1:nopack_start:2] & 0xF
        out[:, :nb] = lo | (hi << 4)
    if nopack_len > 0:
        out[:, nb:nb + nopack_len] = codes[:, nopack_start:nopack_start + nopack_len]
    return out


def pack_nibble4(codes: np.ndarray) -> np.ndarray:
    """byte[i] = code[2i] | code[2i+1] << 4 (quantizer.py:2096-2099)."""
    return ((codes[:, 0::2] & 0xF) | ((codes[:, 1::2] & 0xF) << 4)).astype(np.uint8)


# ---------------------------------------------------------------------------
# K encoder (quantizer.py:800-850; unpacked codes = quant_kernels.py:508-565)
# ---------------------------------------------------------------------------

def encode_k(x16: np.ndarray, meta: dict, *, dtype=F32):
    """Quantise keys.  x16: (N, hd) float16.

    Returns dict: codes (N,hd) u8 in packed order, norms (N,G) float32,
    u (N,hd) bin coordinate before truncation (``dtype`` precision),
    fragile (N,hd) bool -- True where ``u`` is within 2e-3 of a bin edge at
    which the code changes, i.e. where a float32 evaluation with another
    summation order may legitimately land on the neighbouring code.
    """
    perm = np.asarray(meta["head_perm"])
    grp = np.asarray(meta["group_of"])
    G = int(meta["n_groups"])
    x = x16.astype(dtype)[:, perm]
    onehot = (grp[None, :] == np.arange(G)[:, None]).astype(dtype)        # (G, hd)
    gsq = (x * x) @ onehot.T                                               # (N, G)
    gnorm = np.sqrt(gsq + dtype(1e-30))
    per_pos = gnorm[:, grp]
    safe = np.where(per_pos > dtype(1e-10), per_pos, dtype(1.0))
    y = (x / safe) @ np.asarray(meta["rot_t"]).astype(dtype)
    u = (y - np.asarray(meta["lut_off"]).astype(dtype)[None, :]) * \
        np.asarray(meta["lut_inv"]).astype(dtype)[None, :]
    uc = np.minimum(np.maximum(u, dtype(0.0)), dtype(255.0))
    b = uc.astype(np.int32)                                                # trunc toward zero
    lut = np.asarray(meta["code_lut"])
    cb = np.asarray(meta["pos_to_cb"]).astype(np.int64)
    codes = lut[cb[None, :], b]
    # fragile: nearest interior edge e in 1..255 with lut[e-1] != lut[e]
    e = np.clip(np.rint(u).astype(np.int32), 1, 255)
    changes = lut[cb[None, :], e - 1] != lut[cb[None, :], e]
    fragile = changes & (np.abs(u - e) < 2e-3)
    return {"codes": codes.astype(np.uint8), "norms": gnorm.astype(F32), "u": u, "fragile": fragile}


def encode_k_packed(x16, meta, row_bytes=None):
    r = encode_k(x16, meta)
    rb = int(row_bytes if row_bytes is not None else meta["row_bytes"])
    r["packed"] = pack_k(r["codes"], meta["segments"], rb)
    return r


def k_yhat_group_norms(codes: np.ndarray, meta: dict) -> np.ndarray:
    """||centroid[code]|| per norm group, float32 -- the divisor of the
    production layout's norm correction (quantizer.py:1956-1974)."""
    pc = np.asarray(meta["pos_centroids"]).astype(F32)                    # (hd, maxnc)
    grp = np.asarray(meta["group_of"])
    G = int(meta["n_groups"])
    cv = pc[np.arange(pc.shape[0])[None, :], codes.astype(np.int64)]
    onehot = (grp[None, :] == np.arange(G)[:, None]).astype(F32)
    return np.maximum(np.sqrt((cv * cv) @ onehot.T), F32(1e-10))


# ---------------------------------------------------------------------------
# V encoder (quantizer.py:560-590)
# ---------------------------------------------------------------------------

def encode_v(v16: np.ndarray, meta: dict, *, dtype=F32):
    x = v16.astype(dtype)
    raw = np.sqrt((x * x).sum(axis=1) + dtype(1e-30))
    safe = np.where(raw > dtype(1e-8), raw, dtype(1.0))
    y = (x / safe[:, None]) @ np.asarray(meta["v_rot"]).astype(dtype).T
    bounds = np.asarray(meta["v_bounds"]).astype(dtype)
    codes = (y[:, :, None] > bounds[None, None, :]).sum(axis=2).astype(np.uint8)
    cents = np.asarray(meta["v_cents"]).astype(dtype)
    cn = np.sqrt((cents[codes] ** 2).sum(axis=1) + dtype(1e-20))
    cn = np.where(cn > dtype(1e-10), cn, dtype(1.0))
    norms = (raw / cn).astype(F32).astype(F16)
    dist = np.abs(y[:, :, None] - bounds[None, None, :]).min(axis=2)
    return {"codes": codes, "norms": norms, "y": y, "fragile": dist < 1e-6,
            "packed": pack_v(codes, int(meta["v_bits"]))}


# ---------------------------------------------------------------------------
# query preparation (quantizer.py:1160-1187)
# ---------------------------------------------------------------------------

def rotate_q(q16: np.ndarray, meta: dict) -> np.ndarray:
    """q (..., hd) f16 -> f16 query in packed-dim order, rotated like K."""
    q = q16.astype(F32)[..., np.asarray(meta["head_perm"])]
    return (q @ np.asarray(meta["rot_t"]).astype(F32)).astype(F16)


# ---------------------------------------------------------------------------
# decode attention over the packed cache (fused_packed_attention.py:283-894)
# ---------------------------------------------------------------------------

def dequant_k(packed: np.ndarray, k_norms16: np.ndarray, meta: dict, dtype=np.float64):
    """(T, row_bytes) u8 + (T, G) f16 -> (T, hd) keys in rotated packed-dim order."""
    hd = len(meta["head_perm"])
    codes = unpack_k(packed, meta["segments"], hd).astype(np.int64)
    cbk = np.asarray(meta["codebook"]).astype(dtype)
    out = np.zeros((packed.shape[0], hd), dtype=dtype)
    for bw, start, length, _off, lut_off, ni in meta["segments"]:
        out[:, start:start + length] = cbk[lut_off + codes[:, start:start + length]] * \
            k_norms16[:, ni].astype(dtype)[:, None]
    return out


def dequant_v(packed: np.ndarray, v_norms16: np.ndarray, meta: dict, *, f16_product: bool):
    """(T, vb) u8 + (T,) f16 -> (T, hd) values in V's rotated space (float64).

    ``f16_product`` rounds centroid*norm to float16 as the reference kernel
    does (fused_packed_attention.py:861-868)."""
    hd = len(meta["head_perm"])
    codes = unpack_v(packed, int(meta["v_bits"]), hd).astype(np.int64)
    c16 = np.asarray(meta["v_cents"]).astype(F32).astype(F16)
    if f16_product:
        return (c16[codes] * v_norms16.astype(F16)[:, None]).astype(np.float64)
    return c16[codes].astype(np.float64) * v_norms16.astype(np.float64)[:, None]


def attend_packed(q_rot16: np.ndarray, k_packed, k_norms16, v_packed, v_norms16, meta,
                  scale: float, *, unrotate: bool = True, f16_product: bool = True):
    """One KV head, float64 softmax.  q_rot16: (gqa, hd) f16 from :func:`rotate_q`.

    Returns (out (gqa, hd) float64, lse (gqa,) float64).  ``out`` is in the
    original V basis when ``unrotate`` (out_rot @ R, fused_packed_attention.py:877-882).
    An empty cache returns zeros and lse = -inf.
    """
    gqa, hd = q_rot16.shape
    if k_packed.shape[0] == 0:
        return np.zeros((gqa, hd)), np.full((gqa,), -np.inf)
    kh = dequant_k(k_packed, k_norms16, meta)
    vh = dequant_v(v_packed, v_norms16, meta, f16_product=f16_product)
    s = (q_rot16.astype(np.float64) @ kh.T) * scale
    m = s.max(axis=1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(axis=1, keepdims=True)
    o = (p @ vh) / l
    if unrotate:
        o = o @ np.asarray(meta["v_rot"]).astype(np.float64)
    return o, (m + np.log(l))[:, 0]


def attend_packed_mirror(q_rot16, k_packed, k_norms16, v_packed, v_norms16, meta, scale,
                         *, t_splits: int, block_t: int = 64, unrotate: bool = True):
    """Same attention with the reference kernel's rounding points: float32
    logits and running softmax per ``block_t`` tile, float16 ``p`` and
    float16 ``centroid*norm`` into a float32 accumulator, float16 per-split
    partial outputs merged in float32 and stored as float16
    (fused_packed_attention.py:257-283, 770-894, 59-103)."""
    gqa, hd = q_rot16.shape
    T = k_packed.shape[0]
    kh = dequant_k(k_packed, k_norms16, meta, dtype=F32)
    vh = dequant_v(v_packed, v_norms16, meta, f16_product=True).astype(F32)
    q = q_rot16.astype(F32)
    R = np.asarray(meta["v_rot"]).astype(F32)
    chunk = (T + t_splits - 1) // t_splits
    po = np.zeros((t_splits, gqa, hd), dtype=F16)
    pl = np.full((t_splits, gqa), -np.inf, dtype=F32)
    for c in range(t_splits):
        t0, t1 = c * chunk, min((c + 1) * chunk, T)
        m = np.full((gqa,), -np.inf, dtype=F32)
        l = np.zeros((gqa,), dtype=F32)
        acc = np.zeros((gqa, hd), dtype=F32)
        for b0 in range(t0, t1, block_t):
            b1 = min(b0 + block_t, t1)
            s = (q @ kh[b0:b1].T) * F32(scale)
            m_new = np.maximum(m, s.max(axis=1))
            alpha = np.exp(m - m_new)
            p = np.exp(s - m_new[:, None]).astype(F32)
            l = alpha * l + p.sum(axis=1)
            acc = acc * alpha[:, None] + p.astype(F16).astype(F32) @ vh[b0:b1]
            m = m_new
        if t1 <= t0:
            continue                      # the reference never schedules an empty split
        o = acc / l[:, None]
        if unrotate:
            o = o @ R
        po[c] = o.astype(F16)
        pl[c] = m + np.log(l)
    out = combine(po.astype(F32), pl)[0].astype(F16)
    lse = np.logaddexp.reduce(pl.astype(np.float64), axis=0)
    return out, lse


# ---------------------------------------------------------------------------
# split merge (fused_packed_attention.py:59-103, 1856-1860)
# ---------------------------------------------------------------------------

def combine(part_o: np.ndarray, part_lse: np.ndarray):
    """part_o (S, rows, hd), part_lse (S, rows) -> (out (rows, hd), lse (rows,)).

    Splits with lse = -inf (no tokens) are ignored; if every split is empty
    the row is zero with lse = -inf."""
    lse = part_lse.astype(np.float64)
    m = lse.max(axis=0)
    m_safe = np.where(np.isfinite(m), m, 0.0)
    a = np.where(np.isfinite(lse), np.exp(lse - m_safe[None, :]), 0.0)
    den = a.sum(axis=0)
    o = np.where(np.isfinite(lse)[:, :, None], part_o.astype(np.float64), 0.0)
    num = (a[:, :, None] * o).sum(axis=0)
    out = np.where(den[:, None] > 0, num / np.where(den > 0, den, 1.0)[:, None], 0.0)
    with np.errstate(divide="ignore"):
        tot = np.where(den > 0, m_safe + np.log(np.where(den > 0, den, 1.0)), -np.inf)
    return out, tot


# ---------------------------------------------------------------------------
# fp16 sink / recent-window region (semantics: unaccelerated.py:163-244)
# ---------------------------------------------------------------------------

def attend_fp16(q16: np.ndarray, k16: np.ndarray, v16: np.ndarray, scale: float):
    """Plain attention of (gqa, hd) queries over fp16 tokens held unquantised.
    q is the *original* query (no permutation or rotation).  Returns
    (out (gqa, hd) float64 in the original V basis, lse (gqa,))."""
    gqa, hd = q16.shape
    if k16.shape[0] == 0:
        return np.zeros((gqa, hd)), np.full((gqa,), -np.inf)
    s = (q16.astype(np.float64) @ k16.astype(np.float64).T) * scale
    m = s.max(axis=1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(axis=1, keepdims=True)
    return (p @ v16.astype(np.float64)) / l, (m + np.log(l))[:, 0]


def three_region_plan(seq_len: int, n_sink: int, recent_window: int, block_size: int = 1):
    """How many tokens sit in each region after ``seq_len`` tokens were
    appended one at a time under the flush rule of unaccelerated.py:226-233:
    returns (n_sink_tokens, n_quantised, n_recent)."""
    sink = min(seq_len, n_sink)
    avail = max(0, seq_len - n_sink)
    flushed = 0
    need = block_size + recent_window
    if avail >= need:
        flushed = ((avail - need) // block_size + 1) * block_size
    return sink, flushed, avail - flushed
