"""Generate the golden fixtures in this folder by running the reference.

Run once, in a container where the reference checkout is available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference [manager]

(a second argument, ``manager``, ``production``, ``prefill`` or the name of a layer-shaped case, regenerates only
that fixture; each has its own seed)

The reference's Triton kernels are executed by Triton's CPU interpreter
(``tl.dot`` is a float32 ``np.matmul`` there), so the vectors are the
reference's own encoder/decoder outputs without TF32 rounding.  The tests only
read the ``.npz`` files written here; they never import the reference.

Fixtures
  tables_<case>.npz   calibration inputs (or scores), bit map and every static table
  encode_<case>.npz   K/V rows -> packed bytes, norms, unpacked codes, nibble/mixed layouts
  decode_<case>.npz   packed cache + query -> attention output and LSE per KV head
  prefill.npz         packed cache + 24 queries at positions 40..63 -> causal prefill attention output
  manager.npz         BlockGTQKVManager: bulk encode + two append_and_attend steps, batch 2
  buffer_policy.npz   the reference's fp16 sink / recent-window flush policy, recorded from its own hook
  shape_<name>.npz    layer-shaped cases (8 KV heads, thousands of tokens): per-head bit maps, the packed cache
                      of every head and the decode output for one query past the end; the fp16 K/V inputs
                      are not stored but regenerated from the seed by ``helpers.synth_layer_case``
  production.npz      BlockGTQProductionCache (nibble/mixed layout): bulk encode + two decode steps, batch 1
"""
import hashlib
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path to a checkout of the reference> [manager|production|prefill]")
ref_path = sys.argv[1]
sys.path.insert(0, ref_path)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from blockgtq.quantizer import (  # noqa: E402
    BlockGTQQuantizer, build_batched_encode_args, compress_k_packed_batched,
    compress_v_packed_batched, compress_k_mixed_batched, compress_v_nibble4_batched)
from blockgtq.kernels.fused_packed_attention import (fused_blockgtq_decode_attention,  # noqa: E402
                                                     fused_blockgtq_prefill_attention)
from blockgtq.packed_kv_manager import BlockGTQKVManager  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
HD = 128
CPU = torch.device("cpu")


def sha(t):
    return hashlib.sha256(np.ascontiguousarray(t.numpy()).tobytes()).hexdigest()


def rope(x, pos, theta):
    """split-half RoPE on (..., T, hd) float32."""
    half = x.shape[-1] // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def synth_head(gen, n_k, gqa, theta=500000.0):
    """Keys/queries with lognormal per-block scales and two x8 outlier blocks, post-RoPE."""
    s = torch.exp(torch.randn(HD // 2, generator=gen))
    s[torch.randperm(HD // 2, generator=gen)[:2]] *= 8
    scale = torch.cat([s, s])
    pos = torch.arange(n_k)
    k = rope((torch.randn(n_k, HD, generator=gen) * scale).half().float(), pos, theta).half()
    q = rope((torch.randn(gqa, n_k, HD, generator=gen) * scale).half().float(), pos, theta).half()
    return q.reshape(-1, HD), k


CASES = {
    # name: (avg_bits, min_bits, max_bits, rotation_threshold, v_bits)
    "a3_1to6": (3.0, 1, 6, 2, 3),
    "a3_1to8": (3.0, 1, 8, 2, 3),
    "a2_1to8": (2.0, 1, 8, 2, 2),
    "a4_rt1": (4.0, 1, 8, 1, 4),
    "u3": (3.0, 3, 3, 2, 1),
}


def make_quantizers(case, n_kv, gen, n_cal=256, gqa=4):
    avg, mn, mx, rt, vb = CASES[case]
    qs, cal = [], []
    for hi in range(n_kv):
        q, k = synth_head(gen, n_cal, gqa)
        z = BlockGTQQuantizer(HD, avg_bits=avg, rotation_threshold=rt, min_bits=mn,
                              max_bits=mx, device=CPU)
        z.calibrate(q.float(), k.float())
        z.init_v_quantizer(v_bits=vb, seed=42 + hi)
        qs.append(z)
        cal.append((q, k))
    return qs, cal


def dump_tables(case, qs, cal):
    out = {"case": np.array(CASES[case], dtype=np.float64)}
    for hi, (z, (q, k)) in enumerate(zip(qs, cal)):
        p = f"h{hi}_"
        ka = z.build_kernel_args()
        from blockgtq.freq_analysis import compute_freq_importance_energy
        from blockgtq.rope_utils import decompose_freq_blocks
        sc = compute_freq_importance_energy(decompose_freq_blocks(q.float(), HD),
                                            decompose_freq_blocks(k.float(), HD))
        out[p + "scores"] = sc.numpy()
        if hi == 0:
            out[p + "cal_q"] = q.numpy()
            out[p + "cal_k"] = k.numpy()
            out[p + "rot_t"] = z._block_rot_T.numpy()
            out[p + "v_rot"] = z._v_quantizer.rotation.numpy()
        out[p + "rot_t_sha"] = np.array(sha(z._block_rot_T))
        out[p + "v_rot_sha"] = np.array(sha(z._v_quantizer.rotation))
        out[p + "alloc"] = z.bit_allocation.numpy()
        out[p + "head_perm"] = z._head_perm.numpy()
        out[p + "group_of"] = (z._group_of if z._group_of is not None
                               else torch.zeros(HD, dtype=torch.long)).numpy()
        out[p + "pos_centroids"] = z._pos_centroids.numpy()
        out[p + "pos_boundaries"] = z._pos_boundaries.numpy()
        out[p + "code_lut"] = z._code_lut.numpy()
        out[p + "pos_to_cb"] = z._pos_to_cb.numpy()
        out[p + "lut_off"] = z._lut_offsets.numpy()
        out[p + "lut_inv"] = z._lut_inv_scales.numpy()
        out[p + "segments"] = np.array(ka["segments_b"], dtype=np.int64)
        out[p + "codebook"] = ka["codebook_flat"].numpy()
        out[p + "total_packed_bytes"] = np.array(z._total_packed_bytes)
        pm = z._pack_meta
        out[p + "nopack"] = np.array([pm["nopack_start"], pm["nopack_len"], pm["nopack_off"]])
        out[p + "v_cents"] = z._v_quantizer.centroids.numpy()
        out[p + "v_bounds"] = z._v_quantizer.boundaries.numpy()
    np.savez_compressed(os.path.join(HERE, f"tables_{case}.npz"), **out)


def edge_rows(x, gen):
    """Overwrite a few rows with corner cases: zero, tiny, huge, single spike."""
    x = x.clone()
    x[:, 3] = 0
    x[:, 5] = (torch.randn(HD, generator=gen) * 1e-4).half()
    x[:, 7] = (torch.randn(HD, generator=gen) * 200).half()
    x[:, 9] = 0
    x[:, 9, 17] = 3.0
    return x


def dump_encode(case, qs, gen, n_rows=80):
    n_kv = len(qs)
    ba = build_batched_encode_args(qs, device="cpu")
    ks = []
    for hi in range(n_kv):
        _q, k = synth_head(gen, n_rows, 1)
        ks.append(k)
    k_flat = edge_rows(torch.stack(ks), gen).contiguous()
    v_flat = edge_rows(torch.randn(n_kv, n_rows, HD, generator=gen).half(), gen).contiguous()
    kp, kn = compress_k_packed_batched(k_flat, ba)
    vp, vn = compress_v_packed_batched(v_flat, ba)
    km, knc = compress_k_mixed_batched(k_flat, ba, norm_correct=True)
    vnib, vn2 = compress_v_nibble4_batched(v_flat, ba)
    codes = torch.stack([qs[hi].compress(k_flat[hi])[0] for hi in range(n_kv)])
    vcodes = torch.stack([qs[hi].compress_v(v_flat[hi])[0] for hi in range(n_kv)])
    np.savez_compressed(
        os.path.join(HERE, f"encode_{case}.npz"),
        k=k_flat.numpy(), v=v_flat.numpy(),
        k_packed=kp.numpy(), k_norms=kn.numpy(), k_codes=codes.numpy(),
        v_packed=vp.numpy(), v_norms=vn.numpy(), v_codes_torch=vcodes.numpy(),
        k_mixed=km.numpy(), k_norms_corrected=knc.numpy(),
        v_nibble=vnib.numpy(), v_norms_nibble=vn2.numpy(),
        max_tpb=np.array(ba["max_tpb"]), max_ng=np.array(ba["max_n_groups"]),
        max_mixed=np.array(ba["max_mixed_bytes"]))
    return ba


def dump_decode(case, qs, gen, T=333, B=2, gqa=4):
    """Bulk-encode a (B, n_kv, T) cache and run the reference decode per KV head."""
    n_kv = len(qs)
    ba = build_batched_encode_args(qs, device="cpu")
    ks, qn = [], []
    for b in range(B):
        row_k, row_q = [], []
        for hi in range(n_kv):
            q, k = synth_head(gen, T + 1, gqa)
            row_k.append(k[:T])
            row_q.append(q.reshape(gqa, T + 1, HD)[:, T])      # query at position T
        ks.append(torch.stack(row_k))
        qn.append(torch.cat(row_q))
    k = torch.stack(ks)                                      # (B, n_kv, T, hd)
    q = torch.stack(qn).unsqueeze(2)                         # (B, n_q, 1, hd)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half()
    k_flat = k.permute(1, 0, 2, 3).reshape(n_kv, B * T, HD).contiguous()
    v_flat = v.permute(1, 0, 2, 3).reshape(n_kv, B * T, HD).contiguous()
    kp, kn = compress_k_packed_batched(k_flat, ba)
    vp, vn = compress_v_packed_batched(v_flat, ba)
    kp = kp.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).contiguous()
    kn = kn.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).to(torch.float16).contiguous()
    vp = vp.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).contiguous()
    vn = vn.reshape(n_kv, B, T).permute(1, 0, 2).contiguous()
    t_splits = 1
    while t_splits < max(1, min((T + 63) // 64, 32)):
        t_splits *= 2
    outs, lses, qrots = [], [], []
    for hi in range(n_kv):
        z = qs[hi]
        ka = z.build_kernel_args()
        q_h = q[:, hi * gqa:(hi + 1) * gqa]
        q_rot = z.rotate_q_for_packed_kernel(q_h.reshape(-1, HD)).reshape(q_h.shape)
        o, lse = fused_blockgtq_decode_attention(
            q_rot, kp[:, hi:hi + 1], kn[:, hi:hi + 1], ka["codebook_flat"], ka["lut_offset"],
            ka["norm_group"], ka["segments_b"], vp[:, hi:hi + 1], vn[:, hi:hi + 1], z.v_lut,
            scale=1.0 / HD ** 0.5, t_splits=t_splits, v_bits=z.v_bits,
            v_rotation=z._v_rot, return_lse=True)
        outs.append(o)
        lses.append(lse)
        qrots.append(q_rot)
    np.savez_compressed(
        os.path.join(HERE, f"decode_{case}.npz"),
        q=q.numpy(), q_rot=torch.cat(qrots, dim=1).numpy(),
        k_packed=kp.numpy(), k_norms=kn.numpy(), v_packed=vp.numpy(), v_norms=vn.numpy(),
        out=torch.cat(outs, dim=1).numpy(), lse=torch.cat(lses, dim=1).numpy(),
        t_splits=np.array(t_splits), gqa=np.array(gqa))


def dump_manager(gen, T0=150, B=2, n_kv=2, gqa=2, steps=2):
    """Whole-class run: calibrate one layer, bulk encode, then decode steps."""
    n_q = n_kv * gqa
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=T0 + steps + 2, batch_size=B,
                            k_avg_bits=3.0, v_bits=3, device="cpu")
    cq, ck = [], []
    for hi in range(n_kv):
        q, k = synth_head(gen, 256, gqa)
        cq.append(q)
        ck.append(k)
    cq, ck = torch.stack(cq).float(), torch.stack(ck).float()
    mgr.calibrate(0, cq, ck)
    k0 = torch.stack([torch.stack([synth_head(gen, T0, 1)[1] for _ in range(n_kv)])
                      for _ in range(B)])
    v0 = torch.randn(B, n_kv, T0, HD, generator=gen).half()
    mgr._encode_kv(0, k0, v0, 0, T0)
    mgr.seq_len = T0
    rec = {"cal_q": cq.numpy(), "cal_k": ck.numpy(), "k_init": k0.numpy(), "v_init": v0.numpy()}
    for s in range(steps):
        q = (torch.randn(B, n_q, 1, HD, generator=gen) * 2).half()
        kn = torch.stack([torch.stack([synth_head(gen, 1, 1)[1] for _ in range(n_kv)])
                          for _ in range(B)])
        vn = torch.randn(B, n_kv, 1, HD, generator=gen).half()
        out = mgr.append_and_attend(0, q, kn, vn)
        mgr.increment_seq_len()
        rec[f"q{s}"], rec[f"k{s}"], rec[f"v{s}"], rec[f"out{s}"] = (
            q.numpy(), kn.numpy(), vn.numpy(), out.numpy())
    T = mgr.seq_len
    rec["k_packed"] = mgr._k_packed[:, :, :, :T].numpy()
    rec["k_norms"] = mgr._k_norms[:, :, :, :T].numpy()
    rec["v_packed"] = mgr._v_packed[:, :, :, :T].numpy()
    rec["v_norms"] = mgr._v_norms[:, :, :, :T].numpy()
    rec["alloc"] = np.stack([mgr.quantizers[0][h].bit_allocation.numpy() for h in range(n_kv)])
    np.savez_compressed(os.path.join(HERE, "manager.npz"), **rec)


def dump_production(gen, T0=150, n_kv=2, gqa=4, steps=2):
    """BlockGTQProductionCache (nibble/mixed layout, batch 1): bulk encode + decode steps.  The T=1 encode
    goes through the batched encoder instead of the CUDA-graph replay (same kernels, no GPU needed)."""
    from blockgtq.production_cache import BlockGTQProductionCache
    n_q = n_kv * gqa
    qs, cal = make_quantizers("a3_1to8", n_kv, gen, gqa=gqa)
    ba = [build_batched_encode_args(qs, device="cpu")]
    ka = [[z.build_kernel_args() for z in qs]]
    cache = BlockGTQProductionCache([qs], ba, ka, 1, n_kv, n_q, HD, T0 + steps + 2, v_bits=3, device="cpu")
    cache._encode_graphed = lambda li, k, v, t: cache._encode_batched(li, k, v, t)
    k0 = torch.stack([synth_head(gen, T0, 1)[1] for _ in range(n_kv)]).unsqueeze(0)
    v0 = torch.randn(1, n_kv, T0, HD, generator=gen).half()
    cache._encode_batched(0, k0, v0, 0)
    cache.seq_len = T0
    rec = {"alloc": np.stack([z.bit_allocation.numpy() for z in qs]), "k_init": k0.numpy(), "v_init": v0.numpy()}
    for s in range(steps):
        q = (torch.randn(1, n_q, 1, HD, generator=gen) * 2).half()
        kn = torch.stack([synth_head(gen, 1, 1)[1] for _ in range(n_kv)]).unsqueeze(0)
        vn = torch.randn(1, n_kv, 1, HD, generator=gen).half()
        out = cache.encode_and_attend(0, q, kn, vn)
        cache.increment_seq_len()
        rec[f"q{s}"], rec[f"k{s}"], rec[f"v{s}"], rec[f"out{s}"] = q.numpy(), kn.numpy(), vn.numpy(), out.numpy()
    T = cache.seq_len
    rec["k_packed"] = cache.k_packed[:, :, :, :T].numpy()
    rec["k_norms"] = cache.k_norms[:, :, :, :T].numpy()
    rec["v_packed"] = cache.v_packed[:, :, :, :T].numpy()
    rec["v_norms"] = cache.v_norms[:, :, :, :T].numpy()
    np.savez_compressed(os.path.join(HERE, "production.npz"), **rec)


def dump_prefill(gen, case="a3_1to8", S_q=24, offset=40, B=2, n_kv=2, gqa=4):
    """Causal prefill attention of S_q queries at positions offset .. offset+S_q-1 over a packed cache of
    offset+S_q tokens, through the reference's prefill kernel, per KV head.  Self-contained fixture: its own
    bit allocations, cache and outputs."""
    qs, _cal = make_quantizers(case, n_kv, gen, gqa=gqa)
    ba = build_batched_encode_args(qs, device="cpu")
    T = offset + S_q
    ks, qn = [], []
    for b in range(B):
        row_k, row_q = [], []
        for hi in range(n_kv):
            q, k = synth_head(gen, T, gqa)
            row_k.append(k)
            row_q.append(q.reshape(gqa, T, HD)[:, offset:])
        ks.append(torch.stack(row_k))
        qn.append(torch.cat(row_q))
    k = torch.stack(ks)                                      # (B, n_kv, T, hd)
    q = torch.stack(qn)                                      # (B, n_q, S_q, hd)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half()
    k_flat = k.permute(1, 0, 2, 3).reshape(n_kv, B * T, HD).contiguous()
    v_flat = v.permute(1, 0, 2, 3).reshape(n_kv, B * T, HD).contiguous()
    kp, kn = compress_k_packed_batched(k_flat, ba)
    vp, vn = compress_v_packed_batched(v_flat, ba)
    kp = kp.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).contiguous()
    kn = kn.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).to(torch.float16).contiguous()
    vp = vp.reshape(n_kv, B, T, -1).permute(1, 0, 2, 3).contiguous()
    vn = vn.reshape(n_kv, B, T).permute(1, 0, 2).contiguous()
    outs, qrots = [], []
    for hi in range(n_kv):
        z = qs[hi]
        ka = z.build_kernel_args()
        q_h = q[:, hi * gqa:(hi + 1) * gqa]
        q_rot = z.rotate_q_for_packed_kernel(q_h.reshape(-1, HD)).reshape(q_h.shape)
        o = fused_blockgtq_prefill_attention(
            q_rot, kp[:, hi:hi + 1], kn[:, hi:hi + 1], ka["codebook_flat"], ka["lut_offset"], ka["norm_group"],
            ka["segments_b"], vp[:, hi:hi + 1], vn[:, hi:hi + 1], z.v_lut, scale=1.0 / HD ** 0.5,
            block_q=32, block_t=64, v_bits=z.v_bits, v_rotation=z._v_rot, is_causal=True, q_pos_offset=offset)
        outs.append(o)
        qrots.append(q_rot)
    rec = dict(q=q.numpy(), q_rot=torch.cat(qrots, dim=1).numpy(), k_packed=kp.numpy(), k_norms=kn.numpy(),
               v_packed=vp.numpy(), v_norms=vn.numpy(), out=torch.cat(outs, dim=1).numpy(),
               offset=np.array(offset), gqa=np.array(gqa), case=np.array(case))
    for hi, z in enumerate(qs):
        rec[f"h{hi}_alloc"] = z.bit_allocation.cpu().numpy()
    np.savez_compressed(os.path.join(HERE, "prefill.npz"), **rec)


SHAPE_CASES = {
    # name: (avg_bits, min_bits, max_bits, v_bits, n_kv, gqa, T, theta, seed)
    # one layer of the single-layer op configuration: 32 query / 8 KV heads, context 4096, avg 3.0 in [1, 6], V 3-bit
    "cfg0_a3_1to6_h8_t4096": (3.0, 1, 6, 3, 8, 4, 4096, 500000.0, 0),
    # an 8-head K2V2 layer (avg 2.0 in [1, 8], V 2-bit)
    "k2v2_h8_t2048": (2.0, 1, 8, 2, 8, 4, 2048, 500000.0, 1),
}


def dump_shape_case(name):
    """One decode query at position T over a T-token cache of one whole layer (batch 1, every KV head), all of
    it through the reference: calibration per head on the head's own queries and keys, batched encoders,
    per-head decode kernel with the reference's split rule."""
    sys.path.insert(0, os.path.dirname(HERE))
    from helpers import synth_layer_case
    avg, mn, mx, vb, n_kv, gqa, T, theta, seed = SHAPE_CASES[name]
    data = synth_layer_case(seed, n_kv, gqa, T, theta)
    qs = []
    for hi in range(n_kv):
        z = BlockGTQQuantizer(HD, avg_bits=avg, min_bits=mn, max_bits=mx, rope_base=theta, device=CPU)
        z.calibrate(data["q_all"][hi][:, :T].reshape(-1, HD).float(), data["k"][hi].float())
        z.init_v_quantizer(v_bits=vb, seed=42 + hi)
        qs.append(z)
        print("calibrated", hi, flush=True)
    ba = build_batched_encode_args(qs, device="cpu")
    kp, kn = compress_k_packed_batched(data["k"].contiguous(), ba)
    print("K encoded", flush=True)
    vp, vn = compress_v_packed_batched(data["v"].contiguous(), ba)
    print("V encoded", flush=True)
    kp, kn = kp.unsqueeze(0), kn.to(torch.float16).unsqueeze(0)       # (1, n_kv, T, ...)
    vp, vn = vp.unsqueeze(0), vn.unsqueeze(0)
    q = data["q"].unsqueeze(0).unsqueeze(2)                            # (1, n_q, 1, hd)
    t_splits = 1
    while t_splits < max(1, min((T + 63) // 64, 32)):
        t_splits *= 2
    outs, lses, qrots = [], [], []
    for hi in range(n_kv):
        z = qs[hi]
        ka = z.build_kernel_args()
        q_h = q[:, hi * gqa:(hi + 1) * gqa]
        q_rot = z.rotate_q_for_packed_kernel(q_h.reshape(-1, HD)).reshape(q_h.shape)
        o, lse = fused_blockgtq_decode_attention(
            q_rot, kp[:, hi:hi + 1], kn[:, hi:hi + 1], ka["codebook_flat"], ka["lut_offset"],
            ka["norm_group"], ka["segments_b"], vp[:, hi:hi + 1], vn[:, hi:hi + 1], z.v_lut,
            scale=1.0 / HD ** 0.5, t_splits=t_splits, v_bits=z.v_bits,
            v_rotation=z._v_rot, return_lse=True)
        outs.append(o)
        lses.append(lse)
        qrots.append(q_rot)
        print("decoded", hi, flush=True)
    np.savez_compressed(
        os.path.join(HERE, f"shape_{name}.npz"),
        case=np.array(SHAPE_CASES[name], dtype=np.float64),
        alloc=np.stack([z.bit_allocation.numpy() for z in qs]),
        input_sha=np.array(sha(torch.cat([data["k"].reshape(-1), data["v"].reshape(-1), data["q"].reshape(-1)]))),
        q=q.numpy(), q_rot=torch.cat(qrots, dim=1).numpy(),
        k_packed=kp.numpy(), k_norms=kn.numpy(), v_packed=vp.numpy(), v_norms=vn.numpy(),
        out=torch.cat(outs, dim=1).numpy(), lse=torch.cat(lses, dim=1).numpy(), t_splits=np.array(t_splits))


BUFFER_SETTINGS = [(4, 128, 1), (0, 16, 1), (4, 32, 8), (2, 0, 4)]     # (n_sink, recent_window, block_size)


def dump_buffer_policy(n_steps=300, prefill=37):
    """The three-region flush policy as the reference executes it: its _BufferedKVPatch hook
    (blockgtq/unaccelerated.py:163-244) is driven with a stub model and a fake ``past_key_values`` whose
    caches grow by a prefill and then one token per forward; ``_flush`` is replaced by a recorder.  Stored per
    setting: the sequence length after every forward, the packed-token count (n_flushed) after it, and every
    (start, end) flush call."""
    import types
    from blockgtq.unaccelerated import _BufferedKVPatch
    rec = {"settings": np.array(BUFFER_SETTINGS, dtype=np.int64)}
    for si, (n_sink, window, bs) in enumerate(BUFFER_SETTINGS):
        stub = torch.nn.Identity()
        patch = _BufferedKVPatch(stub, None, None, HD, 1, 1, block_size=bs, recent_window=window, n_sink_token=n_sink)
        calls = []
        patch._flush = lambda k, v, li, start, end, calls=calls: calls.append((start, end))
        seqs, flushed, call_step = [], [], []
        seq = 0
        for step in range(n_steps):
            seq += prefill if step == 0 else 1
            pkv = types.SimpleNamespace(key_cache=[torch.zeros(1, 1, seq, HD)], value_cache=[torch.zeros(1, 1, seq, HD)])
            n_before = len(calls)
            patch._hook_fn(stub, (), {"past_key_values": pkv}, None)
            seqs.append(seq)
            flushed.append(patch.state[0]["n_flushed"])
            call_step += [step] * (len(calls) - n_before)
        patch.remove()
        rec[f"s{si}_seq"] = np.array(seqs, dtype=np.int64)
        rec[f"s{si}_n_flushed"] = np.array(flushed, dtype=np.int64)
        rec[f"s{si}_flush_calls"] = np.array(calls, dtype=np.int64).reshape(-1, 2)
        rec[f"s{si}_flush_step"] = np.array(call_step, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "buffer_policy.npz"), **rec)


def main():
    only = sys.argv[2] if len(sys.argv) > 2 else None
    if only == "buffer_policy":
        dump_buffer_policy()
        print("done buffer_policy")
        return
    if only in SHAPE_CASES:
        dump_shape_case(only)
        print("done", only)
        return
    gen = torch.Generator().manual_seed(20240607)
    for case in CASES:
        if only is not None:
            break
        qs, cal = make_quantizers(case, 2, gen)
        dump_tables(case, qs, cal)
        dump_encode(case, qs, gen)
        if case in ("a3_1to6", "a3_1to8", "a2_1to8", "a4_rt1"):
            dump_decode(case, qs, gen)
        print("done", case, flush=True)
    if only in (None, "manager"):
        dump_manager(torch.Generator().manual_seed(777))
        print("done manager")
    if only in (None, "production"):
        dump_production(torch.Generator().manual_seed(778))
        print("done production")
    if only in (None, "prefill"):
        dump_prefill(torch.Generator().manual_seed(779))
        print("done prefill")


if __name__ == "__main__":
    main()
