"""Shared helpers for the test suite: fixture loading, oracle meta dicts, synthetic data."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from blockgtq_b200 import calib  # noqa: E402

HD = 128
CASES = {
    "a3_1to6": (3.0, 1, 6, 2, 3),
    "a3_1to8": (3.0, 1, 8, 2, 3),
    "a2_1to8": (2.0, 1, 8, 2, 2),
    "a4_rt1": (4.0, 1, 8, 1, 4),
    "u3": (3.0, 3, 3, 2, 1),
}


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def tables_for(case, hi, gold=None):
    """Product-built tables for head ``hi`` of a golden case (bit map from the fixture)."""
    gold = gold if gold is not None else load("tables_" + case)
    avg, mn, mx, rt, vb = CASES[case]
    kt = calib.build_k_tables(None, None, head_dim=HD, avg_bits=avg, rotation_threshold=rt,
                              min_bits=mn, max_bits=mx,
                              bit_allocation=torch.from_numpy(gold[f"h{hi}_alloc"]))
    vt = calib.build_v_tables(HD, vb, 42 + hi)
    return kt, vt


def oracle_meta(kt, vt, row_bytes=None):
    """Dict of NumPy tables in the form oracle/bgtq_oracle.py expects."""
    return {
        "head_perm": kt.head_perm.numpy(), "group_of": kt.group_of.numpy(),
        "n_groups": kt.n_groups, "rot_t": kt.block_rot.T.contiguous().numpy(),
        "code_lut": kt.code_lut.numpy(), "pos_to_cb": kt.pos_to_cb.numpy(),
        "lut_off": kt.lut_offsets.numpy(), "lut_inv": kt.lut_inv_scales.numpy(),
        "segments": kt.segments, "row_bytes": row_bytes or kt.total_packed_bytes,
        "codebook": kt.codebook_flat.numpy(), "pos_centroids": kt.pos_centroids.numpy(),
        "v_bits": vt.bits, "v_rot": vt.rotation.numpy(), "v_bounds": vt.boundaries.numpy(),
        "v_cents": vt.centroids.numpy(),
    }


def rope(x, pos, theta):
    half = x.shape[-1] // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def synth_head(gen, n_k, gqa, theta=500000.0, hd=HD):
    """Post-RoPE keys (n_k, hd) and queries (gqa*n_k, hd), fp16: N(0,1) times a
    lognormal(0,1) per-block scale with two blocks scaled x8."""
    s = torch.exp(torch.randn(hd // 2, generator=gen))
    s[torch.randperm(hd // 2, generator=gen)[:2]] *= 8
    scale = torch.cat([s, s])
    pos = torch.arange(n_k)
    k = rope((torch.randn(n_k, hd, generator=gen) * scale).half().float(), pos, theta).half()
    q = rope((torch.randn(gqa, n_k, hd, generator=gen) * scale).half().float(), pos, theta).half()
    return q.reshape(-1, hd), k


def synth_layer_case(seed, n_kv, gqa, T, theta):
    """Inputs of a layer-shaped golden case, regenerated from the seed alone (the fixture stores only their
    hash): per KV head post-RoPE keys (T, hd) and queries of its ``gqa`` heads at positions 0..T (the last one
    is the decode query), values N(0,1).  Returns fp16 tensors ``k`` (n_kv, T, hd), ``v`` (n_kv, T, hd),
    ``q`` (n_kv*gqa, hd) and ``q_all`` (n_kv, gqa, T+1, hd)."""
    gen = torch.Generator().manual_seed(seed)
    ks, qs = [], []
    for _ in range(n_kv):
        q, k = synth_head(gen, T + 1, gqa, theta=theta)
        ks.append(k[:T])
        qs.append(q.reshape(gqa, T + 1, HD))
    v = torch.randn(n_kv, T, HD, generator=gen).half()
    q_all = torch.stack(qs)
    return {"k": torch.stack(ks), "v": v, "q": q_all[:, :, T].reshape(n_kv * gqa, HD), "q_all": q_all}
