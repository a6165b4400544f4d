"""GPU parity at the shapes of the benchmark configurations: all 8 KV heads of a layer in one launch,
thousands of tokens per pair (many reuses of every pipeline stage), batches of 1..8, GQA groups of 4 and 8.

* ``shape_*.npz`` goldens: the reference's own encoders and decode kernel, run per head on a whole layer
  (tests/golden/make_golden.py); the fp16 inputs are regenerated from the seed and checked by hash.
* long contexts (32768 tokens) have no reference vector (the interpreter would need hours): there the
  float64 oracle decodes sampled (batch, head) pairs of the same packed cache.
"""
import hashlib

import numpy as np
import pytest
import torch

from helpers import HD, load, oracle_meta, synth_head, synth_layer_case
from oracle import bgtq_oracle as O

from blockgtq_b200 import calib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ATOL = 2e-3

SHAPE_CASES = ["cfg0_a3_1to6_h8_t4096", "k2v2_h8_t2048"]


def _tables_from_alloc(alloc, avg, mn, mx, vb, theta=500000.0):
    tabs = []
    for h in range(alloc.shape[0]):
        kt = calib.build_k_tables(None, None, head_dim=HD, avg_bits=avg, min_bits=mn, max_bits=mx,
                                  bit_allocation=torch.from_numpy(alloc[h]))
        tabs.append((kt, calib.build_v_tables(HD, vb, 42 + h)))
    return tabs


def _sha(*tensors):
    flat = torch.cat([t.reshape(-1) for t in tensors])
    return hashlib.sha256(np.ascontiguousarray(flat.numpy()).tobytes()).hexdigest()


@pytest.mark.parametrize("name", SHAPE_CASES)
def test_layer_shaped_decode_matches_reference(name):
    """One launch over the 8 KV heads of the golden layer, library-chosen slot count and two others."""
    from blockgtq_b200.layer import LayerTables, combine, decode, default_splits, rotate_q
    g = load("shape_" + name)
    avg, mn, mx, vb, n_kv, gqa, T, theta, seed = g["case"]
    n_kv, gqa, T = int(n_kv), int(gqa), int(T)
    tabs = _tables_from_alloc(g["alloc"], avg, int(mn), int(mx), int(vb))
    lt = LayerTables([t[0] for t in tabs], [t[1] for t in tabs], DEV)
    q = torch.from_numpy(g["q"]).to(DEV)
    q_rot = rotate_q(lt, q)
    torch.cuda.synchronize()
    d = q_rot.cpu().numpy().astype(np.float32) - g["q_rot"][:, :, 0].astype(np.float32)
    assert np.abs(d).max() <= np.abs(g["q_rot"]).max() * 1e-3
    kp, kn = torch.from_numpy(g["k_packed"]).to(DEV), torch.from_numpy(g["k_norms"]).to(DEV)
    vp, vn = torch.from_numpy(g["v_packed"]).to(DEV), torch.from_numpy(g["v_norms"]).to(DEV)
    gq = torch.from_numpy(g["q_rot"][:, :, 0]).to(DEV).contiguous()
    for ns in (default_splits(1, n_kv, T), int(g["t_splits"]), 1):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        po, pl = decode(lt, gq, kp, kn, vp, vn, 0, T, n_splits=ns, status=status)
        out, _, lse = combine(po, pl, n_kv, v_rot=lt.v_rot, want_lse=True)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        err = np.abs(out.cpu().numpy().astype(np.float64) - g["out"][:, :, 0].astype(np.float64))
        assert err.max() <= ATOL, f"{name} n_splits={ns}: max-abs {err.max()} at head {np.argmax(err.max(axis=(0, 2)))}"
        np.testing.assert_allclose(lse.cpu().numpy(), g["lse"], atol=5e-4, rtol=0)


@pytest.mark.parametrize("name", SHAPE_CASES)
def test_layer_shaped_encode_matches_reference(name):
    """The bulk encoder on the regenerated fp16 inputs of the golden layer: packed rows and norms of all 8
    heads against the reference's, code mismatches only where the float64 coordinate sits on a bin edge."""
    from blockgtq_b200.layer import LayerTables, encode
    g = load("shape_" + name)
    avg, mn, mx, vb, n_kv, gqa, T, theta, seed = g["case"]
    n_kv, gqa, T = int(n_kv), int(gqa), int(T)
    data = synth_layer_case(int(seed), n_kv, gqa, T, float(theta))
    assert _sha(data["k"], data["v"], data["q"]) == str(g["input_sha"]), "regenerated inputs differ from the fixture's"
    tabs = _tables_from_alloc(g["alloc"], avg, int(mn), int(mx), int(vb))
    lt = LayerTables([t[0] for t in tabs], [t[1] for t in tabs], DEV)
    kp = torch.zeros(1, n_kv, T + 64, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(1, n_kv, T + 64, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(1, n_kv, T + 64, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(1, n_kv, T + 64, dtype=torch.float16, device=DEV)
    encode(lt, data["k"].unsqueeze(0).to(DEV), data["v"].unsqueeze(0).to(DEV), 0, kp, kn, vp, vn)
    torch.cuda.synchronize()
    assert kp.shape[3] == g["k_packed"].shape[3] and kn.shape[3] == g["k_norms"].shape[3]
    n_bad_rows = 0
    for h in range(n_kv):
        kt, vt = tabs[h]
        got, want = kp[0, h, :T].cpu().numpy(), g["k_packed"][0, h]
        rows = np.nonzero((got != want).any(axis=1))[0]
        n_bad_rows += len(rows)
        if len(rows):
            meta = oracle_meta(kt, vt, int(lt.max_tpb))
            orc = O.encode_k(data["k"][h][rows].numpy(), meta, dtype=np.float64)
            # a differing row must contain a fragile coordinate, and re-packing the oracle's codes with only
            # fragile positions allowed to move must be able to explain it
            assert orc["fragile"].any(axis=1).all(), f"head {h}: packed rows differ off bin edges"
        gv, wv = vp[0, h, :T].cpu().numpy(), g["v_packed"][0, h]
        vrows = np.nonzero((gv != wv).any(axis=1))[0]
        if len(vrows):
            meta = oracle_meta(kt, vt, int(lt.max_tpb))
            vo = O.encode_v(data["v"][h][vrows].numpy(), meta, dtype=np.float64)
            assert vo["fragile"].any(axis=1).all(), f"head {h}: packed V rows differ off bin edges"
        assert len(vrows) <= max(2, T // 500)
        dn = np.abs(kn[0, h, :T].float().cpu().numpy() - g["k_norms"][0, h].astype(np.float32))
        assert (dn <= np.abs(g["k_norms"][0, h].astype(np.float32)) * 1e-3 + 1e-7).all()
        dv = np.abs(vn[0, h, :T].float().cpu().numpy() - g["v_norms"][0, h].astype(np.float32))
        assert (dv <= np.abs(g["v_norms"][0, h].astype(np.float32)) * 1e-3 + 1e-7).all()
    assert n_bad_rows <= max(4, n_kv * T // 500)          # < 0.2 % of rows may hold an edge coordinate


@pytest.mark.parametrize("B,gqa,T,avg,vb,max_mult", [(8, 8, 32768, 3.0, 3, 1), (2, 4, 32768, 2.0, 2, 1),
                                                      (1, 4, 4096, 3.0, 3, 4), (3, 8, 5000, 3.0, 3, 2)])
def test_long_context_decode_against_the_oracle(B, gqa, T, avg, vb, max_mult):
    """8 KV heads (2 for the 8-query-group case), long contexts, batch up to 8, through the manager's
    graph-replayed step (device-side length, capacity ``max_mult`` x the live length): sampled (batch, head)
    pairs against the float64 oracle on the same packed rows."""
    from blockgtq_b200 import BlockGTQKVManager
    n_kv = 2 if gqa == 8 else 8
    n_q = n_kv * gqa
    gen = torch.Generator().manual_seed(B * 1000 + T)
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=max_mult * T + 8, batch_size=B, k_avg_bits=avg, v_bits=vb,
                            device=DEV)
    cal = [synth_head(gen, 512, gqa) for _ in range(n_kv)]
    mgr.calibrate(0, torch.stack([c[0] for c in cal]).float(), torch.stack([c[1] for c in cal]).float())
    dgen = torch.Generator(device=DEV).manual_seed(7)
    scale = torch.exp(torch.randn(n_kv, 1, HD, generator=dgen, device=DEV))
    for t in range(0, T, 8192):
        n = min(8192, T - t)
        k = (torch.randn(B, n_kv, n, HD, generator=dgen, device=DEV) * scale).half()
        v = torch.randn(B, n_kv, n, HD, generator=dgen, device=DEV).half()
        mgr._encode_kv(0, k, v, t, t + n)
    mgr.seq_len = T
    for step in range(2):
        q = (torch.randn(B, n_q, 1, HD, generator=gen) * 2).half().to(DEV)
        k1 = (torch.randn(B, n_kv, 1, HD, generator=gen)).half().to(DEV)
        v1 = torch.randn(B, n_kv, 1, HD, generator=gen).half().to(DEV)
        out = mgr.append_and_attend(0, q, k1, v1).clone()
        mgr.increment_seq_len()
        torch.cuda.synchronize()
        mgr.check_status()
        n_tok = T + step + 1
        pairs = [(0, 0), (B - 1, n_kv - 1), (B // 2, n_kv // 2)]
        worst = 0.0
        for b, h in pairs:
            qz = mgr.quantizers[0][h]
            meta = oracle_meta(qz._tables, qz._v_tables)
            sl = slice(h * gqa, (h + 1) * gqa)
            qr = O.rotate_q(q[b, sl, 0].cpu().numpy(), meta)
            ro, _ = O.attend_packed(qr, mgr._k_packed[0, b, h, :n_tok, :qz._total_packed_bytes].cpu().numpy(),
                                    mgr._k_norms[0, b, h, :n_tok].cpu().numpy(),
                                    mgr._v_packed[0, b, h, :n_tok].cpu().numpy(),
                                    mgr._v_norms[0, b, h, :n_tok].cpu().numpy(), meta, mgr.scale)
            worst = max(worst, float(np.abs(out[b, sl, 0].float().cpu().numpy() - ro).max()))
        assert worst <= ATOL, f"step {step}: max-abs {worst}"
