"""GPU parity: the CUDA kernels, called through the C ABI, against the reference's golden vectors
and the NumPy oracle.  Integer outputs must be bit-exact (except where the oracle proves the fp32
coordinate sits on a bin edge); attention outputs within max-abs 2e-3 (fp16 out, fp32 accumulate)."""
import numpy as np
import pytest
import torch

from helpers import CASES, HD, load, oracle_meta, synth_head, tables_for
from oracle import bgtq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ATOL = 2e-3


def _layer(case, n_kv=2):
    from blockgtq_b200.layer import LayerTables
    gt = load("tables_" + case)
    tabs = [tables_for(case, h, gt) for h in range(n_kv)]
    return LayerTables([t[0] for t in tabs], [t[1] for t in tabs], DEV), tabs


def _quantizers(case, n_kv=2):
    from blockgtq_b200 import BlockGTQQuantizer
    gt = load("tables_" + case)
    avg, mn, mx, rt, vb = CASES[case]
    qs = []
    for h in range(n_kv):
        z = BlockGTQQuantizer(HD, avg_bits=avg, rotation_threshold=rt, min_bits=mn, max_bits=mx, device=DEV)
        z.calibrate(None, None, bit_allocation=torch.from_numpy(gt[f"h{h}_alloc"]))
        z.init_v_quantizer(v_bits=vb, seed=42 + h)
        qs.append(z)
    return qs


@pytest.mark.parametrize("case", list(CASES))
def test_encode_matches_reference(case):
    from blockgtq_b200 import (build_batched_encode_args, compress_k_mixed_batched, compress_k_packed_batched,
                               compress_v_nibble4_batched, compress_v_packed_batched)
    ge = load("encode_" + case)
    qs = _quantizers(case)
    ba = build_batched_encode_args(qs, device=DEV)
    k = torch.from_numpy(ge["k"]).to(DEV)
    v = torch.from_numpy(ge["v"]).to(DEV)
    kp, kn = compress_k_packed_batched(k, ba)
    vp, vn = compress_v_packed_batched(v, ba)
    km, knc = compress_k_mixed_batched(k, ba)
    vnib, vn2 = compress_v_nibble4_batched(v, ba)
    torch.cuda.synchronize()
    assert kp.shape == ge["k_packed"].shape and kn.shape == ge["k_norms"].shape
    assert vp.shape == ge["v_packed"].shape and km.shape == ge["k_mixed"].shape
    gt = load("tables_" + case)
    for h in range(2):
        kt, vt = tables_for(case, h, gt)
        meta = oracle_meta(kt, vt, int(ge["max_tpb"]))
        orc = O.encode_k(ge["k"][h], meta, dtype=np.float64)
        codes = qs[h].compress(k[h])[0].cpu().numpy()
        bad = codes != ge["k_codes"][h]
        # any disagreement must sit on a bin edge of the float64 coordinate
        assert not (bad & ~orc["fragile"]).any(), f"{case} head {h}: {bad.sum()} code mismatches off bin edges"
        assert bad.mean() < 1e-3
        if not bad.any():
            assert np.array_equal(kp[h].cpu().numpy(), ge["k_packed"][h])
            assert np.array_equal(km[h].cpu().numpy(), ge["k_mixed"][h])
        else:   # the bytes must still be the exact packing of the codes the kernel chose
            assert np.array_equal(kp[h].cpu().numpy(), O.pack_k(codes, kt.segments, int(ge["max_tpb"])))
        np.testing.assert_allclose(kn[h].cpu().numpy(), ge["k_norms"][h], rtol=2e-6, atol=1e-30)
        np.testing.assert_allclose(knc[h].cpu().numpy(), ge["k_norms_corrected"][h], rtol=5e-6, atol=1e-30)
        vo = O.encode_v(ge["v"][h], meta, dtype=np.float64)
        vcodes = qs[h].compress_v(v[h])[0].cpu().numpy()
        vbad = vcodes != ge["v_codes_torch"][h]
        assert not (vbad & ~vo["fragile"]).any()
        if not vbad.any():
            assert np.array_equal(vp[h].cpu().numpy(), ge["v_packed"][h])
            assert np.array_equal(vnib[h].cpu().numpy(), ge["v_nibble"][h])
        dn = np.abs(vn[h].cpu().numpy().astype(np.float32) - ge["v_norms"][h].astype(np.float32))
        assert (dn <= np.abs(ge["v_norms"][h].astype(np.float32)) * 1e-3).all()      # <= 1 fp16 ulp
        assert (dn > 0).mean() < 0.02


@pytest.mark.parametrize("case", ["a3_1to6", "a3_1to8", "a2_1to8", "a4_rt1"])
@pytest.mark.parametrize("n_splits", [None, 1, 8])
def test_decode_matches_reference(case, n_splits):
    from blockgtq_b200.layer import combine, decode, rotate_q
    gd = load("decode_" + case)
    lt, tabs = _layer(case)
    q = torch.from_numpy(gd["q"]).to(DEV)
    q_rot = rotate_q(lt, q)
    torch.cuda.synchronize()
    d = (q_rot.cpu().numpy().astype(np.float32) - gd["q_rot"][:, :, 0].astype(np.float32))
    assert np.abs(d).max() <= np.abs(gd["q_rot"]).max() * 1e-3 and (d != 0).mean() < 0.01
    kp, kn = torch.from_numpy(gd["k_packed"]).to(DEV), torch.from_numpy(gd["k_norms"]).to(DEV)
    vp, vn = torch.from_numpy(gd["v_packed"]).to(DEV), torch.from_numpy(gd["v_norms"]).to(DEV)
    T = kp.shape[2]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ns = int(gd["t_splits"]) if n_splits is None else n_splits
    po, pl = decode(lt, torch.from_numpy(gd["q_rot"][:, :, 0]).to(DEV).contiguous(), kp, kn, vp, vn, 0, T,
                    n_splits=ns, status=status)
    out, _, lse = combine(po, pl, lt.n_kv, v_rot=lt.v_rot, want_lse=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    err = np.abs(out.cpu().numpy().astype(np.float64) - gd["out"][:, :, 0].astype(np.float64)).max()
    assert err <= ATOL, f"max-abs {err}"
    np.testing.assert_allclose(lse.cpu().numpy(), gd["lse"], atol=5e-4, rtol=0)


def test_operator_api_matches_reference():
    """fused_blockgtq_decode_attention with the reference's per-head calling convention."""
    from blockgtq_b200 import fused_blockgtq_decode_attention
    case = "a3_1to8"
    gd = load("decode_" + case)
    qs = _quantizers(case)
    gqa = int(gd["gqa"])
    for h in range(2):
        ka = qs[h].build_kernel_args()
        sl = slice(h * gqa, (h + 1) * gqa)
        o, lse = fused_blockgtq_decode_attention(
            torch.from_numpy(gd["q_rot"][:, sl]).to(DEV),
            torch.from_numpy(gd["k_packed"][:, h:h + 1]).to(DEV), torch.from_numpy(gd["k_norms"][:, h:h + 1]).to(DEV),
            ka["codebook_flat"], ka["lut_offset"], ka["norm_group"], ka["segments_b"],
            torch.from_numpy(gd["v_packed"][:, h:h + 1]).to(DEV), torch.from_numpy(gd["v_norms"][:, h:h + 1]).to(DEV),
            qs[h].v_lut, scale=1.0 / HD ** 0.5, t_splits=int(gd["t_splits"]), v_bits=qs[h].v_bits,
            v_rotation=qs[h]._v_rot, return_lse=True)
        assert o.shape == (2, gqa, 1, HD) and o.dtype == torch.float16
        err = np.abs(o.cpu().numpy().astype(np.float64) - gd["out"][:, sl].astype(np.float64)).max()
        assert err <= ATOL


def test_manager_matches_reference():
    from blockgtq_b200 import BlockGTQKVManager
    g = load("manager")
    B, n_kv, T0, _ = g["k_init"].shape
    n_q = g["q0"].shape[1]
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=T0 + 4, batch_size=B, k_avg_bits=3.0, v_bits=3, device=DEV)
    mgr.calibrate(0, torch.from_numpy(g["cal_q"]), torch.from_numpy(g["cal_k"]))
    assert np.array_equal(np.stack([mgr.quantizers[0][h].bit_allocation.numpy() for h in range(n_kv)]), g["alloc"])
    mgr._encode_kv(0, torch.from_numpy(g["k_init"]).to(DEV), torch.from_numpy(g["v_init"]).to(DEV), 0, T0)
    mgr.seq_len = T0
    for s in range(2):
        out = mgr.append_and_attend(0, torch.from_numpy(g[f"q{s}"]).to(DEV), torch.from_numpy(g[f"k{s}"]).to(DEV),
                                    torch.from_numpy(g[f"v{s}"]).to(DEV))
        mgr.increment_seq_len()
        err = np.abs(out.cpu().numpy().astype(np.float64) - g[f"out{s}"].astype(np.float64)).max()
        assert out.shape == g[f"out{s}"].shape and err <= ATOL, f"step {s}: {err}"
    mgr.check_status()
    T = mgr.seq_len
    same = (mgr._k_packed[:, :, :, :T].cpu().numpy() == g["k_packed"]).mean()
    assert same > 0.9999, same
    assert (mgr._v_packed[:, :, :, :T].cpu().numpy() == g["v_packed"]).mean() > 0.9999
    ng = g["k_norms"].shape[-1]          # (the manager pads norm rows to an even number of values, zeros behind)
    assert not mgr._k_norms[..., ng:].any()
    kn = mgr._k_norms[:, :, :, :T, :ng].float().cpu().numpy()
    assert (np.abs(kn - g["k_norms"].astype(np.float32)) <= np.abs(kn) * 1e-3).all()


@pytest.mark.parametrize("T", [0, 1, 63, 64, 65, 129, 1000])
def test_decode_ragged_lengths_vs_oracle(T):
    """Edge lengths around the 64-token tile, empty cache included, against the float64 oracle."""
    from blockgtq_b200.layer import combine, decode, encode, rotate_q
    case = "a3_1to8"
    lt, tabs = _layer(case)
    gen = torch.Generator().manual_seed(100 + T)
    B, n_kv, gqa = 2, 2, 4
    cap = max(T, 1) + 7
    ks, qs_ = [], []
    for b in range(B):
        hk, hq = [], []
        for h in range(n_kv):
            q, k = synth_head(gen, T + 1, gqa)
            hk.append(k[:T] if T else k[:0])
            hq.append(q.reshape(gqa, T + 1, HD)[:, T])
        ks.append(torch.stack(hk))
        qs_.append(torch.cat(hq))
    k = torch.stack(ks).to(DEV)
    q = torch.stack(qs_).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, cap, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, cap, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, cap, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, cap, dtype=torch.float16, device=DEV)
    if T:
        encode(lt, k, v, 0, kp, kn, vp, vn)
    q_rot = rotate_q(lt, q)
    po, pl = decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=3)
    out, o32, lse = combine(po, pl, n_kv, v_rot=lt.v_rot, want_f32=True, want_lse=True)
    torch.cuda.synchronize()
    for b in range(B):
        for h in range(n_kv):
            meta = oracle_meta(*tabs[h])
            sl = slice(h * gqa, (h + 1) * gqa)
            ro, rl = O.attend_packed(q_rot[b, sl].cpu().numpy(), kp[b, h, :T].cpu().numpy(), kn[b, h, :T].cpu().numpy(),
                                     vp[b, h, :T].cpu().numpy(), vn[b, h, :T].cpu().numpy(), meta, 1 / HD ** 0.5)
            assert np.abs(o32[b, sl].cpu().numpy() - ro).max() <= ATOL
            if T:
                np.testing.assert_allclose(lse[b, sl].cpu().numpy(), rl, atol=5e-4)
            else:
                assert np.isneginf(lse[b, sl].cpu().numpy()).all() and (out[b, sl] == 0).all()


def test_combine_and_buffer_vs_oracle():
    from blockgtq_b200.layer import buffer_attn, combine
    gen = torch.Generator().manual_seed(5)
    B, n_kv, gqa, S = 2, 2, 4, 5
    n_q = n_kv * gqa
    po = torch.randn(B, n_q, S, HD, generator=gen)
    pl = torch.randn(B, n_q, S, generator=gen) * 3
    pl[0, 0, :] = float("-inf")              # a row with every split empty
    pl[1, 2, 1] = float("-inf")
    out, o32, lse = combine(po.to(DEV), pl.to(DEV), n_kv, want_f32=True, want_lse=True)
    torch.cuda.synchronize()
    ro, rl = O.combine(po.numpy().transpose(2, 0, 1, 3).reshape(S, B * n_q, HD), pl.numpy().transpose(2, 0, 1).reshape(S, -1))
    np.testing.assert_allclose(o32.cpu().numpy().reshape(-1, HD), ro, atol=2e-6)
    np.testing.assert_allclose(lse.cpu().numpy().reshape(-1), rl, atol=2e-6)
    assert not torch.isnan(out).any()
    # fp16 buffer attention with a wrapped ring
    n_sink, ring, cap = 4, 9, 13
    kb = (torch.randn(B, n_kv, cap, HD, generator=gen) * 2).half()
    vb = torch.randn(B, n_kv, cap, HD, generator=gen).half()
    q = torch.randn(B, n_q, HD, generator=gen).half()
    first, n_ring = 6, 7
    bo, bl = buffer_attn(q.to(DEV), kb.to(DEV), vb.to(DEV), n_kv, 0.0884, n_sink_tokens=n_sink,
                         n_ring_tokens=n_ring, sink_cap=n_sink, ring_first=first, ring_size=ring)
    torch.cuda.synchronize()
    slots = list(range(n_sink)) + [n_sink + (first + i) % ring for i in range(n_ring)]
    for b in range(B):
        for hq in range(n_q):
            h = hq // gqa
            ro, rl = O.attend_fp16(q[b, hq:hq + 1].numpy(), kb[b, h, slots].numpy(), vb[b, h, slots].numpy(), 0.0884)
            np.testing.assert_allclose(bo[b, hq].cpu().numpy(), ro[0], atol=2e-5)
            np.testing.assert_allclose(bl[b, hq].cpu().numpy(), rl[0], atol=2e-5)


@pytest.mark.parametrize("n_sink,window,bs", [(2, 5, 1), (3, 4, 3), (0, 6, 2), (0, 6, 1), (4, 3, 1)])
def test_three_region_manager_vs_oracle(n_sink, window, bs):
    """fp16 sink + packed middle + fp16 recent ring: every decode step against the float64 oracle built
    from the same token stream (flush order of blockgtq/unaccelerated.py:226-233)."""
    from blockgtq_b200 import BlockGTQKVManager
    gen = torch.Generator().manual_seed(11)
    B, n_kv, gqa = 2, 2, 4
    n_q = n_kv * gqa
    T0, steps = 9, 14
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=64, batch_size=B, k_avg_bits=3.0, v_bits=3, device=DEV,
                            n_sink=n_sink, recent_window=window, block_size=bs)
    cal = [synth_head(gen, 256, gqa) for _ in range(n_kv)]
    mgr.calibrate(0, torch.stack([c[0] for c in cal]).float(), torch.stack([c[1] for c in cal]).float())
    k_all = torch.stack([torch.stack([synth_head(gen, T0 + steps, 1)[1] for _ in range(n_kv)]) for _ in range(B)])
    v_all = torch.randn(B, n_kv, T0 + steps, HD, generator=gen).half()
    mgr._append_tokens(0, k_all[:, :, :T0].to(DEV), v_all[:, :, :T0].to(DEV), 0)      # bulk prefill
    mgr.seq_len = T0
    metas = [oracle_meta(mgr.quantizers[0][h]._tables, mgr.quantizers[0][h]._v_tables) for h in range(n_kv)]
    for s in range(steps):
        t = T0 + s
        q = (torch.randn(B, n_q, 1, HD, generator=gen) * 2).half()
        # regions the step must see: flushed count as of the previous step, new token still fp16
        _sink, f_prev, _ = O.three_region_plan(t, n_sink, window, bs)
        out = mgr.append_and_attend(0, q.to(DEV), k_all[:, :, t:t + 1].to(DEV), v_all[:, :, t:t + 1].to(DEV))
        mgr.increment_seq_len()
        torch.cuda.synchronize()
        n_sk = min(t + 1, n_sink)
        fp16_idx = list(range(n_sk)) + list(range(n_sink + f_prev, t + 1))
        for b in range(B):
            for h in range(n_kv):
                sl = slice(h * gqa, (h + 1) * gqa)
                qz = mgr.quantizers[0][h]
                qr = O.rotate_q(q[b, sl, 0].numpy(), metas[h])
                po, pl = O.attend_packed(qr, mgr._k_packed[0, b, h, :f_prev, :qz._total_packed_bytes].cpu().numpy(),
                                         mgr._k_norms[0, b, h, :f_prev].cpu().numpy(),
                                         mgr._v_packed[0, b, h, :f_prev].cpu().numpy(),
                                         mgr._v_norms[0, b, h, :f_prev].cpu().numpy(), metas[h], mgr.scale)
                bo, bl = O.attend_fp16(q[b, sl, 0].numpy(), k_all[b, h, fp16_idx].numpy(), v_all[b, h, fp16_idx].numpy(),
                                       mgr.scale)
                want, _ = O.combine(np.stack([po, bo]), np.stack([pl, bl]))
                err = np.abs(out[b, sl, 0].float().cpu().numpy() - want).max()
                assert err <= 3e-3, f"step {s} b{b} h{h}: {err}"
        # packed rows hold exactly the non-sink tokens in order
        _s2, f_now, n_rec = mgr._region_sizes(mgr.seq_len)
        assert (_s2, f_now, n_rec) == O.three_region_plan(t + 1, n_sink, window, bs)
    h = 0
    enc = O.encode_k_packed(k_all[0, h, n_sink:n_sink + f_now].numpy(), metas[h])
    got = mgr._k_packed[0, 0, h, :f_now, :mgr.quantizers[0][h]._total_packed_bytes].cpu().numpy()
    assert (got != enc["packed"]).mean() < 2e-3


def test_production_cache_matches_reference():
    """Nibble/mixed layout end to end: bytes of the bulk encode and two decode steps vs the reference class."""
    from blockgtq_b200 import BlockGTQProductionCache, BlockGTQQuantizer, build_batched_encode_args
    g = load("production")
    n_kv, T0 = g["k_init"].shape[1], g["k_init"].shape[2]
    n_q = g["q0"].shape[1]
    qs = []
    for h in range(n_kv):
        z = BlockGTQQuantizer(HD, avg_bits=3.0, device=DEV)
        z.calibrate(None, None, bit_allocation=torch.from_numpy(g["alloc"][h]))
        z.init_v_quantizer(v_bits=3, seed=42 + h)
        qs.append(z)
    ba = [build_batched_encode_args(qs, device=DEV)]
    ka = [[z.build_kernel_args() for z in qs]]
    for graph in (False, True):
        cache = BlockGTQProductionCache([qs], ba, ka, 1, n_kv, n_q, HD, T0 + 4, v_bits=3, device=DEV,
                                        use_cuda_graph=graph)
        assert cache.k_packed.shape[-1] == g["k_packed"].shape[-1] and cache.vpb == HD // 2
        cache._encode_batched(0, torch.from_numpy(g["k_init"]).to(DEV), torch.from_numpy(g["v_init"]).to(DEV), 0)
        cache.seq_len = T0
        for s in range(2):
            out = cache.encode_and_attend(0, torch.from_numpy(g[f"q{s}"]).to(DEV), torch.from_numpy(g[f"k{s}"]).to(DEV),
                                          torch.from_numpy(g[f"v{s}"]).to(DEV))
            cache.increment_seq_len()
            err = np.abs(out.cpu().numpy().astype(np.float64) - g[f"out{s}"].astype(np.float64)).max()
            assert out.shape == g[f"out{s}"].shape and err <= ATOL, f"graph={graph} step {s}: {err}"
        T = cache.seq_len
        assert (cache.k_packed[:, :, :, :T].cpu().numpy() == g["k_packed"]).mean() > 0.9995
        assert (cache.v_packed[:, :, :, :T].cpu().numpy() == g["v_packed"]).mean() > 0.9995
        kn = cache.k_norms[:, :, :, :T].float().cpu().numpy()
        assert (np.abs(kn - g["k_norms"].astype(np.float32)) <= np.abs(kn) * 2e-3 + 1e-6).all()


@pytest.mark.parametrize("case", ["a3_1to8", "a4_rt1", "u3"])
@pytest.mark.parametrize("mixed", [False, True])
def test_encoder_tensor_core_and_fp32_paths_vs_oracle(case, mixed):
    """Bulk row counts run the tensor-core encoder (tcgen05 + tensor memory by default, warp MMA with
    BGTQ_ENC_NO_TCGEN05), small ones (or BGTQ_ENC_FORCE_SIMT) the fp32 one.  All must give the oracle's
    codes off bin edges, and bytes that are the exact packing
    of the codes each chose; rows land at the requested slot offset; ragged tile tails."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import encode
    lt, tabs = _layer(case)
    gen = torch.Generator().manual_seed(31)
    B, n_kv, S, t0 = 3, 2, 150, 5          # 450 rows: 7 full 64-row tiles + a 2-row tail
    k = torch.stack([torch.stack([synth_head(gen, S, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, S, HD, generator=gen).half().to(DEV)
    k[0, 0, 3] = 0
    v[1, 1, 7] = 0
    k[2, 1, 11] *= 1e-4
    base = (_lib.ENC_K_MIXED | _lib.ENC_V_NIBBLE) if mixed else 0
    outs = []
    for extra in (0, _lib.ENC_FORCE_SIMT, _lib.ENC_NO_TCGEN05):
        kb = lt.max_mixed_bytes if mixed else lt.max_tpb
        kp = torch.full((B, n_kv, t0 + S + 2, kb), 0xEE, dtype=torch.uint8, device=DEV)
        kn = torch.full((B, n_kv, t0 + S + 2, lt.max_ng), -1.0, dtype=torch.float32, device=DEV)
        vp = torch.full((B, n_kv, t0 + S + 2, HD // 2 if mixed else lt.vpb), 0xEE, dtype=torch.uint8, device=DEV)
        vn = torch.full((B, n_kv, t0 + S + 2), -1.0, dtype=torch.float16, device=DEV)
        kc = torch.zeros(B, n_kv, S, HD, dtype=torch.uint8, device=DEV)
        vc = torch.zeros(B, n_kv, S, HD, dtype=torch.uint8, device=DEV)
        encode(lt, k, v, t0, kp, kn, vp, vn, flags=base | extra, k_codes=kc, v_codes=vc)
        torch.cuda.synchronize()
        outs.append([t.cpu().numpy() for t in (kp, kn, vp, vn, kc, vc)])
    for kp, kn, vp, vn, kc, vc in outs:
        # rows outside [t0, t0+S) untouched
        assert (kp[:, :, :t0] == 0xEE).all() and (kp[:, :, t0 + S:] == 0xEE).all()
        assert (vn[:, :, :t0] == -1).all() and (vn[:, :, t0 + S:] == -1).all()
        for b in range(B):
            for h in range(n_kv):
                kt, vt = tabs[h]
                meta = oracle_meta(kt, vt, lt.max_tpb)
                ok = O.encode_k(k[b, h].cpu().numpy(), meta, dtype=np.float64)
                bad = kc[b, h] != ok["codes"]
                assert not (bad & ~ok["fragile"]).any()
                live = np.abs(k[b, h].cpu().numpy()).max(axis=1) > 0    # an all-zero row sits exactly on the middle edge
                assert bad[live].mean() < 2e-3
                rows = kp[b, h, t0:t0 + S]
                if mixed:
                    pm = kt.pack_meta
                    assert np.array_equal(rows, O.pack_k_mixed(kc[b, h], pm["nopack_start"], pm["nopack_len"], rows.shape[1]))
                else:
                    assert np.array_equal(rows, O.pack_k(kc[b, h], kt.segments, lt.max_tpb))
                    np.testing.assert_allclose(kn[b, h, t0:t0 + S, :kt.n_groups], ok["norms"], rtol=3e-6, atol=1e-30)
                ov = O.encode_v(v[b, h].cpu().numpy(), meta, dtype=np.float64)
                vbad = vc[b, h] != ov["codes"]
                assert not (vbad & ~ov["fragile"]).any()
                vrows = vp[b, h, t0:t0 + S]
                want = O.pack_nibble4(vc[b, h]) if mixed else O.pack_v(vc[b, h], vt.bits)
                assert np.array_equal(vrows, want)
    # the two paths agree with each other except on bin edges (already bounded above), norms to fp32 noise
    assert _lib.lib().bgtq_encode_tcgen05_status() == 0
    for other in outs[1:]:
        np.testing.assert_allclose(outs[0][1], other[1], rtol=1e-5, atol=1e-30)
        assert (outs[0][4] != other[4]).mean() < 2e-3


def test_combine_ranks_matches_single_range():
    """Sequence sharding on one GPU: two token chunks decoded and combined separately, their
    [O | LSE] messages laid out like an all-gather receive buffer and merged by bgtq_combine_ranks,
    against one decode over the whole range.  A third, empty "rank" (LSE = -inf) must be ignored."""
    from blockgtq_b200.layer import combine, combine_ranks, decode, encode, rotate_q
    case = "a3_1to8"
    lt, tabs = _layer(case)
    gen = torch.Generator().manual_seed(77)
    B, n_kv, gqa, T = 2, 2, 4, 1000
    n_q = n_kv * gqa
    ks, qs_ = [], []
    for b in range(B):
        hk, hq = [], []
        for h in range(n_kv):
            q, k = synth_head(gen, T + 1, gqa)
            hk.append(k[:T])
            hq.append(q.reshape(gqa, T + 1, HD)[:, T])
        ks.append(torch.stack(hk))
        qs_.append(torch.cat(hq))
    k = torch.stack(ks).to(DEV)
    q = torch.stack(qs_).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 8, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 8, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 8, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 8, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn)
    q_rot = rotate_q(lt, q)
    rows = B * n_q
    gathered = torch.zeros(3, rows * (HD + 1) + 5, dtype=torch.float32, device=DEV)[:, :rows * (HD + 1) + 5]
    for r, (lo, hi) in enumerate([(0, 400), (400, 1000), (1000, 1000)]):
        po, pl = decode(lt, q_rot, kp, kn, vp, vn, lo, hi, n_splits=2)
        msg = gathered[r]
        combine(po, pl, n_kv, v_rot=lt.v_rot, o32_out=msg[:rows * HD].view(B, n_q, HD),
                lse_out=msg[rows * HD:rows * (HD + 1)].view(B, n_q))
    assert torch.isneginf(gathered[2, rows * HD:rows * (HD + 1)]).all()
    out = combine_ranks(gathered, B, n_q)
    po, pl = decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=3)
    ref, ref32, _ = combine(po, pl, n_kv, v_rot=lt.v_rot, want_f32=True)
    torch.cuda.synchronize()
    assert (out.float() - ref32).abs().max().item() <= 1e-3
    assert (out.float() - ref.float()).abs().max().item() <= 2e-3


@pytest.mark.parametrize("case,gqa,S_q,offset,causal", [("a3_1to8", 4, 70, 50, True), ("a2_1to8", 8, 33, 0, True),
                                                        ("a4_rt1", 2, 40, 88, True), ("a3_1to6", 4, 20, 100, False)])
def test_prefill_attention_vs_oracle(case, gqa, S_q, offset, causal):
    """Causal multi-query attention over the packed cache: every query row against the float64 oracle
    decode over exactly the tokens it may see (query i sits at position offset + i)."""
    from blockgtq_b200.layer import encode, prefill_attention, rotate_q, rotate_q_bulk
    lt, tabs = _layer(case)
    gen = torch.Generator().manual_seed(11 + S_q)
    B, n_kv = 2, 2
    n_q = n_kv * gqa
    T = offset + S_q
    ks, qs_ = [], []
    for b in range(B):
        hk, hq = [], []
        for h in range(n_kv):
            q, k = synth_head(gen, T, gqa)
            hk.append(k)
            hq.append(q.reshape(gqa, T, HD)[:, offset:])
        ks.append(torch.stack(hk))
        qs_.append(torch.cat(hq))
    k = torch.stack(ks).to(DEV)
    q = torch.stack(qs_).to(DEV)                     # (B, n_q, S_q, 128)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 5, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 5, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 5, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 5, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn)
    q_rot = rotate_q_bulk(lt, q)
    # the bulk rotation equals the per-row kernel up to fp16 rounding of the result
    one = rotate_q(lt, q[:, :, 3].contiguous())
    assert (q_rot[:, :, 3].float() - one.float()).abs().max().item() <= 2e-3 * max(1.0, one.float().abs().max().item())
    out = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=offset, causal=causal, v_rot=lt.v_rot)
    out_rot = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=offset, causal=causal)
    torch.cuda.synchronize()
    assert out.shape == (B, n_q, S_q, HD) and out.dtype == torch.float16
    worst = 0.0
    for b in range(B):
        for h in range(n_kv):
            meta = oracle_meta(*tabs[h])
            sl = slice(h * gqa, (h + 1) * gqa)
            for i in (0, 1, S_q // 2, S_q - 2, S_q - 1):
                lim = offset + i + 1 if causal else T
                args = (q_rot[b, sl, i].cpu().numpy(), kp[b, h, :lim].cpu().numpy(), kn[b, h, :lim].cpu().numpy(),
                        vp[b, h, :lim].cpu().numpy(), vn[b, h, :lim].cpu().numpy(), meta, 1 / HD ** 0.5)
                ro_rot, _ = O.attend_packed(*args, unrotate=False)
                ro, _ = O.attend_packed(*args)
                worst = max(worst, np.abs(out_rot[b, sl, i].float().cpu().numpy() - ro_rot).max())
                worst = max(worst, np.abs(out[b, sl, i].float().cpu().numpy() - ro).max())
    assert worst <= ATOL, worst


def test_prefill_attention_matches_reference_golden():
    """The operator with the reference's signature against the reference's own prefill kernel output."""
    from blockgtq_b200 import BlockGTQQuantizer, fused_blockgtq_prefill_attention
    g = load("prefill")
    avg, mn, mx, rt, vb = CASES[str(g["case"])]
    gqa, off = int(g["gqa"]), int(g["offset"])
    kp, kn = torch.from_numpy(g["k_packed"]).to(DEV), torch.from_numpy(g["k_norms"]).to(DEV)
    vp, vn = torch.from_numpy(g["v_packed"]).to(DEV), torch.from_numpy(g["v_norms"]).to(DEV)
    q = torch.from_numpy(g["q"]).to(DEV)
    for h in range(2):
        z = BlockGTQQuantizer(HD, avg_bits=avg, rotation_threshold=rt, min_bits=mn, max_bits=mx, device=DEV)
        z.calibrate(None, None, bit_allocation=torch.from_numpy(g[f"h{h}_alloc"]))
        z.init_v_quantizer(v_bits=vb, seed=42 + h)
        ka = z.build_kernel_args()
        q_h = q[:, h * gqa:(h + 1) * gqa]
        q_rot = z.rotate_q_for_packed_kernel(q_h.reshape(-1, HD)).reshape(q_h.shape)
        ref_rot = torch.from_numpy(g["q_rot"][:, h * gqa:(h + 1) * gqa]).to(DEV)
        assert (q_rot.float() - ref_rot.float()).abs().max().item() <= 2e-3 * max(1.0, ref_rot.float().abs().max().item())
        out = fused_blockgtq_prefill_attention(
            ref_rot, kp[:, h:h + 1], kn[:, h:h + 1], ka["codebook_flat"], ka["lut_offset"], ka["norm_group"],
            ka["segments_b"], vp[:, h:h + 1], vn[:, h:h + 1], z.v_lut, scale=1.0 / HD ** 0.5, block_q=32, block_t=64,
            v_bits=z.v_bits, v_rotation=z._v_rot, is_causal=True, q_pos_offset=off)
        torch.cuda.synchronize()
        ref = torch.from_numpy(g["out"][:, h * gqa:(h + 1) * gqa]).to(DEV)
        assert out.shape == ref.shape and out.dtype == torch.float16
        assert (out.float() - ref.float()).abs().max().item() <= ATOL


def test_prefill_attention_mixed_layout_matches_decode_kernel():
    """Nibble/raw K rows + nibble V rows (the production cache's layout): every prefill query row must
    equal the decode kernel run over exactly the tokens that row may see."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import combine, decode, encode, prefill_attention, rotate_q_bulk
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(5150)
    B, n_kv, gqa, S_q, off = 1, 2, 4, 37, 100
    n_q, T = n_kv * gqa, off + S_q
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    q = (torch.randn(B, n_q, S_q, HD, generator=gen) * 2).half().to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 3, lt.max_mixed_bytes, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 3, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 3, HD // 2, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 3, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn, flags=_lib.ENC_K_MIXED | _lib.ENC_V_NIBBLE)
    q_rot = rotate_q_bulk(lt, q)
    fl = _lib.DEC_K_MIXED | _lib.DEC_V_NIBBLE
    out = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=off, causal=True, flags=fl, v_rot=lt.v_rot)
    for i in (0, 7, 20, S_q - 1):
        po, pl = decode(lt, q_rot[:, :, i].contiguous(), kp, kn, vp, vn, 0, off + i + 1, n_splits=2, flags=fl)
        ref, _, _ = combine(po, pl, n_kv, v_rot=lt.v_rot)
        torch.cuda.synchronize()
        assert (out[:, :, i].float() - ref.float()).abs().max().item() <= ATOL


def test_bulk_encoder_single_sided_and_strided_cache():
    """tcgen05 bulk encoder with only K or only V given, writing into a cache whose token stride is larger
    than the row (the per-row store path), against the warp-MMA path: same bytes off bin edges, the other
    side's cache untouched, status word clean."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import encode
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(4242)
    B, n_kv, S = 2, 2, 200                  # 400 rows: three full 128-row tiles and a 16-row tail
    k = torch.stack([torch.stack([synth_head(gen, S, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, S, HD, generator=gen).half().to(DEV)
    res = []
    for extra in (0, _lib.ENC_NO_TCGEN05):
        kp = torch.full((B, n_kv, S + 3, lt.max_tpb + 5), 0xAB, dtype=torch.uint8, device=DEV)[..., :lt.max_tpb]
        kn = torch.zeros(B, n_kv, S + 3, lt.max_ng, dtype=torch.float16, device=DEV)
        vp = torch.full((B, n_kv, S + 3, lt.vpb + 3), 0xAB, dtype=torch.uint8, device=DEV)[..., :lt.vpb]
        vn = torch.full((B, n_kv, S + 3), -2.0, dtype=torch.float16, device=DEV)
        kc = torch.zeros(B, n_kv, S, HD, dtype=torch.uint8, device=DEV)
        vc = torch.zeros(B, n_kv, S, HD, dtype=torch.uint8, device=DEV)
        encode(lt, k, None, 1, kp, kn, None, None, flags=extra, k_codes=kc)
        torch.cuda.synchronize()
        assert (vp == 0xAB).all() and (vn == -2.0).all()            # V side untouched by a K-only call
        encode(lt, None, v, 1, None, None, vp, vn, flags=extra, v_codes=vc)
        torch.cuda.synchronize()
        res.append([t.cpu().numpy() for t in (kp, kn, vp, vn, kc, vc)])
    assert _lib.lib().bgtq_encode_tcgen05_status() == 0
    a, b = res
    assert (a[4] != b[4]).mean() < 2e-3 and (a[5] != b[5]).mean() < 2e-3
    np.testing.assert_allclose(a[1].astype(np.float32), b[1].astype(np.float32), rtol=2e-3, atol=1e-6)
    np.testing.assert_allclose(a[3].astype(np.float32), b[3].astype(np.float32), rtol=2e-3, atol=1e-6)
    for r in res:
        for bb in range(B):
            for h in range(n_kv):
                assert np.array_equal(r[0][bb, h, 1:1 + S], O.pack_k(r[4][bb, h], tabs[h][0].segments, lt.max_tpb))
                assert np.array_equal(r[2][bb, h, 1:1 + S], O.pack_v(r[5][bb, h], tabs[h][1].bits))
        assert (r[0][:, :, 0] == 0xAB).all() and (r[0][:, :, 1 + S:] == 0xAB).all()
        assert (r[2][:, :, 0] == 0xAB).all() and (r[2][:, :, 1 + S:] == 0xAB).all()


def test_bulk_encoder_rows_that_wrap_batches():
    """Tensor-core path with a token count that is not a multiple of the 16-row slab: slabs span two
    batch entries and take the per-row store path; must equal the fp32 kernel's bytes off bin edges."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import encode
    lt, tabs = _layer("a2_1to8")
    gen = torch.Generator().manual_seed(808)
    B, n_kv, S = 7, 2, 19
    k = torch.stack([torch.stack([synth_head(gen, S, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, S, HD, generator=gen).half().to(DEV)
    outs = []
    for extra in (0, _lib.ENC_FORCE_SIMT, _lib.ENC_NO_TCGEN05):
        kp = torch.zeros(B, n_kv, S + 4, lt.max_tpb, dtype=torch.uint8, device=DEV)
        kn = torch.zeros(B, n_kv, S + 4, lt.max_ng, dtype=torch.float16, device=DEV)
        vp = torch.zeros(B, n_kv, S + 4, lt.vpb, dtype=torch.uint8, device=DEV)
        vn = torch.zeros(B, n_kv, S + 4, dtype=torch.float16, device=DEV)
        kc = torch.zeros(B, n_kv, S, HD, dtype=torch.uint8, device=DEV)
        encode(lt, k, v, 2, kp, kn, vp, vn, flags=extra, k_codes=kc)
        torch.cuda.synchronize()
        outs.append((kp.cpu().numpy(), kn.cpu().numpy(), vp.cpu().numpy(), vn.cpu().numpy(), kc.cpu().numpy()))
    assert _lib.lib().bgtq_encode_tcgen05_status() == 0
    b = outs[1]
    for a in (outs[0], outs[2]):       # 133 rows: the tcgen05 path (outs[0]) runs one full 128-row tile and a 5-row tail
        assert (a[4] != b[4]).mean() < 2e-3
        if np.array_equal(a[4], b[4]):
            assert np.array_equal(a[0], b[0])
        assert (a[2] != b[2]).mean() < 2e-3
        np.testing.assert_allclose(a[1].astype(np.float32), b[1].astype(np.float32), rtol=2e-3, atol=1e-6)
        np.testing.assert_allclose(a[3].astype(np.float32), b[3].astype(np.float32), rtol=2e-3, atol=1e-6)
        for h in range(n_kv):
            for bb in range(B):
                assert np.array_equal(a[0][bb, h, 2:2 + S], O.pack_k(a[4][bb, h], tabs[h][0].segments, lt.max_tpb))
        assert (a[0][:, :, :2] == 0).all() and (a[0][:, :, 2 + S:] == 0).all()


@pytest.mark.parametrize("gqa,S_q,offset", [(1, 1, 300), (1, 130, 0), (8, 1, 0)])
def test_prefill_attention_edge_shapes(gqa, S_q, offset):
    """Single query, MHA (one query head per KV head), and more positions than one CTA holds."""
    from blockgtq_b200.layer import combine, decode, encode, prefill_attention, rotate_q_bulk
    lt, tabs = _layer("a3_1to6")
    gen = torch.Generator().manual_seed(99)
    B, n_kv = 1, 2
    n_q, T = n_kv * gqa, offset + S_q
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    q = (torch.randn(B, n_q, S_q, HD, generator=gen) * 2).half().to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 1, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 1, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 1, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 1, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn)
    q_rot = rotate_q_bulk(lt, q)
    out = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=offset, causal=True, v_rot=lt.v_rot)
    for i in sorted({0, S_q // 2, S_q - 1}):
        po, pl = decode(lt, q_rot[:, :, i].contiguous(), kp, kn, vp, vn, 0, offset + i + 1, n_splits=2)
        ref, _, _ = combine(po, pl, n_kv, v_rot=lt.v_rot)
        torch.cuda.synchronize()
        assert (out[:, :, i].float() - ref.float()).abs().max().item() <= ATOL


@pytest.mark.parametrize("gqa,S_q,offset,mixed", [(4, 300, 700, False), (8, 40, 1500, False), (2, 513, 0, True), (3, 50, 200, False)])
def test_prefill_tcgen05_and_mma_sync_kernels_agree(gqa, S_q, offset, mixed):
    """The tensor-memory kernel (default when the group size divides 256) and the mma.sync kernel
    (BGTQ_PF_NO_TCGEN05, and the only one for a group of 3) dequantise to the same fp16 operands and differ in
    the order of the fp32 sums and in when the accumulator is rescaled only: fp16 outputs within 1e-3 plus one fp16
    ulp of the value (outputs reach magnitude 4, where an ulp is 2e-3), several 128-token
    tiles, a partial last tile, rows past the end of the last block, both cache layouts; and no bounded wait of
    the tensor-memory kernel gave up."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import encode, prefill_attention, rotate_q_bulk
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(1234 + S_q)
    B, n_kv = 2, 2
    n_q, T = n_kv * gqa, offset + S_q
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    q = (torch.randn(B, n_q, S_q, HD, generator=gen) * 2).half().to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 1, lt.max_mixed_bytes if mixed else lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 1, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 1, HD // 2 if mixed else lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 1, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn, flags=(_lib.ENC_K_MIXED | _lib.ENC_V_NIBBLE) if mixed else 0)
    q_rot = rotate_q_bulk(lt, q)
    fl = (_lib.DEC_K_MIXED | _lib.DEC_V_NIBBLE) if mixed else 0
    a = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=offset, causal=True, v_rot=lt.v_rot, flags=fl)
    b = prefill_attention(lt, q_rot, kp, kn, vp, vn, T, q_pos_offset=offset, causal=True, v_rot=lt.v_rot,
                          flags=fl | _lib.PF_NO_TCGEN05)
    torch.cuda.synchronize()
    assert torch.isfinite(a.float()).all()
    assert ((a.float() - b.float()).abs() <= 1e-3 + b.float().abs() * 2.0 ** -10).all()
    assert _lib.lib().bgtq_prefill_tcgen05_status() == 0


@pytest.mark.parametrize("gqa,T", [(4, 1000), (8, 300), (2, 64), (4, 2500)])
def test_decode_result_does_not_depend_on_the_slot_count(gqa, T):
    """The number of partial slots only sets how finely the launch balances its work: one slot, a few, the
    library's own choice and far more slots than 32-token units must all merge to the same output, and slots
    without a partial must carry LSE = -inf (their output rows are poisoned with NaN beforehand)."""
    from blockgtq_b200.layer import combine, decode, default_splits, encode, rotate_q
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(4242 + T)
    B, n_kv = 3, 2
    n_q = n_kv * gqa
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 8, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 8, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 8, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 8, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn)
    q = (torch.randn(B, n_q, HD, generator=gen) * 2).half().to(DEV)
    q_rot = rotate_q(lt, q)
    outs = []
    for n_splits in (1, 3, default_splits(B, n_kv, T), 200):
        po = torch.full((B, n_q, n_splits, HD), float("nan"), dtype=torch.float32, device=DEV)
        pl = torch.full((B, n_q, n_splits), float("nan"), dtype=torch.float32, device=DEV)
        decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=n_splits, part_o=po, part_lse=pl)
        out, _, lse = combine(po, pl, n_kv, v_rot=lt.v_rot, want_lse=True)
        torch.cuda.synchronize()
        assert not torch.isnan(pl).any(), "a slot's LSE was left unwritten"
        live = pl > -float("inf")
        assert torch.isfinite(po[live]).all()
        assert torch.isfinite(out).all()
        outs.append((out.float(), lse))
    for o, l in outs[1:]:
        assert (o - outs[0][0]).abs().max().item() <= 1e-3
        assert (l - outs[0][1]).abs().max().item() <= 1e-4


@pytest.mark.parametrize("B,T,n_splits", [(8, 20000, 40), (8, 4000, 18), (3, 9000, 256)])
def test_decode_with_an_item_range_table(B, T, n_splits):
    """An item-range table (bgtq_decode_partition) moves the boundaries between the CTAs' ranges and nothing
    else: same attention output as the equal-count split; a table made for another cache length is ignored
    (bit-identical partials to a launch without one); one whose ranges are degenerate (every item in the last
    CTA) still covers every item."""
    from blockgtq_b200.layer import combine, decode, decode_grid_size, decode_partition, encode, rotate_q
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(777 + T)
    n_kv, gqa = 2, 4
    n_q = n_kv * gqa
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kp = torch.zeros(B, n_kv, T + 8, lt.max_tpb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 8, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 8, lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 8, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn)
    q_rot = rotate_q(lt, (torch.randn(B, n_q, HD, generator=gen) * 2).half().to(DEV))

    def run():
        po = torch.full((B, n_q, n_splits, HD), float("nan"), dtype=torch.float32, device=DEV)
        pl = torch.full((B, n_q, n_splits), float("nan"), dtype=torch.float32, device=DEV)
        decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=n_splits, part_o=po, part_lse=pl)
        out, _, lse = combine(po, pl, n_kv, v_rot=lt.v_rot, want_lse=True)
        torch.cuda.synchronize()
        assert not torch.isnan(pl).any(), "a slot's LSE was left unwritten"
        return po, pl, out.float(), lse

    try:
        po0, pl0, out0, lse0 = run()
        n_cta = decode_grid_size(B, n_kv, n_splits)
        table = decode_partition(B, n_kv, T, n_splits, n_cta)
        lt.set_partition(table.to(DEV))
        _, pl1, out1, lse1 = run()
        assert (out1 - out0).abs().max().item() <= 1e-3 and (lse1 - lse0).abs().max().item() <= 1e-4
        # every item in the last CTA's range: legal, if slow
        worst = table.clone()
        worst[0:4] = torch.tensor([int(x) for x in _kernel_item_key(B, n_kv, T, n_splits, n_cta)], dtype=torch.int32)
        worst[4:4 + n_cta] = 0
        lt.set_partition(worst.to(DEV))
        _, pl2, out2, lse2 = run()
        assert (out2 - out0).abs().max().item() <= 1e-3 and (lse2 - lse0).abs().max().item() <= 1e-4
        # a table for another length: ignored
        lt.set_partition(decode_partition(B, n_kv, T // 3, n_splits, n_cta).to(DEV))
        po3, pl3, _, _ = run()
        assert torch.equal(pl3, pl0)
        live = pl0 > -float("inf")
        assert torch.equal(po3[live], po0[live])
    finally:
        lt.set_partition(None)


def test_specialised_kernel_with_fixed_row_strides_and_its_fallback():
    """A layer whose specialised kernel was compiled for fixed row strides: launches with exactly those strides and
    16-byte aligned slices run it; launches with wider rows, or with slices that start off a 16-byte boundary, run
    the general kernel.  All three give bit-identical partials to a layer specialised without fixed strides."""
    from blockgtq_b200.layer import LayerTables, decode, encode, rotate_q
    lt0, tabs = _layer("a3_1to8")
    lt1 = LayerTables(lt0.k_tables, lt0.v_tables, DEV)
    ng = lt1.max_ng + (lt1.max_ng & 1)
    lt1.set_row_strides(lt1.max_tpb, ng, lt1.vpb, 1)
    gen = torch.Generator().manual_seed(5150)
    B, n_kv, gqa, T = 2, 2, 4, 1300
    n_q = n_kv * gqa
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    q_rot = rotate_q(lt0, (torch.randn(B, n_q, HD, generator=gen) * 2).half().to(DEV))

    rows = 1376                        # a multiple of 16: every (batch, head) slice starts on a 16-byte boundary

    def cache(kb, first_row):          # rows [first_row, first_row + T + 8) of the allocation
        kp = torch.zeros(B, n_kv, rows, kb, dtype=torch.uint8, device=DEV)[:, :, first_row:first_row + T + 8]
        kn = torch.zeros(B, n_kv, rows, ng, dtype=torch.float16, device=DEV)[:, :, first_row:first_row + T + 8]
        vp = torch.zeros(B, n_kv, rows, lt0.vpb, dtype=torch.uint8, device=DEV)[:, :, first_row:first_row + T + 8]
        vn = torch.zeros(B, n_kv, rows, dtype=torch.float16, device=DEV)[:, :, first_row:first_row + T + 8]
        encode(lt0, k, v, 0, kp, kn, vp, vn)
        return kp, kn, vp, vn

    ref = decode(lt0, q_rot, *cache(lt0.max_tpb, 0), 0, T, n_splits=5)
    torch.cuda.synchronize()
    live = ref[1] > -float("inf")
    for kb, first_row in ((lt0.max_tpb, 0), (lt0.max_tpb + 3, 0), (lt0.max_tpb, 1)):
        po, pl = decode(lt1, q_rot, *cache(kb, first_row), 0, T, n_splits=5)
        torch.cuda.synchronize()
        assert torch.equal(pl, ref[1]), (kb, first_row)
        assert torch.equal(po[live], ref[0][live]), (kb, first_row)


def _kernel_item_key(B, n_kv, T, n_splits, n_cta):
    """The four words the decode kernel derives for a launch and compares with a table's header."""
    units = (T + 31) // 32
    c_units = max(1, -(-units // n_splits))
    return -(-units // c_units), B * n_kv, n_cta, c_units


@pytest.mark.parametrize("case", ["a3_1to6", "a3_1to8", "a2_1to8", "a4_rt1"])
@pytest.mark.parametrize("mixed", [False, True])
def test_specialised_and_general_decode_kernels_agree_bit_for_bit(case, mixed):
    """The kernel compiled at run time for the layer's heads (default) and the general ahead-of-time kernel
    (BGTQ_DEC_GENERIC) run the same arithmetic in the same order: identical partials."""
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import decode, encode, rotate_q
    lt, tabs = _layer(case)
    gen = torch.Generator().manual_seed(99)
    B, n_kv, gqa, T = 2, 2, 4, 1500
    n_q = n_kv * gqa
    k = torch.stack([torch.stack([synth_head(gen, T, 1)[1] for _ in range(n_kv)]) for _ in range(B)]).to(DEV)
    v = torch.randn(B, n_kv, T, HD, generator=gen).half().to(DEV)
    kb = lt.max_mixed_bytes if mixed else lt.max_tpb
    kp = torch.zeros(B, n_kv, T + 8, kb, dtype=torch.uint8, device=DEV)
    kn = torch.zeros(B, n_kv, T + 8, lt.max_ng, dtype=torch.float16, device=DEV)
    vp = torch.zeros(B, n_kv, T + 8, HD // 2 if mixed else lt.vpb, dtype=torch.uint8, device=DEV)
    vn = torch.zeros(B, n_kv, T + 8, dtype=torch.float16, device=DEV)
    encode(lt, k, v, 0, kp, kn, vp, vn, flags=(_lib.ENC_K_MIXED | _lib.ENC_V_NIBBLE) if mixed else 0)
    q_rot = rotate_q(lt, (torch.randn(B, n_q, HD, generator=gen) * 2).half().to(DEV))
    fl = (_lib.DEC_K_MIXED | _lib.DEC_V_NIBBLE) if mixed else 0
    po_s, pl_s = decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=7, flags=fl)
    po_g, pl_g = decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=7, flags=fl | _lib.DEC_GENERIC)
    torch.cuda.synchronize()
    assert torch.equal(pl_s, pl_g)
    live = pl_s > -float("inf")
    assert live.any() and torch.equal(po_s[live], po_g[live])


def test_step_prepare_with_fused_rope_is_bit_identical():
    """Rotary embedding applied inside the append kernel against the fp16 expression
    (x * cos) + (rotate_half(x) * sin) evaluated by torch first: same packed rows, norms and q_rot."""
    from blockgtq_b200.layer import step_prepare
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(321)
    B, n_kv, gqa = 4, 2, 4
    n_q = n_kv * gqa
    q = (torch.randn(B, n_q, 1, HD, generator=gen) * 3).half().to(DEV)
    k = (torch.randn(B, n_kv, 1, HD, generator=gen) * 3).half().to(DEV)
    v = torch.randn(B, n_kv, 1, HD, generator=gen).half().to(DEV)
    pos = torch.tensor([5.0, 77.0, 1234.0, 31000.0])
    inv = 1.0 / (500000.0 ** (torch.arange(0, HD // 2, dtype=torch.float32) / (HD // 2)))
    ang = pos[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], dim=-1).half().to(DEV)          # (B, 128), as transformers builds them
    sin = torch.cat([ang.sin(), ang.sin()], dim=-1).half().to(DEV)

    def rot_half(x):
        return torch.cat([-x[..., HD // 2:], x[..., :HD // 2]], dim=-1)

    c4, s4 = cos[:, None, None, :], sin[:, None, None, :]
    q_ref = (q * c4) + (rot_half(q) * s4)
    k_ref = (k * c4) + (rot_half(k) * s4)
    outs = []
    for fused in (False, True):
        kp = torch.zeros(B, n_kv, 8, lt.max_tpb, dtype=torch.uint8, device=DEV)
        kn = torch.zeros(B, n_kv, 8, lt.max_ng, dtype=torch.float16, device=DEV)
        vp = torch.zeros(B, n_kv, 8, lt.vpb, dtype=torch.uint8, device=DEV)
        vn = torch.zeros(B, n_kv, 8, dtype=torch.float16, device=DEV)
        if fused:
            qr = step_prepare(lt, q, k, v, 3, kp, kn, vp, vn, rope=(cos, sin))
        else:
            qr = step_prepare(lt, q_ref, k_ref, v, 3, kp, kn, vp, vn)
        torch.cuda.synchronize()
        outs.append((qr, kp, kn, vp, vn))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("gqa", [4, 2])
def test_large_batch_step_kernels_match_the_small_batch_ones(gqa):
    """Beyond one wave of CTAs the combine switches to four rows of a KV head per CTA (or, where the head grouping
    does not allow it, to a leaner one-row variant), and the query rotation always takes four heads per CTA when
    it can.  A batch of 48 against six batches of 8: the rotation and the append in the same bits, the combine
    within fp32 summation order."""
    from blockgtq_b200.layer import combine, step_prepare
    lt, tabs = _layer("a3_1to8")
    gen = torch.Generator().manual_seed(99 + gqa)
    B, n_kv, S, chunk = 48, 2, 6, 8
    n_q = n_kv * gqa
    q = (torch.randn(B, n_q, 1, HD, generator=gen) * 3).half().to(DEV)
    k = (torch.randn(B, n_kv, 1, HD, generator=gen) * 3).half().to(DEV)
    v = torch.randn(B, n_kv, 1, HD, generator=gen).half().to(DEV)

    def cache(nb):
        return (torch.zeros(nb, n_kv, 8, lt.max_tpb, dtype=torch.uint8, device=DEV),
                torch.zeros(nb, n_kv, 8, lt.max_ng, dtype=torch.float16, device=DEV),
                torch.zeros(nb, n_kv, 8, lt.vpb, dtype=torch.uint8, device=DEV),
                torch.zeros(nb, n_kv, 8, dtype=torch.float16, device=DEV))

    big = cache(B)
    qr_big = step_prepare(lt, q, k, v, 5, *big)
    for b0 in range(0, B, chunk):
        sl = slice(b0, b0 + chunk)
        small = cache(chunk)
        qr = step_prepare(lt, q[sl], k[sl], v[sl], 5, *small)
        torch.cuda.synchronize()
        assert torch.equal(qr, qr_big[sl])
        for a, b in zip(small, big):
            assert torch.equal(a, b[sl])
    assert qr_big.float().abs().max() > 1.0
    po = torch.randn(B, n_q, S, HD, generator=gen).to(DEV)
    pl = (torch.randn(B, n_q, S, generator=gen) * 3).to(DEV)
    pl[3, 1, :] = float("-inf")
    pl[:, :, 2] = float("-inf")
    bo = torch.randn(B, n_q, HD, generator=gen).to(DEV)
    bl = torch.randn(B, n_q, generator=gen).to(DEV)
    out_big, o32_big, lse_big = combine(po, pl, n_kv, v_rot=lt.rot_v, buf_o=bo, buf_lse=bl, want_f32=True, want_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(out_big, o32_big.half())
    for b0 in range(0, B, chunk):
        sl = slice(b0, b0 + chunk)
        out, o32, lse = combine(po[sl].contiguous(), pl[sl].contiguous(), n_kv, v_rot=lt.rot_v, buf_o=bo[sl].contiguous(),
                                buf_lse=bl[sl].contiguous(), want_f32=True, want_lse=True)
        torch.cuda.synchronize()
        np.testing.assert_allclose(o32.cpu().numpy(), o32_big[sl].cpu().numpy(), atol=5e-6)
        np.testing.assert_allclose(lse.cpu().numpy(), lse_big[sl].cpu().numpy(), atol=5e-6)
    # and the big launch against the float64 oracle, un-rotation applied on the host
    ro, rl = O.combine(po.cpu().numpy().transpose(2, 0, 1, 3).reshape(S, B * n_q, HD),
                       pl.cpu().numpy().transpose(2, 0, 1).reshape(S, -1))
    rot = lt.rot_v.double().cpu().numpy()
    ro = ro.reshape(B, n_q, HD).astype(np.float64)
    ro = np.stack([ro[:, h] @ rot[h // gqa] for h in range(n_q)], 1)
    rl = rl.reshape(B, n_q).astype(np.float64)
    blc, boc = bl.double().cpu().numpy(), bo.double().cpu().numpy()
    m2 = np.maximum(rl, blc)
    wp, wb = np.exp(rl - m2), np.exp(blc - m2)
    want = (wp[..., None] * ro + wb[..., None] * boc) / (wp + wb)[..., None]
    np.testing.assert_allclose(o32_big.cpu().numpy(), want, atol=2e-5)
    np.testing.assert_allclose(lse_big.cpu().numpy(), m2 + np.log(wp + wb), atol=2e-5)


@pytest.mark.parametrize("n_sink,n_ring", [(4, 128), (0, 1), (7, 600), (256, 0)])
def test_buffer_attention_lengths_vs_oracle(n_sink, n_ring):
    """fp16 buffer attention at lengths below, at and above one pass of the CTA's threads."""
    from blockgtq_b200.layer import buffer_attn
    gen = torch.Generator().manual_seed(1000 + n_sink + n_ring)
    B, n_kv, gqa = 2, 2, 4
    n_q = n_kv * gqa
    ring = max(n_ring, 1) + 1
    cap = n_sink + ring
    kb = (torch.randn(B, n_kv, cap, HD, generator=gen) * 1.5).half()
    vb = torch.randn(B, n_kv, cap, HD, generator=gen).half()
    q = torch.randn(B, n_q, HD, generator=gen).half()
    first = ring // 2
    bo, bl = buffer_attn(q.to(DEV), kb.to(DEV), vb.to(DEV), n_kv, 0.0884, n_sink_tokens=n_sink,
                         n_ring_tokens=n_ring, sink_cap=n_sink, ring_first=first, ring_size=ring)
    torch.cuda.synchronize()
    slots = list(range(n_sink)) + [n_sink + (first + i) % ring for i in range(n_ring)]
    for b in range(B):
        for hq in range(n_q):
            h = hq // gqa
            ro, rl = O.attend_fp16(q[b, hq:hq + 1].numpy(), kb[b, h, slots].numpy(), vb[b, h, slots].numpy(), 0.0884)
            np.testing.assert_allclose(bo[b, hq].cpu().numpy(), ro[0], atol=3e-5)
            np.testing.assert_allclose(bl[b, hq].cpu().numpy(), rl[0], atol=3e-5)
    # one CTA per KV head with the rows staged in shared memory (grouped heads, small buffers) and one CTA per
    # query head reading global memory (every head its own KV head here) add the same terms in the same order
    bo1, bl1 = buffer_attn(q.to(DEV), kb.repeat_interleave(gqa, 1).contiguous().to(DEV),
                           vb.repeat_interleave(gqa, 1).contiguous().to(DEV), n_q, 0.0884, n_sink_tokens=n_sink,
                           n_ring_tokens=n_ring, sink_cap=n_sink, ring_first=first, ring_size=ring)
    torch.cuda.synchronize()
    assert torch.equal(bo1, bo) and torch.equal(bl1, bl)
