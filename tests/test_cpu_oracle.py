"""CPU tests: the NumPy oracle against the reference-generated golden vectors, and its own
pack/unpack round trips.  These pin the checker that the GPU tests rely on."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from helpers import CASES, HD, load, oracle_meta, tables_for
from oracle import bgtq_oracle as O


@pytest.mark.parametrize("case", list(CASES))
def test_encoder_oracle_reproduces_reference(case):
    gt, ge = load("tables_" + case), load("encode_" + case)
    for h in range(2):
        kt, vt = tables_for(case, h, gt)
        meta = oracle_meta(kt, vt, int(ge["max_tpb"]))
        r = O.encode_k_packed(ge["k"][h], meta)
        assert np.array_equal(r["codes"], ge["k_codes"][h])
        assert np.array_equal(r["packed"], ge["k_packed"][h])
        g = kt.n_groups
        np.testing.assert_allclose(r["norms"], ge["k_norms"][h][:, :g], rtol=1e-6)
        assert (ge["k_norms"][h][:, g:] == 0).all()
        assert np.array_equal(O.unpack_k(ge["k_packed"][h], kt.segments, HD), ge["k_codes"][h])
        rv = O.encode_v(ge["v"][h], meta)
        assert np.array_equal(rv["codes"], ge["v_codes_torch"][h])
        assert np.array_equal(rv["packed"], ge["v_packed"][h])
        assert np.array_equal(rv["norms"], ge["v_norms"][h])
        nb = gt[f"h{h}_nopack"]
        assert np.array_equal(O.pack_k_mixed(ge["k_codes"][h], int(nb[0]), int(nb[1]), int(ge["max_mixed"])),
                              ge["k_mixed"][h])
        assert np.array_equal(O.pack_nibble4(rv["codes"]), ge["v_nibble"][h])
        corr = ge["k_norms"][h][:, :g] / O.k_yhat_group_norms(ge["k_codes"][h], meta)
        np.testing.assert_allclose(corr, ge["k_norms_corrected"][h][:, :g], rtol=2e-6)


@pytest.mark.parametrize("case", ["a3_1to6", "a3_1to8", "a2_1to8", "a4_rt1"])
def test_decode_oracle_reproduces_reference(case):
    gt, gd = load("tables_" + case), load("decode_" + case)
    gqa, B, ts = int(gd["gqa"]), gd["q"].shape[0], int(gd["t_splits"])
    for h in range(2):
        kt, vt = tables_for(case, h, gt)
        meta = oracle_meta(kt, vt)
        for b in range(B):
            sl = slice(h * gqa, (h + 1) * gqa)
            qr = O.rotate_q(gd["q"][b, sl, 0], meta)
            assert np.array_equal(qr, gd["q_rot"][b, sl, 0])
            args = (qr, gd["k_packed"][b, h], gd["k_norms"][b, h], gd["v_packed"][b, h], gd["v_norms"][b, h], meta,
                    1 / HD ** 0.5)
            g = gd["out"][b, sl, 0].astype(np.float64)
            om, lm = O.attend_packed_mirror(*args, t_splits=ts)
            assert np.abs(om.astype(np.float64) - g).max() <= 1e-3        # same rounding points: <= 1 fp16 step
            oe, le = O.attend_packed(*args)
            assert np.abs(oe - g).max() <= 2e-3
            np.testing.assert_allclose(le, gd["lse"][b, sl], atol=5e-4)
            np.testing.assert_allclose(lm, gd["lse"][b, sl], atol=5e-4)


@settings(max_examples=60, deadline=None)
@given(bw=st.integers(1, 8), n=st.integers(1, 64).map(lambda x: 2 * x), rows=st.integers(1, 5),
       seed=st.integers(0, 2 ** 31 - 1))
def test_pack_unpack_round_trip(bw, n, rows, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 1 << bw, size=(rows, n), dtype=np.uint8)
    p = O.pack_run(codes, bw)
    assert p.shape == (rows, O.seg_bytes(bw, n)) and p.dtype == np.uint8
    assert np.array_equal(O.unpack_run(p, bw, n), codes)
    if bw <= 4:     # unused high bits of the last byte(s) are zero
        tail = O.unpack_run(p, bw, (p.shape[1] * 8) // bw)[:, n:]
        assert (tail == 0).all()


def test_three_bit_group_layout_matches_reference_formula():
    """8 codes -> 3 bytes exactly as quantizer.py:957-959 spells it out."""
    c = np.array([[1, 7, 5, 2, 0, 6, 3, 4]], dtype=np.uint8)
    b0 = c[0, 0] | (c[0, 1] << 3) | ((c[0, 2] << 6) & 0xFF)
    b1 = (c[0, 2] >> 2) | (c[0, 3] << 1) | (c[0, 4] << 4) | ((c[0, 5] << 7) & 0xFF)
    b2 = (c[0, 5] >> 1) | (c[0, 6] << 2) | (c[0, 7] << 5)
    assert O.pack_run(c, 3).tolist() == [[b0 & 0xFF, b1 & 0xFF, b2 & 0xFF]]


def test_combine_handles_empty_splits():
    po = np.random.default_rng(0).normal(size=(3, 2, HD))
    pl = np.array([[0.5, -np.inf], [-np.inf, -np.inf], [1.5, -np.inf]])
    out, lse = O.combine(po, pl)
    assert np.isfinite(out).all() and (out[1] == 0).all() and np.isneginf(lse[1])
    w = np.exp(np.array([0.5, 1.5]) - 1.5)
    np.testing.assert_allclose(out[0], (w[0] * po[0, 0] + w[1] * po[2, 0]) / w.sum())


def test_three_region_policy_matches_the_reference_hook():
    """The packed / fp16 split of the three-region cache against the reference's own policy, recorded by
    driving its _BufferedKVPatch hook (tests/golden/buffer_policy.npz: a 37-token prefill, then one token per
    forward, four (sink, window, block) settings): the oracle's closed form, the manager's bookkeeping, and the
    (start, end) ranges the manager would flush must all agree with what the hook did."""
    from blockgtq_b200 import BlockGTQKVManager
    g = load("buffer_policy")
    for si, (n_sink, window, bs) in enumerate(g["settings"].tolist()):
        mgr = BlockGTQKVManager(1, 2, 1, HD, max_seq_len=512, device="cpu", n_sink=n_sink, recent_window=window,
                                block_size=bs, use_cuda_graph=False)
        seqs, flushed = g[f"s{si}_seq"], g[f"s{si}_n_flushed"]
        calls, call_step = g[f"s{si}_flush_calls"], g[f"s{si}_flush_step"]
        prev = 0
        for step, (seq, nf) in enumerate(zip(seqs.tolist(), flushed.tolist())):
            avail = max(0, seq - n_sink)
            assert O.three_region_plan(seq, n_sink, window, bs) == (min(seq, n_sink), nf, avail - nf)
            assert mgr._region_sizes(seq) == (min(seq, n_sink), nf, avail - nf)
            assert mgr._flushed(avail) == nf
            # the hook's flush calls of this forward tile [n_sink + prev, n_sink + nf) in block_size pieces
            mine = [(n_sink + f, n_sink + f + bs) for f in range(prev, nf, bs)]
            assert calls[call_step == step].tolist() == [list(c) for c in mine]
            prev = nf


def test_oracle_prefill_attention_vs_reference_golden():
    """The reference's causal prefill kernel (run under the Triton interpreter, tests/golden/prefill.npz)
    against the oracle's per-query attention over the tokens each query may see."""
    import torch
    from blockgtq_b200 import calib
    g = load("prefill")
    avg, mn, mx, rt, vb = CASES[str(g["case"])]
    gqa, off = int(g["gqa"]), int(g["offset"])
    worst = 0.0
    for h in range(2):
        kt = calib.build_k_tables(None, None, head_dim=HD, avg_bits=avg, rotation_threshold=rt, min_bits=mn,
                                  max_bits=mx, bit_allocation=torch.from_numpy(g[f"h{h}_alloc"]))
        meta = oracle_meta(kt, calib.build_v_tables(HD, vb, 42 + h))
        sl = slice(h * gqa, (h + 1) * gqa)
        for b in range(2):
            for i in range(0, g["q"].shape[2], 5):
                lim = off + i + 1
                ro, _ = O.attend_packed(g["q_rot"][b, sl, i], g["k_packed"][b, h, :lim], g["k_norms"][b, h, :lim],
                                        g["v_packed"][b, h, :lim], g["v_norms"][b, h, :lim], meta, 1 / HD ** 0.5)
                worst = max(worst, np.abs(ro - g["out"][b, sl, i].astype(np.float64)).max())
    assert worst <= 2e-3, worst
