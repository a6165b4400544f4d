"""CPU tests of the host layer: calibration tables against the reference's, the allocator, the C-ABI
library (loads, exports every declared symbol, plans build) and the manager's bookkeeping."""
import ctypes as C
import hashlib
import os
import re

import numpy as np
import pytest
import torch

from helpers import CASES, HD, ROOT, load, tables_for
from blockgtq_b200 import _lib, calib, greedy_bit_allocation


def _sha(t):
    return hashlib.sha256(np.ascontiguousarray(t.numpy()).tobytes()).hexdigest()


@pytest.mark.parametrize("case", list(CASES))
def test_tables_equal_reference(case):
    g = load("tables_" + case)
    avg, mn, mx, rt, vb = CASES[case]
    for h in range(2):
        p = f"h{h}_"
        alloc = greedy_bit_allocation(torch.from_numpy(g[p + "scores"]), int(64 * avg), mn, mx)
        assert np.array_equal(alloc.numpy(), g[p + "alloc"])
        kt, vt = tables_for(case, h, g)
        assert np.array_equal(kt.head_perm.numpy(), g[p + "head_perm"])
        assert np.array_equal(kt.group_of.numpy(), g[p + "group_of"])
        assert np.array_equal(kt.pos_centroids.numpy(), g[p + "pos_centroids"])
        assert np.array_equal(kt.pos_boundaries.numpy(), g[p + "pos_boundaries"])
        assert np.array_equal(kt.code_lut.numpy(), g[p + "code_lut"])
        assert np.array_equal(kt.pos_to_cb.numpy(), g[p + "pos_to_cb"])
        assert np.array_equal(kt.lut_offsets.numpy(), g[p + "lut_off"])
        assert np.array_equal(kt.lut_inv_scales.numpy(), g[p + "lut_inv"])
        assert np.array_equal(np.array(kt.segments), g[p + "segments"])
        assert np.array_equal(kt.codebook_flat.numpy(), g[p + "codebook"])
        assert kt.total_packed_bytes == int(g[p + "total_packed_bytes"])
        pm = kt.pack_meta
        assert [pm["nopack_start"], pm["nopack_len"], pm["nopack_off"]] == g[p + "nopack"].tolist()
        assert _sha(kt.block_rot.T.contiguous()) == str(g[p + "rot_t_sha"])
        assert _sha(vt.rotation) == str(g[p + "v_rot_sha"])
        assert np.array_equal(vt.centroids.numpy(), g[p + "v_cents"])
        assert np.array_equal(vt.boundaries.numpy(), g[p + "v_bounds"])
    # end to end from calibration data (head 0 carries it)
    kt = calib.build_k_tables(torch.from_numpy(g["h0_cal_q"]).float(), torch.from_numpy(g["h0_cal_k"]).float(),
                              head_dim=HD, avg_bits=avg, rotation_threshold=rt, min_bits=mn, max_bits=mx)
    assert np.array_equal(kt.scores.numpy(), g["h0_scores"])
    assert np.array_equal(kt.bit_allocation.numpy(), g["h0_alloc"])
    assert np.array_equal(kt.block_rot.T.contiguous().numpy(), g["h0_rot_t"])


def test_allocator_edges():
    s = torch.tensor([1.0, 1.0, 4.0, 0.0])
    assert greedy_bit_allocation(s, 4, 1, 8).tolist() == [1, 1, 1, 1]          # budget == floor
    assert greedy_bit_allocation(s, 2, 1, 8).tolist() == [1, 1, 1, 1]          # budget below floor
    assert greedy_bit_allocation(s, 5, 1, 8).tolist() == [1, 1, 2, 1]
    assert greedy_bit_allocation(s, 6, 1, 8).tolist() == [2, 1, 2, 1]          # tie -> first index
    assert greedy_bit_allocation(s, 100, 1, 3).tolist() == [3, 3, 3, 1]        # zero score never gets a bit
    assert greedy_bit_allocation(torch.ones(3), 100, 2, 4).tolist() == [4, 4, 4]


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "bgtq.h")).read()
    declared = sorted(set(re.findall(r"^(?:int|int64_t|const char\*)\s+(bgtq_\w+)\s*\(", header, flags=re.M)))
    assert declared, "no declarations found"
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in bgtq.h but not exported"
    assert sorted(_lib.exported_symbols()) == declared
    assert lib.bgtq_abi_version() == 1
    assert lib.bgtq_desc_size() == C.sizeof(_lib.HeadDesc)
    assert lib.bgtq_error_string(-3) == b"misaligned pointer"


@pytest.mark.parametrize("case", list(CASES))
def test_descriptor_and_decode_plan(case):
    """Descriptor packing and the host-side decode plan (no GPU work)."""
    from blockgtq_b200.layer import _fill_desc
    descs = (_lib.HeadDesc * 2)()
    for h in range(2):
        kt, vt = tables_for(case, h)
        _fill_desc(descs[h], kt, vt)
        d = descs[h]
        assert d.n_seg == kt.n_groups and d.k_row_bytes == kt.total_packed_bytes
        assert [d.seg_bw[i] for i in range(d.n_seg)] == kt.group_bits
        assert bytes(d.head_perm) == bytes(kt.head_perm.numpy().astype(np.uint8))
        assert bytes(d.code_lut[d.n_seg - 1]) == bytes(kt.code_lut[d.n_seg - 1].numpy())
    for flags in (0, 1, 2, 3):
        plan = _lib.DecodePlan()
        assert _lib.lib().bgtq_decode_plan(C.byref(descs), 2, flags, C.byref(plan)) == 0
    assert _lib.lib().bgtq_decode_plan(C.byref(descs), 9, 0, C.byref(plan)) == -5
    assert _lib.lib().bgtq_decode_plan(None, 2, 0, C.byref(plan)) == -1
    descs[0].seg_len[0] = 3
    assert _lib.lib().bgtq_decode_plan(C.byref(descs), 2, 0, C.byref(plan)) == -1


def test_entry_points_reject_bad_arguments_without_a_gpu():
    L = _lib.lib()
    assert L.bgtq_decode(None, None, None, None, 0, 0, 0, None, 0, 0, 0, None, 0, 0, 0, None, 0, 0, 0,
                         1, 8, 2, 0, 10, 1, 0.1, None, None, None, None, 0, None) == -1
    assert L.bgtq_combine(None, None, 1, None, None, None, 1, 8, 2, None, 0, 0, None, None, 0, None) == -1
    assert L.bgtq_combine_ranks(None, 2, 8 * 129, 1, 8, None, 0, 0, 0, None) == -1
    import ctypes as C
    dummy = (C.c_float * 4)()           # never dereferenced: the stride check fails first
    assert L.bgtq_combine_ranks(C.addressof(dummy), 2, 8 * 128, 1, 8, C.addressof(dummy), 0, 0, 0, None) == -1
    assert L.bgtq_encode(None, None, None, None, 0, 0, 0, None, 0, 0, 0, 1, 2, 1, 0, None, 0, 0, 0, 8,
                         None, 0, 0, 0, 1, None, 0, 0, 0, None, 0, 0, 0, None, None, 0, None, 0, None, None) == -1
    # a destination range given on the host that leaves the cache is refused before anything is dereferenced
    d = (C.c_float * 4)()
    p = C.addressof(d)
    assert L.bgtq_encode(p, p, p, p, 0, 0, 0, p, 0, 0, 0, 1, 2, 4, 61, p, 0, 0, 0, 8,
                         p, 0, 0, 0, 1, p, 0, 0, 0, p, 0, 0, 0, None, None, 0, None, 64, None, None) == -1
    # fp16-region attention: key/value buffers must be 16-byte aligned with strides in multiples of 8 elements
    buf = (C.c_float * 64)()
    a = C.addressof(buf)
    a16 = (a + 15) & ~15
    args = lambda kb, sb: (a16, 1024, 128, kb, a16, sb, 128 * 8, 2, 3, 4, 0, 5, 1, 8, 2, 0.1, a16, a16, None)
    assert L.bgtq_buffer_attn(*args(a16 + 2, 4096)) == -3
    assert L.bgtq_buffer_attn(*args(a16, 4100)) == -3
    assert L.bgtq_buffer_attn(None, 0, 0, None, None, 0, 0, 0, 0, 4, 0, 5, 1, 8, 2, 0.1, None, None, None) == -1


def test_operators_refuse_cpu_tensors():
    from blockgtq_b200.layer import LayerTables, rotate_q
    kt, vt = tables_for("a3_1to8", 0)
    lt = LayerTables([kt], [vt], "cpu")
    with pytest.raises(RuntimeError, match="no CPU path"):
        rotate_q(lt, torch.zeros(1, 4, HD, dtype=torch.float16))


def test_manager_region_bookkeeping():
    from blockgtq_b200 import BlockGTQKVManager
    from oracle.bgtq_oracle import three_region_plan
    for n_sink, window, bs in [(4, 128, 1), (0, 16, 4), (2, 5, 3)]:
        m = BlockGTQKVManager(1, 8, 2, HD, 1024, n_sink=n_sink, recent_window=window, block_size=bs, device="cpu")
        for seq in range(0, 400, 7):
            assert m._region_sizes(seq) == three_region_plan(seq, n_sink, window, bs)
            _s, f, r = m._region_sizes(seq)
            assert r <= window + bs - 1 or seq - n_sink < window + bs
    m = BlockGTQKVManager(1, 8, 2, HD, 1024, device="cpu")
    assert m._region_sizes(77) == (0, 77, 0)


def test_calib_cache_round_trip(tmp_path):
    """Activations -> calib cache file (the reference's payload keys) -> the same tables."""
    import time
    from blockgtq_b200 import calib, load_calib_cache, save_calib_cache
    from helpers import synth_head
    gen = torch.Generator().manual_seed(3)
    data = {}
    for li in range(2):
        qk = [synth_head(gen, 128, 2) for _ in range(2)]
        data[li] = {"q": torch.stack([q for q, _ in qk]), "k": torch.stack([k for _, k in qk])}
    payload = save_calib_cache(tmp_path / "c.pt", data, model_name="tiny")
    assert payload["calib_k"].shape == (2, 2, 128, 128) and payload["calib_q"].shape == (2, 2, 256, 128)
    assert payload["q_per_kv"] == 2 and payload["n_q"] == 4
    back = load_calib_cache(tmp_path / "c.pt")
    t0 = time.time()
    for li in range(2):
        for h in range(2):
            a = calib.build_k_tables(data[li]["q"][h].float(), data[li]["k"][h].float(), head_dim=128, avg_bits=3.0)
            b = calib.build_k_tables(back[li]["q"][h].float(), back[li]["k"][h].float(), head_dim=128, avg_bits=3.0)
            assert torch.equal(a.bit_allocation, b.bit_allocation) and torch.equal(a.code_lut, b.code_lut)
    assert (time.time() - t0) / 8 < 2.0          # vectorised table construction: well under a second per head


def test_default_split_counts_for_the_benchmark_shapes():
    """Host-side rule for the number of partial slots per (batch, head) pair (148 SMs assumed without a GPU):
    items of at most one 512-token tile, about four per SM for small launches, at most 256 slots."""
    L = _lib.lib()
    assert L.bgtq_decode_default_splits(8, 2, 32768) == 64        # 1024 one-tile items over 148 CTAs
    assert L.bgtq_decode_default_splits(1, 8, 131072) == 256
    assert L.bgtq_decode_default_splits(32, 8, 16384) == 32
    assert L.bgtq_decode_default_splits(32, 8, 65536) == 128
    assert L.bgtq_decode_default_splits(1, 8, 4096) == 64         # 1024 units over 592 item slots: 2 units each
    assert L.bgtq_decode_default_splits(1, 1, 100) == 4 and L.bgtq_decode_default_splits(64, 8, 1024) == 2
    assert L.bgtq_decode_default_splits(1, 1, 0) == 1 and L.bgtq_decode_default_splits(4, 2, 32) == 1
    assert L.bgtq_decode_default_splits(1, 1, 1 << 20) == 256     # capped: 128-unit items


def test_baked_q_projection_reproduces_the_query_rotation():
    """bake_permutation_into_qproj folds head permutation + rotation into q_proj: projecting with the baked
    weight (and bias) must give what rotating the original projection's output gives (the oracle's rotate_q,
    itself pinned on the reference's rotate_q_for_packed_kernel by the decode goldens' q_rot)."""
    from blockgtq_b200 import BlockGTQQuantizer
    from oracle import bgtq_oracle as O
    from helpers import oracle_meta
    gt = load("tables_a3_1to8")
    gen = torch.Generator().manual_seed(3)
    n_kv, gqa = 2, 2
    qs = []
    for h in range(n_kv):
        z = BlockGTQQuantizer(HD, avg_bits=3.0, device="cpu")
        z.calibrate(None, None, bit_allocation=torch.from_numpy(gt[f"h{h}_alloc"]))
        z.init_v_quantizer(v_bits=3, seed=42 + h)
        qs.append(z)
    W = torch.randn(n_kv * gqa * HD, 96, generator=gen)
    bias = torch.randn(n_kv * gqa * HD, generator=gen)
    x = torch.randn(7, 96, generator=gen)
    q_plain = (x @ W.T + bias).reshape(7, n_kv * gqa, HD)
    Wb, bb = W.clone(), bias.clone()
    for h in range(n_kv):
        assert not qs[h]._q_perm_baked
        qs[h].bake_permutation_into_qproj(Wb, kv_head_idx=h, n_kv_heads=n_kv, n_q_heads=n_kv * gqa, q_proj_bias=bb)
        assert qs[h]._q_perm_baked
    q_baked = (x @ Wb.T + bb).reshape(7, n_kv * gqa, HD)
    for h in range(n_kv):
        meta = oracle_meta(qs[h]._tables, qs[h]._v_tables)
        sl = slice(h * gqa, (h + 1) * gqa)
        want = q_plain[:, sl].reshape(-1, HD).double().numpy()[:, meta["head_perm"]] @ meta["rot_t"].astype(np.float64)
        got = q_baked[:, sl].reshape(-1, HD).double().numpy()
        assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
        # and the fp16 rotation the decode kernels consume agrees with the oracle's fp16 rotate_q to an ulp
        r16 = O.rotate_q(q_plain[:, sl].reshape(-1, HD).half().numpy(), meta).astype(np.float32)
        assert np.abs(r16 - want).max() <= 4e-3 * np.abs(want).max()


def test_bake_helpers_rewrite_every_layers_q_proj():
    """BlockGTQKVManager.bake_q_permutations and calibration.bake_q_rotations walk the model's layers and
    fold each KV head's permutation + rotation into the q_proj rows of its query group (weights and flags
    checked against the per-head formula).  Note: with rotary embeddings applied AFTER q_proj the baked
    projection is not equivalent to rotating the post-RoPE query (the block rotation mixes dims of different
    RoPE blocks); the reference has the same limitation and leaves a TODO in its decode path
    (blockgtq/packed_kv_manager.py:318-322), so no model-level equivalence is claimed."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from blockgtq_b200 import BlockGTQKVManager
    from blockgtq_b200.calibration import bake_q_rotations
    from helpers import synth_head
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      num_hidden_layers=2, intermediate_size=128, vocab_size=64, max_position_embeddings=128)
    model = LlamaForCausalLM(cfg).eval()
    L, nq, nkv = 2, 4, 2
    gen = torch.Generator().manual_seed(11)
    mgr = BlockGTQKVManager(L, nq, nkv, HD, max_seq_len=64, batch_size=1, device="cpu")
    for li in range(L):
        cal = [synth_head(gen, 128, nq // nkv) for _ in range(nkv)]
        mgr.calibrate(li, torch.stack([c[0] for c in cal]).float(), torch.stack([c[1] for c in cal]).float())
    before = [model.model.layers[li].self_attn.q_proj.weight.data.clone() for li in range(L)]
    twin = LlamaForCausalLM(cfg).eval()
    twin.load_state_dict(model.state_dict())
    mgr.bake_q_permutations(model, nkv, nq)
    for li in range(L):
        w = model.model.layers[li].self_attn.q_proj.weight.data
        for h in range(nkv):
            z = mgr.quantizers[li][h]
            assert z._q_perm_baked
            for g in range(nq // nkv):
                s = (h * (nq // nkv) + g) * HD
                want = (z._block_rot_T.float().T @ before[li][s:s + HD][z._head_perm].float())[z._pack_perm]
                assert torch.allclose(w[s:s + HD], want.to(w.dtype), atol=1e-5, rtol=1e-4)
    # the calibration-module helper does the same walk
    for row in mgr.quantizers:
        for z in row:
            z._q_perm_baked = False
    bake_q_rotations(twin, mgr.quantizers, L, nkv, nq)
    for li in range(L):
        assert torch.equal(twin.model.layers[li].self_attn.q_proj.weight.data,
                           model.model.layers[li].self_attn.q_proj.weight.data)
    assert all(z._q_perm_baked for row in mgr.quantizers for z in row)


def test_decode_partition_tables():
    """bgtq_decode_partition: header = what the kernel derives for the launch; offsets non-decreasing from 0 to
    the item count; CTAs whose range straddles two (batch, head) pairs get fewer items than those inside one
    pair; shapes where the equal-count split is already as good carry a header that matches no launch."""
    L = _lib.lib()

    def table(B, H, T, ns, n_cta):
        buf = (C.c_int32 * (n_cta + 5))()
        assert L.bgtq_decode_partition(B, H, T, ns, n_cta, buf, n_cta + 5) == 0
        return np.frombuffer(buf, dtype=np.int32).copy()

    for B, H, T, ns, n_cta in [(8, 2, 32768, 64, 148), (8, 2, 8192, 37, 148), (8, 2, 65536, 128, 148),
                               (32, 8, 16384, 32, 148), (1, 2, 8192, 256, 148), (8, 2, 100, 4, 64),
                               (8, 2, 0, 4, 64), (2, 2, 33, 7, 28), (5, 3, 12345, 11, 132)]:
        t = table(B, H, T, ns, n_cta)
        units = (T + 31) // 32
        c_units = max(1, -(-units // ns))
        n_live = -(-units // c_units)
        assert t[1] == B * H and t[2] == n_cta and t[3] == c_units
        assert t[0] in (n_live, -1)
        off = t[4:]
        assert off[0] == 0 and off[-1] == B * H * n_live and (np.diff(off) >= 0).all()
    # the headline shape: 16 pairs of 64 one-tile items on 148 CTAs; ranges that straddle a pair take 6, the others 7
    t = table(8, 2, 32768, 64, 148)
    assert t[0] == 64
    off = t[4:].astype(np.int64)
    n = np.diff(off)
    straddles = (off[:-1] // 64) != ((off[1:] - 1) // 64)
    assert straddles.sum() == 12 and (n[straddles] == 6).all() and (n[~straddles] == 7).all()
    # nothing to gain: many short pairs per CTA
    assert table(32, 8, 16384, 32, 148)[0] == -1
    # argument checks
    buf = (C.c_int32 * 8)()
    assert L.bgtq_decode_partition(8, 2, 1000, 4, 64, buf, 8) == -1
    assert L.bgtq_decode_partition(0, 2, 1000, 4, 64, buf, 8) == -1
    assert L.bgtq_decode_partition(8, 2, 1000, 4, 64, None, 100) == -1
    assert L.bgtq_decode_plan_set_partition(None, None) == -1


def test_decode_plan_option_setters_check_their_arguments():
    """Row strides, early fetch and the item-range table are options of a decode plan: the setters take only what
    the kernel can honour (strides inside the launch wrapper's limits, before the specialisation that bakes them
    in; a non-negative row count; a 4-byte aligned table) and leave the plan usable."""
    from test_cpu_decode_plan import Plan, _fill_desc
    L = _lib.lib()
    descs = (_lib.HeadDesc * 2)()
    for h in range(2):
        _fill_desc(descs[h], *tables_for("a3_1to8", h))
    raw = _lib.DecodePlan()
    assert L.bgtq_decode_plan(C.byref(descs), 2, 0, C.byref(raw)) == 0
    view = lambda: Plan.from_buffer_copy(bytes(raw.opaque)[:C.sizeof(Plan)])
    assert list(view().row_st) == [0, 0, 0, 0] and view().early_fresh == 0 and not view().partition
    assert L.bgtq_decode_plan_set_row_strides(C.byref(raw), 57, 8, 48, 1) == 0
    assert list(view().row_st) == [57, 16, 48, 2]                       # bytes, like the kernel's parameters
    assert L.bgtq_decode_plan_set_row_strides(C.byref(raw), 161, 8, 48, 1) == -2
    assert L.bgtq_decode_plan_set_row_strides(C.byref(raw), 57, 17, 48, 1) == -2
    assert L.bgtq_decode_plan_set_row_strides(C.byref(raw), 0, 0, 0, 0) == 0 and list(view().row_st) == [0, 0, 0, 0]
    assert L.bgtq_decode_plan_set_row_strides(None, 57, 8, 48, 1) == -1
    assert L.bgtq_decode_plan_set_early_fetch(C.byref(raw), 1) == 0 and view().early_fresh == 1
    assert L.bgtq_decode_plan_set_early_fetch(C.byref(raw), -1) == -1
    assert L.bgtq_decode_plan_set_early_fetch(C.byref(raw), 0) == 0 and view().early_fresh == 0
    assert L.bgtq_decode_plan_set_partition(C.byref(raw), C.c_void_p(0x1002)) == -3
    assert L.bgtq_decode_plan_set_partition(C.byref(raw), C.c_void_p(0x1000)) == 0 and view().partition == 0x1000
    assert L.bgtq_decode_plan_set_partition(C.byref(raw), None) == 0 and not view().partition
    assert L.bgtq_decode_grid_size(8, 2, 64) == 148 and L.bgtq_decode_grid_size(1, 2, 4) == 8
    assert L.bgtq_decode_grid_size(0, 2, 4) == -1
