"""Host side of the decode kernel, checked without a GPU: the launch plan and the lookup-table image
(``bgtq_decode_plan`` / ``bgtq_decode_build_image``) are read back through a ctypes mirror of the plan and
driven through a lane-by-lane NumPy restatement of the kernel's address arithmetic (unit loads, rotates,
masks, OR-ed table bases, query-fragment positions).  Every (token, packed position) of golden packed rows
must come out as the codebook value of the reference's unpacked code."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import HD, load, tables_for

from blockgtq_b200 import _lib
from blockgtq_b200.layer import _fill_desc

MAX_STEPS = 20


class Seg(C.Structure):
    _fields_ = [("kind", C.c_uint8), ("bw", C.c_uint8), ("q", C.c_uint8), ("f16_norm", C.c_uint8),
                ("bit0", C.c_uint16), ("lane_bits", C.c_uint16), ("tbl", C.c_uint32), ("esh", C.c_uint8),
                ("rep_log2", C.c_uint8), ("ent_log2", C.c_uint8), ("norm_idx", C.c_uint8)]


class StepQ(C.Structure):
    _fields_ = [("pos", C.c_uint8), ("q", C.c_uint8), ("end", C.c_uint8), ("c4", C.c_uint8)]


class HeadPlan(C.Structure):
    _fields_ = [("n_steps", C.c_int32), ("n_seg", C.c_int32), ("v_tbl", C.c_uint32), ("image_bytes", C.c_uint32),
                ("seg", Seg * 8), ("steps", StepQ * MAX_STEPS)]


class Plan(C.Structure):
    _fields_ = [("n_heads", C.c_int32), ("flags", C.c_int32), ("v_bits", C.c_int32), ("v_sbits", C.c_int32),
                ("v_rep_log2", C.c_uint32), ("lut_bytes", C.c_uint32), ("image", C.c_void_p), ("jit_kernel", C.c_void_p), ("partition", C.c_void_p), ("early_fresh", C.c_int32), ("row_st", C.c_int32 * 4),
                ("head", HeadPlan * 8)]


def _plan_and_image(descs, n_kv, flags):
    L = _lib.lib()
    raw = _lib.DecodePlan()
    assert L.bgtq_decode_plan(C.byref(descs), n_kv, flags, C.byref(raw)) == 0
    n = L.bgtq_decode_image_bytes(C.byref(raw))
    assert n > 0
    img = np.zeros(n, dtype=np.uint8)
    assert L.bgtq_decode_build_image(C.byref(raw), C.byref(descs), img.ctypes.data, n) == 0
    assert L.bgtq_decode_build_image(C.byref(raw), C.byref(descs), img.ctypes.data, n - 1) == -1
    plan = Plan.from_buffer_copy(bytes(raw.opaque)[:C.sizeof(Plan)])
    return plan, img


def _rotl(x, n):
    n &= 31
    return ((x << n) | (x >> (32 - n))) & 0xFFFFFFFF if n else x


def _bits32(row, bit):
    """32 bits of the byte stream ``row`` starting at bit ``bit`` (what two aligned loads + a funnel shift give)."""
    b0 = bit >> 3
    chunk = int.from_bytes(bytes(row[b0:b0 + 8]), "little")
    return (chunk >> (bit & 7)) & 0xFFFFFFFF


def _kernel_values(row, sg, img, lane):
    """fp16 bit patterns the kernel feeds the MMA for lane (r, j = lane & 3): list over k-tiles of four values
    (codes c4 .. c4+3 of the lane's run), or None where the kernel skips the lookup."""
    j = lane & 3
    kind, q = sg.kind, sg.q
    sb = kind
    cap = 8 if kind == 3 else 32 // sb
    lbit = sg.bit0 + j * sg.lane_bits
    tb = sg.tbl + ((lane & ((1 << sg.rep_log2) - 1)) << sg.ent_log2)
    words = img.view(np.uint32)

    def w32(addr):
        assert addr % 4 == 0
        return int(words[addr // 4])

    out = []
    for c in range(0, q, cap):
        cur = _bits32(row, lbit + c * sb)
        n = q - c
        for t in range(cap // 4):
            if 4 * t >= n:
                break
            full = n - 4 * t >= 4
            if kind == 1:
                fw = 4 * sb
                mask = ((1 << fw) - 1) << sg.esh
                a = (_rotl(cur, (32 + sg.esh - fw * t) & 31) & mask) | tb
                assert a % 8 == 0
                lo, hi = w32(a), w32(a + 4)
            elif kind <= 4:
                fw = 2 * sb
                mask = ((1 << fw) - 1) << sg.esh
                lo = w32((_rotl(cur, (64 + sg.esh - 2 * fw * t) & 31) & mask) | tb)
                hi = w32((_rotl(cur, (64 + sg.esh - 2 * fw * t - fw) & 31) & mask) | tb) if full else None
            else:
                mask = ((1 << sg.bw) - 1) << sg.esh
                c0 = w32((_rotl(cur, sg.esh) & mask) | tb)
                c1 = w32((_rotl(cur, sg.esh + 24) & mask) | tb)
                lo = (c0 & 0xFFFF) | ((c1 & 0xFFFF) << 16)
                assert c0 >> 16 == c0 & 0xFFFF
                if full:
                    c2 = w32((_rotl(cur, sg.esh + 16) & mask) | tb)
                    c3 = w32((_rotl(cur, sg.esh + 8) & mask) | tb)
                    hi = (c2 & 0xFFFF) | ((c3 & 0xFFFF) << 16)
                else:
                    hi = None
            vals = [lo & 0xFFFF, lo >> 16] + ([None, None] if hi is None else [hi & 0xFFFF, hi >> 16])
            out.append(vals)
    return out


@pytest.mark.parametrize("case", ["a3_1to6", "a3_1to8", "a2_1to8", "a4_rt1", "u3"])
def test_plan_and_image_reproduce_every_code(case):
    enc = load("encode_" + case)
    n_kv = enc["k_packed"].shape[0]
    descs = (_lib.HeadDesc * n_kv)()
    tabs = [tables_for(case, h) for h in range(n_kv)]
    for h in range(n_kv):
        _fill_desc(descs[h], *tabs[h])
    plan, img = _plan_and_image(descs, n_kv, 0)
    assert plan.n_heads == n_kv and plan.lut_bytes % 128 == 0 and plan.lut_bytes * n_kv == img.size
    rng = np.random.default_rng(0)
    for h in range(n_kv):
        hp, kt = plan.head[h], tabs[h][0]
        himg = img[h * plan.lut_bytes:(h + 1) * plan.lut_bytes]
        cb = kt.codebook_flat.view(torch.int16).numpy().astype(np.uint16)
        segs = kt.segments
        assert hp.n_seg == len(segs) and hp.image_bytes <= plan.lut_bytes
        # tables: aligned to their own size, inside the image, not overlapping
        spans = []
        for s in range(hp.n_seg):
            sg = hp.seg[s]
            size = ((16 if sg.kind <= 2 else 64 if sg.kind == 3 else (1 << sg.bw) if sg.kind == 8 else 256)
                    << sg.ent_log2) << sg.rep_log2
            assert sg.esh == sg.ent_log2 + sg.rep_log2 and sg.tbl % size == 0 and size <= 16384
            spans.append((sg.tbl, sg.tbl + size))
        v_size = ((1 << (2 * plan.v_sbits)) * 4) << plan.v_rep_log2
        assert hp.v_tbl % v_size == 0
        spans.append((hp.v_tbl, hp.v_tbl + v_size))
        spans.sort()
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= hp.image_bytes
        # K data path on a few golden rows
        rows = rng.choice(enc["k_packed"].shape[1], size=6, replace=False)
        step_i = 0
        for s, (bw, start, length, pack_off, lut_off, _ni) in enumerate(segs):
            sg = hp.seg[s]
            assert sg.q % 2 == 0 and 4 * sg.q >= length and sg.bw == bw and sg.norm_idx == s
            n_tiles = (sg.q + 3) // 4
            for t in range(n_tiles):
                st = hp.steps[step_i + t]
                assert (st.pos, st.q, st.end, st.c4) == (start + 4 * t, sg.q, start + length, 4 * t)
            for row_i in rows:
                row = np.concatenate([enc["k_packed"][h, row_i], np.zeros(16, np.uint8)])
                codes = enc["k_codes"][h, row_i]
                for lane in (0, 1, 2, 3, 13, 30):
                    j = lane & 3
                    tiles = _kernel_values(row, sg, himg, lane)
                    assert len(tiles) == n_tiles
                    for t, vals in enumerate(tiles):
                        for e, got in enumerate(vals):
                            pos = start + j * sg.q + 4 * t + e
                            if pos < start + length and 4 * t + e < sg.q:
                                assert got is not None and got == cb[lut_off + int(codes[pos])], (case, h, s, lane, t, e)
            step_i += n_tiles
        assert step_i == hp.n_steps
        # every packed position is owned by exactly one (lane, code) whose query fragment is non-zero
        owned = np.zeros(HD, dtype=int)
        for i in range(hp.n_steps):
            st = hp.steps[i]
            for j in range(4):
                for e in range(4):
                    pos = st.pos + j * st.q + e
                    if e >= 2 and st.c4 + 2 >= st.q:
                        continue
                    if (pos - (pos & 1)) < st.end:      # the kernel tests the first position of each fp16 pair
                        owned[pos] += 1
        assert (owned == 1).all()
        # V table: entry e = (code of token A, code of token B) of one dim
        vl = tabs[h][1].lut_f16.view(torch.int16).numpy().astype(np.uint16)
        vb = plan.v_sbits
        vw = himg.view(np.uint32)
        for e in range(1 << (2 * vb)):
            for rep in (0, (1 << plan.v_rep_log2) - 1):
                w = int(vw[(hp.v_tbl + (e << (2 + plan.v_rep_log2)) + 4 * rep) // 4])
                assert w & 0xFFFF == vl[e & ((1 << vb) - 1)] and w >> 16 == vl[e >> vb]


def test_plan_for_the_mixed_layout_and_limits():
    case = "a3_1to8"
    enc = load("encode_" + case)
    descs = (_lib.HeadDesc * 2)()
    tabs = [tables_for(case, h) for h in range(2)]
    for h in range(2):
        _fill_desc(descs[h], *tabs[h])
    plan, img = _plan_and_image(descs, 2, _lib.DEC_K_MIXED | _lib.DEC_V_NIBBLE)
    assert plan.v_sbits == 4
    for h in range(2):
        hp, kt = plan.head[h], tabs[h][0]
        himg = img[h * plan.lut_bytes:(h + 1) * plan.lut_bytes]
        cb = kt.codebook_flat.view(torch.int16).numpy().astype(np.uint16)
        nopack_start = kt.pack_meta["nopack_start"]
        for s, (bw, start, length, pack_off, lut_off, _ni) in enumerate(kt.segments):
            sg = hp.seg[s]
            assert sg.kind == (4 if bw <= 4 else 8)
            for row_i in (0, 11, 42):
                row = np.concatenate([enc["k_mixed"][h, row_i], np.zeros(16, np.uint8)])
                codes = enc["k_codes"][h, row_i]
                for lane in (0, 5, 18, 31):
                    j = lane & 3
                    for t, vals in enumerate(_kernel_values(row, sg, himg, lane)):
                        for e, got in enumerate(vals):
                            pos = start + j * sg.q + 4 * t + e
                            if pos < start + length and 4 * t + e < sg.q:
                                assert got == cb[lut_off + int(codes[pos])], (h, s, lane, t, e, nopack_start)
    L = _lib.lib()
    raw = _lib.DecodePlan()
    assert L.bgtq_decode_image_bytes(None) == -1
    assert L.bgtq_decode_plan_set_image(C.byref(raw), 8) == -3          # image must be 16-byte aligned
    assert L.bgtq_decode_plan_set_image(None, 0) == -1


@pytest.mark.parametrize("case,flags", [("a3_1to8", 0), ("a2_1to8", 0), ("a4_rt1", 0), ("u3", 0), ("a3_1to8", 3)])
def test_specialised_kernel_source_compiles_for_sm100a(case, flags):
    """The run-time (NVRTC) specialisation of the decode kernel for a layer's heads compiles without a GPU;
    loading it needs one and is covered by the GPU tests."""
    descs = (_lib.HeadDesc * 2)()
    for h in range(2):
        _fill_desc(descs[h], *tables_for(case, h))
    L = _lib.lib()
    raw = _lib.DecodePlan()
    assert L.bgtq_decode_plan(C.byref(descs), 2, flags, C.byref(raw)) == 0
    log = C.create_string_buffer(1 << 16)
    rc = L.bgtq_decode_plan_specialize(C.byref(raw), 1, log, len(log))
    if rc == -2:
        pytest.skip("NVRTC is not installed here: " + log.value.decode())
    assert rc == 0, log.value.decode(errors="replace")
    assert " error" not in log.value.decode(errors="replace")
    plan = Plan.from_buffer_copy(bytes(raw.opaque)[:C.sizeof(Plan)])
    assert L.bgtq_decode_plan_specialize(None, 1, None, 0) == -1
