"""The allocation-free decode entry point (bgtq_decode_combined_noalloc) against the regular
decode + combine pair, through the C ABI.

Some users of the library cannot hand it scratch memory: they run where device allocation is not
allowed or not theirs to make (inside a captured stream sequence, inside a host framework's plugin
slot, next to a memory pool they do not own).  For them the split partials live in a fixed array
inside the library.  The array is shared by all calls, so the test calls twice in a row with
different data and checks that the second answer is not polluted by the first."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import HD, load, tables_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_noalloc(lt, q_rot, kp, kn, vp, vn, T, n_splits):
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import _strides3
    B, n_q, _ = q_rot.shape
    out = torch.empty(B, n_q, HD, dtype=torch.float16, device=DEV)
    lse = torch.empty(B, n_q, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    plan = lt.plan(0)
    rc = _lib.lib().bgtq_decode_combined_noalloc(
        C.addressof(plan), lt.desc_dev.data_ptr(), q_rot.data_ptr(),
        kp.data_ptr(), *_strides3(kp), kn.data_ptr(), *_strides3(kn), vp.data_ptr(), *_strides3(vp),
        vn.data_ptr(), vn.stride(0), vn.stride(1), vn.stride(2),
        B, n_q, lt.n_kv, 0, T, n_splits, 1.0 / HD ** 0.5,
        lt.v_rot.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), lse.data_ptr(), status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out, lse


def test_noalloc_matches_regular_entry_point_twice():
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import LayerTables, combine, decode
    outs = []
    for case, n_splits in (("a3_1to8", 5), ("a3_1to6", 2)):      # two calls in a row, different heads and data
        gt, gd = load("tables_" + case), load("decode_" + case)
        tabs = [tables_for(case, h, gt) for h in range(2)]
        lt = LayerTables([t[0] for t in tabs], [t[1] for t in tabs], DEV)
        q_rot = torch.from_numpy(gd["q_rot"][:, :, 0]).to(DEV).contiguous()
        kp, kn = torch.from_numpy(gd["k_packed"]).to(DEV), torch.from_numpy(gd["k_norms"]).to(DEV)
        vp, vn = torch.from_numpy(gd["v_packed"]).to(DEV), torch.from_numpy(gd["v_norms"]).to(DEV)
        T = kp.shape[2]
        got, got_lse = _run_noalloc(lt, q_rot, kp, kn, vp, vn, T, n_splits)
        po, pl = decode(lt, q_rot, kp, kn, vp, vn, 0, T, n_splits=n_splits)
        want, _, want_lse = combine(po, pl, lt.n_kv, v_rot=lt.v_rot, want_lse=True)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (got.float() - want.float()).abs().max()
        assert torch.equal(got_lse, want_lse)
        err = np.abs(got.cpu().numpy().astype(np.float64) - gd["out"][:, :, 0].astype(np.float64)).max()
        assert err <= 2e-3
        outs.append(got)
    # the size limit is enforced with a clear error code, before any GPU work
    rc = _lib.lib().bgtq_decode_combined_noalloc(None, None, None, None, 0, 0, 0, None, 0, 0, 0, None, 0, 0, 0,
                                                 None, 0, 0, 0, 64, 64, 8, 0, 10, 3, 0.1, None, 1, 0, 0, None, None,
                                                 None)
    assert rc == -5
