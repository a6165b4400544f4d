#!/usr/bin/env python
"""Benchmark of the packed-cache decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference|triton]

One "step" is one decode step of the hot path over every layer of the workload:
rotate_q -> encode/append the new token's K,V -> fused packed decode -> combine, for all batch
entries and KV heads (the model's projections and MLP are not part of this path).  Rank 0 prints
one JSON line.  With N > 1 (torchrun, one rank per GPU) every rank holds its own batch slice
(weak scaling, no collective on the data path); the time is the max over ranks.

--impl reference times the reference project's own CPU path (its unaccelerated quantise-dequantise +
attention, imported from baseline/_ref when that git-ignored copy of the reference package is present,
else the NumPy restatement under oracle/) on the host cores.  --impl triton times the reference's own
Triton decode path on this GPU (baseline/_ref again; it never touches this repository's package); the
default run carries that figure as config.reference_triton.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

HD = 128

WORKLOADS = {
    # BASELINE.json configs[1]: Qwen2.5-3B shape, K3V3 packed cache, batch 8 per GPU, context 32768
    "qwen2.5-3b_k3v3_b8_t32768": dict(layers=36, n_q=16, n_kv=2, batch=8, ctx=32768, k_bits=3.0, v_bits=3,
                                      theta=1e6, n_sink=0, window=0),
    # BASELINE.json configs[2]: Llama-3.1-8B shape, K2V2, batch 32, context 16384, fp16 sink 4 + window 128
    "llama3.1-8b_k2v2_b32_t16384_sink4_win128": dict(layers=32, n_q=32, n_kv=8, batch=32, ctx=16384, k_bits=2.0,
                                                     v_bits=2, theta=5e5, n_sink=4, window=128),
    # BASELINE.json configs[3]: one 131072-token sequence, Llama-3.1-8B shape, K2V2, sequence chunks across
    # GPUs with one all-gather of (O, LSE) per layer (strong scaling: the total context is fixed)
    "llama3.1-8b_k2v2_b1_t131072_seqshard": dict(layers=32, n_q=32, n_kv=8, batch=1, ctx=131072, k_bits=2.0,
                                                 v_bits=2, theta=5e5, n_sink=0, window=0, mode="seq"),
    # BASELINE.json configs[4]: bulk (prefill) encode, Mistral-Nemo-12B shape, 4 x 32768 tokens per layer into the
    # BlockGTQKVManager layout, then single-token appends; two layers with separate inputs stand for the 40
    "mistral-nemo-12b_k3v3_encode_b4_t32768": dict(layers=2, n_q=32, n_kv=8, batch=4, ctx=32768, k_bits=3.0,
                                                   v_bits=3, theta=1e6, n_sink=0, window=0, mode="encode"),
    # packed-cache prefill attention (the attention half of layer-major prefill): Llama-3.1-8B shape, one
    # 16384-token prompt, K3V3; a step = bulk encode + causal prefill attention of one layer
    "llama3.1-8b_k3v3_prefill_t16384": dict(layers=1, n_q=32, n_kv=8, batch=1, ctx=16384, k_bits=3.0, v_bits=3,
                                            theta=5e5, n_sink=0, window=0, mode="prefill"),
    # small variant of configs[2] for quick runs and profiler captures
    "llama3.1-8b_k2v2_b32_t16384_sink4_win128_4layers": dict(layers=4, n_q=32, n_kv=8, batch=32, ctx=16384,
                                                             k_bits=2.0, v_bits=2, theta=5e5, n_sink=4, window=128),
    # small variant of configs[1] for quick runs and profiler captures
    "qwen2.5-3b_k3v3_b8_t32768_4layers": dict(layers=4, n_q=16, n_kv=2, batch=8, ctx=32768, k_bits=3.0, v_bits=3,
                                              theta=1e6, n_sink=0, window=0),
}
DEFAULT = "qwen2.5-3b_k3v3_b8_t32768"
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


TRAFFIC_SOURCES = ["blockgtq_b200/csrc/bgtq_decode_kernel.cuh", "blockgtq_b200/csrc/bgtq_decode_plan.cu",
                   "blockgtq_b200/csrc/bgtq_plan.h", "blockgtq_b200/csrc/bgtq_decode.cu",
                   "blockgtq_b200/csrc/bgtq_decode_jit.cu", "blockgtq_b200/csrc/bgtq_common.cuh"]


def sources_key(files):
    import hashlib
    h = hashlib.sha256()
    for f in files:
        h.update(open(os.path.join(ROOT, f), "rb").read())
    return h.hexdigest()[:16]


def dram_traffic(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture
    recorded in profiles/dram_traffic.json (which names the command and the kernel source it was taken
    with).  None when there is no record for the workload or the kernel source changed since the capture."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))[workload]
    except Exception:
        return None
    try:
        return rec["bytes_per_launch"] if sources_key(rec.get("sources", [])) == rec.get("sources_sha16") else None
    except OSError:
        return None


def synth_keys(gen, shape_bt, theta, device):
    """Post-RoPE keys (B, T, 128) fp16: N(0,1) x lognormal(0,1) per-RoPE-block scale, two blocks x8."""
    B, T = shape_bt
    s = torch.exp(torch.randn(HD // 2, generator=gen, device=device))
    s[torch.randperm(HD // 2, generator=gen, device=device)[:2]] *= 8
    scale = torch.cat([s, s])
    x = (torch.randn(B, T, HD, generator=gen, device=device) * scale).half().float()
    half = HD // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=device) / half))
    ang = torch.arange(T, device=device).float()[:, None] * inv[None, :]
    c, sn = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * sn, a * sn + b * c], dim=-1).half()


def build_manager(w, device, seed, extra_tokens, ctx=None, graph=None):
    """Calibrate every (layer, head) on 2048 synthetic tokens, then bulk-encode the context."""
    from blockgtq_b200 import BlockGTQKVManager
    gen = torch.Generator(device=device).manual_seed(seed)
    L, n_q, n_kv, B = w["layers"], w["n_q"], w["n_kv"], w["batch"]
    T = w["ctx"] if ctx is None else ctx
    gqa = n_q // n_kv
    mgr = BlockGTQKVManager(L, n_q, n_kv, HD, max_seq_len=T + extra_tokens, batch_size=B, k_avg_bits=w["k_bits"],
                            v_bits=w["v_bits"], device=device, n_sink=w["n_sink"], recent_window=w["window"],
                            use_cuda_graph=graph)
    for li in range(L):
        ck = torch.stack([synth_keys(gen, (1, 2048), w["theta"], device)[0] for _ in range(n_kv)])
        cq = torch.stack([synth_keys(gen, (gqa, 2048), w["theta"], device).reshape(-1, HD) for _ in range(n_kv)])
        mgr.calibrate(li, cq.float(), ck.float())
    chunk = 8192
    for li in range(L):
        for t in range(0, T, chunk):
            n = min(chunk, T - t)
            k = torch.stack([synth_keys(gen, (B, n), w["theta"], device) for _ in range(n_kv)], dim=1)
            v = torch.randn(B, n_kv, n, HD, generator=gen, device=device).half()
            mgr._append_tokens(li, k, v, t)
    mgr.seq_len = T
    torch.cuda.synchronize()
    return mgr, gen


def clocks_sampler(device_index):
    q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    try:
        return subprocess.Popen(["nvidia-smi", "-i", str(device_index), f"--query-gpu={q}",
                                 "--format=csv,noheader,nounits", "-lms", "20"],
                                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
        return None


def clocks_summary(proc):
    if proc is None:
        return None
    proc.terminate()
    try:
        out = proc.communicate(timeout=5)[0]
    except Exception:
        return None
    sm, mx, reasons = [], 0, set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in out.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 6:
            continue
        try:
            sm.append(float(f[0]))
            mx = max(mx, float(f[1]))
        except ValueError:
            continue
        for n, v in zip(names, f[2:6]):
            if v.lower().startswith("active"):
                reasons.add(n)
    if not sm:
        return None
    return {"sm_mhz": statistics.median(sm), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_decode_sample(w, seed=0, t_sample=None):
    """Time the oracle's decode (unpack + dequantise + attention) for ONE (batch, KV-head) pair of one
    layer on the host cores; returns (seconds per pair, description)."""
    from helpers import oracle_meta
    from blockgtq_b200 import calib
    from oracle import bgtq_oracle as O
    T = t_sample or w["ctx"]
    gqa = w["n_q"] // w["n_kv"]
    gen = torch.Generator().manual_seed(seed)
    ck = synth_keys(gen, (1, 2048), w["theta"], "cpu")[0]
    cq = synth_keys(gen, (gqa, 2048), w["theta"], "cpu").reshape(-1, HD)
    kt = calib.build_k_tables(cq.float(), ck.float(), head_dim=HD, avg_bits=w["k_bits"])
    vt = calib.build_v_tables(HD, w["v_bits"], 42)
    meta = oracle_meta(kt, vt)
    k = synth_keys(gen, (1, T), w["theta"], "cpu")[0].numpy()
    v = torch.randn(T, HD, generator=gen).half().numpy()
    ek = O.encode_k_packed(k, meta)
    ev = O.encode_v(v, meta)
    kn16 = ek["norms"].astype(np.float16)
    q = O.rotate_q(synth_keys(gen, (gqa, 1), w["theta"], "cpu")[:, 0].numpy(), meta)
    t0 = time.perf_counter()
    reps = 0
    while True:
        O.attend_packed(q, ek["packed"], kn16, ev["packed"], ev["norms"], meta, 1 / math.sqrt(HD))
        reps += 1
        if time.perf_counter() - t0 > 8.0 or reps >= 5:
            break
    dt = (time.perf_counter() - t0) / reps
    return dt, f"1 (batch, KV-head) pair of 1 layer, {T} cached tokens, oracle decode x{reps}"


def _import_reference():
    """The reference package from the git-ignored copy under baseline/_ref, or None."""
    if not os.path.isdir(os.path.join(REF_DIR, "blockgtq")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import blockgtq  # noqa: F401
        return blockgtq
    except Exception:
        return None


class RefCpuSlice:
    """The reference's unaccelerated path (blockgtq/unaccelerated.py:121-131) on one slice of the workload:
    one layer, batch 1, every KV head: BlockGTQPipeline.compress_decompress of the cached keys,
    TurboQuantMSE.compress_decompress of the cached values, then scaled_dot_product_attention of the step's
    queries over the de-quantised cache, with torch using all host cores."""

    def __init__(self, w, cores):
        import contextlib
        with contextlib.redirect_stdout(sys.stderr):      # (the reference prints its bit map: stdout is for the JSON line)
            self._init(w, cores)

    def _init(self, w, cores):
        from blockgtq.block_gtq_pipeline import BlockGTQPipeline
        from blockgtq.tq import TurboQuantMSE
        torch.set_num_threads(cores)
        gen = torch.Generator().manual_seed(0)
        T, n_kv, gqa = w["ctx"], w["n_kv"], w["n_q"] // w["n_kv"]
        ck = synth_keys(gen, (1, 2048), w["theta"], "cpu")[0]
        cq = synth_keys(gen, (gqa, 2048), w["theta"], "cpu").reshape(-1, HD)
        # one calibrated pipeline serves every head of the slice: the arithmetic does not depend on the bit map
        self.kq = BlockGTQPipeline(head_dim=HD, avg_bits=float(w["k_bits"]), device=torch.device("cpu"))
        self.kq.calibrate(cq.float().contiguous(), ck.float().contiguous())
        self.vq = TurboQuantMSE(d=HD, bit_width=w["v_bits"], seed=1000, device=torch.device("cpu"))
        self.k = torch.stack([synth_keys(gen, (1, T), w["theta"], "cpu")[0] for _ in range(n_kv)]).float()
        self.v = torch.randn(n_kv, T, HD, generator=gen)
        self.q = torch.randn(1, n_kv * gqa, 1, HD, generator=gen)
        self.n_kv, self.gqa = n_kv, gqa

    def step(self):
        import torch.nn.functional as F
        kh = torch.stack([self.kq.compress_decompress(self.k[h]) for h in range(self.n_kv)])
        vh = torch.stack([self.vq.compress_decompress(self.v[h]) for h in range(self.n_kv)])
        kk = kh.repeat_interleave(self.gqa, dim=0).unsqueeze(0)
        vv = vh.repeat_interleave(self.gqa, dim=0).unsqueeze(0)
        return F.scaled_dot_product_attention(self.q, kk, vv)


def run_reference(args, w, name, rank, world):
    """CPU arm: the reference's own unaccelerated path on a bounded slice per step (one layer, batch 1), all
    host cores; the step time of the full workload is the slice time x layers x batch, and says so."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    L, B = w["layers"], w["batch"]
    if w.get("mode") in ("encode", "prefill"):
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm covers the decode workloads only"}))
        return
    times, kind, sample = [], "port", ""
    if _import_reference() is not None:
        try:
            sl = RefCpuSlice(w, cores)
            for i in range(args.warmup + args.steps):
                t0 = time.perf_counter()
                sl.step()
                if i >= args.warmup:
                    times.append(time.perf_counter() - t0)
            kind = "reference"
            sample = (f"per step: 1 layer x batch 1 x {w['n_kv']} KV heads x {w['ctx']} cached tokens through the "
                      "reference's BlockGTQPipeline.compress_decompress (K) + TurboQuantMSE.compress_decompress (V) + "
                      f"scaled_dot_product_attention, torch.set_num_threads({cores}); step time of the workload = "
                      f"slice x {L * B} (layers x batch)")
            scale = L * B
        except Exception as e:                                     # noqa: BLE001
            sample = f"reference CPU path failed ({type(e).__name__}: {e}); "
            times = []
    if not times:
        for i in range(max(1, min(args.steps, 3))):
            dt, desc = cpu_decode_sample(w, seed=i)
            times.append(dt)
        scale = L * B * w["n_kv"]
        sample += desc + f" (NumPy restatement, one thread); step time = sample x {scale}"
    dt = statistics.median(times)
    step_s = dt * scale
    val = B / step_s
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup if kind == "reference" else 0, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, w, 1) | {
            "sample_ms": dt * 1e3, "scaled_by": scale,
            "note": "ms_per_step is the measured slice time x scaled_by; every step of this arm runs one slice"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores if kind == "reference" else 1, "kind": kind,
                         "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(w):
    """The reported CPU baseline of the default run: a few slices of the reference's unaccelerated path (kind
    "reference") when baseline/_ref is present, else the NumPy restatement (kind "port")."""
    cores = os.cpu_count() or 1
    L, B = w["layers"], w["batch"]
    if _import_reference() is not None:
        try:
            sl = RefCpuSlice(w, cores)
            sl.step()
            times = []
            t_end = time.perf_counter() + 12.0
            while len(times) < 8 and (time.perf_counter() < t_end or not times):
                t0 = time.perf_counter()
                sl.step()
                times.append(time.perf_counter() - t0)
            dt = statistics.median(times)
            return {"value": B / (dt * L * B), "unit": "tok/s", "cores": cores, "kind": "reference",
                    "sample": f"{len(times)} x (1 layer x batch 1 x {w['n_kv']} KV heads x {w['ctx']} cached tokens) through "
                              "the reference's BlockGTQPipeline.compress_decompress + TurboQuantMSE.compress_decompress "
                              f"+ scaled_dot_product_attention on {cores} threads, median {dt * 1e3:.0f} ms; step time "
                              f"= slice x {L * B} (layers x batch)"}
        except Exception:                                          # noqa: BLE001
            pass
    dt, sample = cpu_decode_sample(w)
    pairs = L * B * w["n_kv"]
    return {"value": B / (dt * pairs), "unit": "tok/s", "cores": 1, "kind": "port",
            "sample": sample + f" (NumPy restatement, one thread); step time = sample x {pairs}"}


def parity_check(mgr, w, qkv_step, t_before, outs):
    """Outputs of one decode step of the timed path against the CPU oracle for three sampled (layer, batch,
    KV head) pairs: attention output of the pair's query heads over the packed rows (and, with fp16
    regions, the sink + recent tokens), and the packed row the step appended, against the oracle's encoder
    (skipped for a row with a coordinate on a bin edge).  `qkv_step`: the step's (L, B, n_q + 2 n_kv, 1, hd)
    inputs; `t_before`: tokens cached before the step."""
    from helpers import oracle_meta
    from oracle import bgtq_oracle as O
    if outs is None:
        return None
    L, B, n_q, n_kv = w["layers"], w["batch"], w["n_q"], w["n_kv"]
    gqa = n_q // n_kv
    ns, win = mgr.n_sink, mgr.recent_window
    picks = sorted({(0, 0, 0), (L - 1, B - 1, n_kv - 1), (L // 2, B // 2, n_kv // 2)})
    max_abs, max_excess, max_ref, rows_checked, rows_equal = 0.0, 0.0, 0.0, 0, 0
    for li, b, h in picks:
        qz = mgr.quantizers[li][h]
        meta = oracle_meta(qz._tables, qz._v_tables)
        sl = slice(h * gqa, (h + 1) * gqa)
        q = qkv_step[li, b, sl, 0].cpu().numpy()
        qr = O.rotate_q(q, meta)
        n_packed = t_before + 1 if not mgr._buffered else max(0, t_before - ns - win)
        tb = qz._total_packed_bytes
        if n_packed:
            po, pl = O.attend_packed(qr, mgr._k_packed[li, b, h, :n_packed, :tb].cpu().numpy(),
                                     mgr._k_norms[li, b, h, :n_packed].cpu().numpy(),
                                     mgr._v_packed[li, b, h, :n_packed].cpu().numpy(),
                                     mgr._v_norms[li, b, h, :n_packed].cpu().numpy(), meta, mgr.scale)
        else:
            po, pl = np.zeros((gqa, HD)), np.full(gqa, -np.inf)
        ref = po
        if mgr._buffered:
            ring = win + 1
            idx = list(range(min(ns, t_before + 1)))
            idx += [ns + i % ring for i in range(n_packed, t_before + 1 - ns)]
            kb = mgr._k_buf[li, b, h, idx].cpu().numpy()
            vb = mgr._v_buf[li, b, h, idx].cpu().numpy()
            bo, bl = O.attend_fp16(q, kb, vb, mgr.scale)
            m = np.maximum(pl, bl)
            wp, wb = np.exp(pl - m), np.exp(bl - m)
            ref = (wp[:, None] * po + wb[:, None] * bo) / (wp + wb)[:, None]
        got = outs[li][b, sl].float().cpu().numpy()
        err = np.abs(got - ref)
        max_abs = max(max_abs, float(err.max()))
        max_ref = max(max_ref, float(np.abs(ref).max()))
        # the step's outputs are fp16: half an fp16 ulp of the value itself is not the kernel's error
        max_excess = max(max_excess, float((err - np.abs(ref) * 2.0 ** -11).max()))
        # the row appended by this step (unbuffered caches append at t_before; buffered ones flush token f)
        row = t_before if not mgr._buffered else (n_packed if t_before - ns - win >= 0 else None)
        if row is not None:
            if mgr._buffered:
                k_src = mgr._k_buf[li, b, h, ns + row % (win + 1)].cpu().numpy()[None]
            else:
                k_src = qkv_step[li, b, n_q + h, 0].cpu().numpy()[None]
            enc = O.encode_k_packed(k_src, meta)
            if not enc["fragile"].any():
                rows_checked += 1
                rows_equal += int(np.array_equal(mgr._k_packed[li, b, h, row, :tb].cpu().numpy(), enc["packed"][0]))
    return {"pairs": len(picks), "max_abs": max_abs, "max_abs_beyond_fp16_output_rounding": max(0.0, max_excess),
            "largest_output": max_ref, "tolerance": 2e-3, "appended_rows_checked": rows_checked,
            "appended_rows_bit_equal": rows_equal,
            "ok": bool(max_excess <= 2e-3 and rows_equal == rows_checked)}


def workload_config(name, w, world):
    """The workload keys both arms print, so that their `config` dicts compare equal on the shape."""
    return {"workload": name, "layers": w["layers"], "batch_per_gpu": w["batch"], "n_q": w["n_q"], "n_kv": w["n_kv"],
            "context": w["ctx"], "k_avg_bits": w["k_bits"], "v_bits": w["v_bits"], "fp16_sink": w["n_sink"],
            "fp16_window": w["window"], "parallelism": f"batch x{world}"}


def run_triton(args, w, name):
    """The reference's own Triton decode path on this GPU, through its stock classes: BlockGTQKVManager
    calibrate -> _encode_kv -> append_and_attend (blockgtq/packed_kv_manager.py:85-348), on the same synthetic
    keys/values and shapes, a few layers of the workload (calibration costs seconds per head there), timed the
    way the reference times decode steps (bench/bench_decode_e2e.py:130-156: synchronise, perf_counter, 5
    warm-up + 20 timed steps, median).  Nothing of this repository's package is imported."""
    if _import_reference() is None:
        print(json.dumps({"impl": "triton", "unavailable": "baseline/_ref/blockgtq is not present"}))
        return
    if w.get("mode") in ("encode", "prefill", "seq") or w["n_sink"] or w["window"]:
        note = "the reference's packed path has no fp16 sink/window; timed without them" if w["n_sink"] else ""
    else:
        note = ""
    real_stdout = sys.stdout
    sys.stdout = sys.stderr          # the reference prints while it calibrates: stdout is for the JSON line
    try:
        from blockgtq.packed_kv_manager import BlockGTQKVManager as RefManager
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        L = max(1, min(w["layers"], args.triton_layers))
        n_q, n_kv, B, T = w["n_q"], w["n_kv"], w["batch"], w["ctx"]
        gqa = n_q // n_kv
        n_steps = args.warmup + args.steps
        gen = torch.Generator(device=dev).manual_seed(1234)
        mgr = RefManager(L, n_q, n_kv, HD, max_seq_len=T + n_steps + 8, batch_size=B, k_avg_bits=w["k_bits"],
                         v_bits=w["v_bits"], device=dev)
        for li in range(L):
            ck = torch.stack([synth_keys(gen, (1, 2048), w["theta"], dev)[0] for _ in range(n_kv)])
            cq = torch.stack([synth_keys(gen, (gqa, 2048), w["theta"], dev).reshape(-1, HD) for _ in range(n_kv)])
            mgr.calibrate(li, cq.float(), ck.float())
        for li in range(L):
            for t in range(0, T, 4096):
                n = min(4096, T - t)
                k = torch.stack([synth_keys(gen, (B, n), w["theta"], dev) for _ in range(n_kv)], dim=1)
                v = torch.randn(B, n_kv, n, HD, generator=gen, device=dev).half()
                mgr._encode_kv(li, k, v, t, t + n)
        mgr.seq_len = T
        qs = (torch.randn(n_steps, L, B, n_q, 1, HD, generator=gen, device=dev) * 2).half()
        ks = torch.stack([torch.stack([synth_keys(gen, (B * n_kv, 1), w["theta"], dev).reshape(B, n_kv, 1, HD)
                                       for _ in range(L)]) for _ in range(n_steps)])
        vs = torch.randn(n_steps, L, B, n_kv, 1, HD, generator=gen, device=dev).half()
        times = []
        for s in range(n_steps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for li in range(L):
                mgr.append_and_attend(li, qs[s, li], ks[s, li], vs[s, li])
            mgr.increment_seq_len()
            torch.cuda.synchronize()
            if s >= args.warmup:
                times.append((time.perf_counter() - t0) * 1e3)
        # the decode kernels alone (attention over the cache, per layer): CUDA events around one more step's
        # attention calls would need the reference's internals, so report the whole layer step
        med = statistics.median(times)
        line = {"impl": "triton", "metric": "decode_tokens_per_s", "unit": "tok/s", "n_gpus": 1,
                "value": B / (med / L * w["layers"] * 1e-3), "steps": len(times), "warmup": args.warmup,
                "ms_per_step": med / L * w["layers"], "higher_is_better": True, "scaling": "weak", "dtype": "f16",
                "data": "synthetic", "config": workload_config(name, w, 1) | {
                    "layers_timed": L, "ms_per_step_timed_layers": med, "us_per_layer_step": med / L * 1e3,
                    "protocol": "reference BlockGTQKVManager.append_and_attend per layer, synchronise + perf_counter "
                                "around each decode step, median; step of the full workload = timed layers scaled "
                                f"by {w['layers']}/{L}", "note": note,
                    "triton": __import__("triton").__version__}}
    except Exception as e:                                         # noqa: BLE001
        msg = f"{type(e).__name__}: {e}".splitlines()[0][:300]
        line = {"impl": "triton", "unavailable": msg}
    finally:
        sys.stdout = real_stdout
    print(json.dumps(line), flush=True)


def triton_leg(args, name):
    """Run the Triton arm in a child process (its own CUDA context, none of this package loaded) and return
    the summary the default line carries."""
    if not os.path.isdir(os.path.join(REF_DIR, "blockgtq")):
        return {"unavailable": "baseline/_ref/blockgtq is not present"}
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "triton", "--workload", name, "--steps", "20",
           "--warmup", "5", "--triton-layers", str(args.triton_layers)]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=args.triton_timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference's Triton path did not finish within {args.triton_timeout} s"}
    for ln in reversed(out.stdout.splitlines()):
        if ln.startswith("{"):
            d = json.loads(ln)
            if "unavailable" in d:
                return {"unavailable": d["unavailable"]}
            c = d["config"]
            return {"ms_per_step": d["ms_per_step"], "tok_s": d["value"], "us_per_layer_step": c["us_per_layer_step"],
                    "layers_timed": c["layers_timed"], "steps": d["steps"], "protocol": c["protocol"],
                    "note": c["note"], "triton": c["triton"]}
    return {"unavailable": ("no result line; stderr tail: " + out.stderr.strip().splitlines()[-1][:200])
            if out.stderr.strip() else "no result line"}


def run_seq_sharded(args, w, rank, world, dev, emit=True, shard=True):
    """One long sequence cut into per-rank chunks: per layer the local split-KV decode + combine, one
    exchange of the (O, LSE) messages and the merge of the ranks' messages; the rank that owns the tail also
    appends the step's token; all layers of a step are one CUDA graph.  Strong scaling: the total context is
    fixed."""
    import torch.distributed as dist
    from blockgtq_b200 import _lib
    from blockgtq_b200.layer import combine
    from blockgtq_b200.sharding import chunk_bounds
    K, W = args.steps, args.warmup
    n_total = 2 * (K + W) + 4
    L, B, n_q, n_kv, T = w["layers"], w["batch"], w["n_q"], w["n_kv"], w["ctx"]
    sharded = shard and world > 1           # shard=False: every rank that calls this holds the whole sequence
    lo, hi = chunk_bounds(T, world, rank) if sharded else (0, T)
    owner = world - 1                       # appended tokens extend the last chunk
    mgr, gen = build_manager(w, dev, seed=1234, extra_tokens=n_total + 16, ctx=hi - lo)
    transport = args.seq_transport if sharded else "none"
    if sharded:
        from blockgtq_b200.sharding import SequenceShard
        SequenceShard(mgr, owner=owner, transport=transport)
    qs = (torch.randn(n_total, L, B, n_q, 1, HD, generator=gen, device=dev) * 2).half()
    ks = torch.stack([torch.stack([synth_keys(gen, (B * n_kv, 1), w["theta"], dev).reshape(B, n_kv, 1, HD)
                                   for _ in range(L)]) for _ in range(n_total)])
    vs = torch.randn(n_total, L, B, n_kv, 1, HD, generator=gen, device=dev).half()
    dq = torch.cat([qs, ks, vs], dim=3)                             # (steps, L, B, n_q + 2 n_kv, 1, hd) in HBM
    hq = dq.cpu().pin_memory()
    hout = torch.empty(L, B, n_q, HD, dtype=torch.float16).pin_memory()
    g_all = mgr.static_qkv_all()
    step_no = [0]
    # the whole decode step (all layers, the exchange included) as one CUDA graph on every rank
    for li in range(L):
        mgr.layer_step(li)
    mgr.increment_seq_len()
    torch.cuda.synchronize()
    step_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(step_graph):
        for li in range(L):
            mgr.layer_step(li)
    per_step = ((4 if transport == "p2p" else 5) if sharded else 3) * L

    def step_device():
        g_all.copy_(dq[step_no[0]])
        step_graph.replay()
        _lib.count_launch(per_step)
        mgr.increment_seq_len()
        step_no[0] += 1

    def step_e2e():
        g_all.copy_(hq[step_no[0]], non_blocking=True)
        step_graph.replay()
        _lib.count_launch(per_step)
        hout.copy_(mgr.static_outputs(), non_blocking=True)
        mgr.increment_seq_len()
        torch.cuda.synchronize()
        step_no[0] += 1

    def barrier():
        if sharded:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if sharded:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(W):
        step_device()
    sampler = clocks_sampler(dev.index) if rank == 0 else None
    l0 = _lib.launches
    ms_total = timed(step_device, K)
    launches = _lib.launches - l0
    clocks = clocks_summary(sampler)
    for _ in range(W):
        step_e2e()
    ms_e2e = timed(step_e2e, K)
    live = torch.tensor([float(mgr.live_bytes_per_step())], device=dev)
    if sharded:
        dist.all_reduce(live)
    torch.cuda.synchronize()
    mgr.check_status()
    result = {"ms_per_step": ms_total / K, "ms_per_step_e2e": ms_e2e / K, "transport": transport, "layers": L,
              "tokens_per_gpu": hi - lo}
    mgr.release_graphs()
    del step_graph
    if not emit:
        return result
    if rank == 0:
        ms_step = ms_total / K
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        gbs = float(live.item()) / world / (ms_step * 1e-3) / 1e9        # per GPU, whole step
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": B / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "layers": L, "batch": B, "n_q": n_q, "n_kv": n_kv, "context": T,
                       "tokens_per_gpu": hi - lo, "k_avg_bits": w["k_bits"], "v_bits": w["v_bits"],
                       "parallelism": f"sequence chunks x{world}, one exchange of (O, LSE) per layer ({transport})",
                       "exchange_bytes_per_layer": B * n_q * (HD + 1) * 4,
                       "l2": "inputs larger than L2 (packed cache bytes per step >> 126 MB), no flush"},
            "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": gbs, "peak": peak,
                         "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                         "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"},
            "e2e": {"value": B / (ms_e2e / K * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": int(L * hq[0, 0].numel() * 2),
                    "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": ms_e2e / K},
            "gpu_launches": launches, "clocks": clocks}), flush=True)
    return result


def seqshard_leg(args, rank, world, dev):
    """Next to the batch-sharded default workload at N > 1: the sequence-sharded one (one 131072-token
    sequence, Llama-3.1-8B shape, K2V2, 8 of its 32 layers so the leg stays short), timed on all N ranks with
    the (O, LSE) exchange and then on rank 0 alone holding the whole sequence."""
    import torch.distributed as dist
    w = dict(WORKLOADS["llama3.1-8b_k2v2_b1_t131072_seqshard"], layers=8)
    sub = argparse.Namespace(**vars(args))
    sub.steps, sub.warmup, sub.workload = 10, 3, "llama3.1-8b_k2v2_b1_t131072_seqshard"
    many = run_seq_sharded(sub, w, rank, world, dev, emit=False)
    torch.cuda.empty_cache()
    dist.barrier()
    one = run_seq_sharded(sub, w, rank, world, dev, emit=False, shard=False) if rank == 0 else None
    dist.barrier()
    if rank != 0:
        return None
    L = w["layers"]
    return {"workload": "llama3.1-8b_k2v2_b1_t131072_seqshard, 8 of 32 layers", "n_gpus": world,
            "ms_per_step": many["ms_per_step"], "tok_s": 1.0 / (many["ms_per_step"] * 1e-3),
            "ms_per_step_1gpu": one["ms_per_step"], "speedup_vs_1gpu": one["ms_per_step"] / many["ms_per_step"],
            "us_per_layer": many["ms_per_step"] / L * 1e3, "us_per_layer_1gpu": one["ms_per_step"] / L * 1e3,
            "transport": many["transport"], "tokens_per_gpu": many["tokens_per_gpu"],
            "exchange_bytes_per_layer": w["n_q"] * (HD + 1) * 4,
            "note": "1-GPU figure: the same code on rank 0 holding all 131072 tokens, same run"}


def run_encode(args, w, rank, world, dev):
    """Bulk encode of a whole context per layer (prefill), then the latency of single-token appends."""
    import torch.distributed as dist
    from blockgtq_b200 import BlockGTQKVManager, _lib
    K, W = args.steps, args.warmup
    L, B, n_q, n_kv, T = w["layers"], w["batch"], w["n_q"], w["n_kv"], w["ctx"]
    gqa = n_q // n_kv
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    mgr = BlockGTQKVManager(L, n_q, n_kv, HD, max_seq_len=T + 1024, batch_size=B, k_avg_bits=w["k_bits"],
                            v_bits=w["v_bits"], device=dev, use_cuda_graph=False)
    for li in range(L):
        ck = torch.stack([synth_keys(gen, (1, 2048), w["theta"], dev)[0] for _ in range(n_kv)])
        cq = torch.stack([synth_keys(gen, (gqa, 2048), w["theta"], dev).reshape(-1, HD) for _ in range(n_kv)])
        mgr.calibrate(li, cq.float(), ck.float())
    ks = [torch.stack([synth_keys(gen, (B, T), w["theta"], dev) for _ in range(n_kv)], dim=1) for _ in range(L)]
    vs = [torch.randn(B, n_kv, T, HD, generator=gen, device=dev).half() for _ in range(L)]
    hk = [k.cpu().pin_memory() for k in ks]
    hv = [v.cpu().pin_memory() for v in vs]
    stage_k, stage_v = torch.empty_like(ks[0]), torch.empty_like(vs[0])

    def step_device():
        for li in range(L):
            mgr._append_tokens(li, ks[li], vs[li], 0)

    def step_e2e():
        for li in range(L):
            stage_k.copy_(hk[li], non_blocking=True)
            stage_v.copy_(hv[li], non_blocking=True)
            mgr._append_tokens(li, stage_k, stage_v, 0)
        torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(W):
        step_device()
    sampler = clocks_sampler(dev.index) if rank == 0 else None
    l0 = _lib.launches
    ms_total = timed(step_device, K)
    launches = _lib.launches - l0
    clocks = clocks_summary(sampler)
    step_e2e()
    ms_e2e = timed(step_e2e, max(1, K // 4))
    # single-token appends (B rows per KV head): latency of one layer's append
    mgr.seq_len = T
    k1, v1 = ks[0][:, :, :1].contiguous(), vs[0][:, :, :1].contiguous()
    for i in range(8):
        mgr._append_tokens(0, k1, v1, T + i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(512):
        mgr._append_tokens(i % L, k1, v1, T + 8 + i)
    e1.record()
    torch.cuda.synchronize()
    append_us = e0.elapsed_time(e1) / 512 * 1e3
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        pms = [mgr.quantizers[0][h].pack_meta for h in range(n_kv)]
        row_bytes = sum(pm["total_packed_bytes"] + 2 * sum(1 for key in pm if isinstance(key, int)) for pm in pms) \
            + n_kv * (mgr._layers[0].vpb + 2)
        alg = B * T * (n_kv * 512 + row_bytes)               # per launch (one layer)
        ms_launch = ms_total / (K * L)
        print(json.dumps({
            "metric": "prefill_encode_tokens_per_s", "value": world * B * T * L / (ms_total / K * 1e-3),
            "unit": "token-layers/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "layers_per_step": L, "batch_per_gpu": B, "n_kv": n_kv, "tokens": T,
                       "k_avg_bits": w["k_bits"], "v_bits": w["v_bits"], "parallelism": f"batch x{world}",
                       "l2": "each layer's fp16 K/V input is 537 MB, larger than L2; no flush",
                       "append_us_per_layer": append_us},
            "roofline": {"bound": "hbm", "kernel": "encode_t5w_kernel", "achieved": alg / (ms_launch * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": alg / (ms_launch * 1e-3) / 1e9 / peak, "traffic": None,
                         "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback",
                         "algorithmic_bytes_per_launch": alg, "launch_ms": ms_launch},
            "e2e": {"value": world * B * T * L / (ms_e2e / max(1, K // 4) * 1e-3), "unit": "token-layers/s",
                    "h2d_bytes_per_step": int(L * 2 * ks[0].numel() * 2), "d2h_bytes_per_step": 0,
                    "ms_per_step": ms_e2e / max(1, K // 4)},
            "gpu_launches": launches, "clocks": clocks}), flush=True)


def run_prefill(args, w, rank, world, dev):
    """Layer-major prefill of one layer: bulk encode of the prompt's K/V, then causal attention of every
    prompt position over the packed cache (queries rotated with one GEMM, V un-rotated with one GEMM)."""
    import torch.distributed as dist
    from blockgtq_b200 import BlockGTQKVManager, _lib
    from blockgtq_b200.layer import prefill_attention, rotate_q_bulk
    K, W = args.steps, args.warmup
    B, n_q, n_kv, T = w["batch"], w["n_q"], w["n_kv"], w["ctx"]
    gqa = n_q // n_kv
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=T, batch_size=B, k_avg_bits=w["k_bits"], v_bits=w["v_bits"],
                            device=dev, use_cuda_graph=False)
    ck = torch.stack([synth_keys(gen, (1, 2048), w["theta"], dev)[0] for _ in range(n_kv)])
    cq = torch.stack([synth_keys(gen, (gqa, 2048), w["theta"], dev).reshape(-1, HD) for _ in range(n_kv)])
    mgr.calibrate(0, cq.float(), ck.float())
    k = torch.stack([synth_keys(gen, (B, T), w["theta"], dev) for _ in range(n_kv)], dim=1)
    q = torch.stack([synth_keys(gen, (B, T), w["theta"], dev) for _ in range(n_q)], dim=1)
    v = torch.randn(B, n_kv, T, HD, generator=gen, device=dev).half()
    hq, hk, hv = q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory()
    sq, sk, sv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    hout = torch.empty(B, n_q, T, HD, dtype=torch.float16).pin_memory()
    lt = None
    t_attn = []

    def layer(q_, k_, v_):
        mgr._append_tokens(0, k_, v_, 0)
        q_rot = rotate_q_bulk(mgr._layers[0], q_)
        return prefill_attention(mgr._layers[0], q_rot, mgr._k_packed[0], mgr._k_norms[0], mgr._v_packed[0],
                                 mgr._v_norms[0], T, causal=True, scale=mgr.scale, v_rot=mgr._layers[0].v_rot)

    def step_device():
        layer(q, k, v)

    def step_e2e():
        sq.copy_(hq, non_blocking=True)
        sk.copy_(hk, non_blocking=True)
        sv.copy_(hv, non_blocking=True)
        hout.copy_(layer(sq, sk, sv), non_blocking=True)
        torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(W):
        step_device()
    sampler = clocks_sampler(dev.index) if rank == 0 else None
    l0 = _lib.launches
    ms_total = timed(step_device, K)
    launches = _lib.launches - l0
    clocks = clocks_summary(sampler)
    # the attention kernel alone
    q_rot = rotate_q_bulk(mgr._layers[0], q)
    args_ = (mgr._layers[0], q_rot, mgr._k_packed[0], mgr._k_norms[0], mgr._v_packed[0], mgr._v_norms[0], T)
    prefill_attention(*args_)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        prefill_attention(*args_)
    e1.record()
    torch.cuda.synchronize()
    ms_kernel = e0.elapsed_time(e1) / 3
    step_e2e()
    ms_e2e = timed(step_e2e, max(1, K // 2))
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("bf16_tflops", 1590.0))
        flops = 4.0 * (T * (T + 1) / 2) * HD * n_q * B              # QK^T and PV over the causal triangle
        tf = flops / (ms_kernel * 1e-3) / 1e12
        print(json.dumps({
            "metric": "prefill_tokens_per_s", "value": world * B * T / (ms_total / K * 1e-3), "unit": "token-layers/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "layers_per_step": 1, "batch_per_gpu": B, "n_q": n_q, "n_kv": n_kv,
                       "tokens": T, "k_avg_bits": w["k_bits"], "v_bits": w["v_bits"], "parallelism": f"batch x{world}",
                       "l2": "q/k/v inputs of a layer are 0.8 GB, larger than L2; no flush",
                       "attention_kernel_ms": ms_kernel},
            "roofline": {"bound": "tensor", "kernel": "prefill_t5_kernel (tcgen05, tensor memory)", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                         "frac": tf / peak, "traffic": None,
                         "peak_source": "MEASURED_PEAKS.json (bf16 burst)" if peaks else "fallback",
                         "algorithmic_flops_per_launch": flops, "launch_ms": ms_kernel},
            "e2e": {"value": world * B * T / (ms_e2e / max(1, K // 2) * 1e-3), "unit": "token-layers/s",
                    "h2d_bytes_per_step": int((hq.numel() + hk.numel() + hv.numel()) * 2),
                    "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": ms_e2e / max(1, K // 2)},
            "gpu_launches": launches, "clocks": clocks}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference-Triton leg of the default run")
    ap.add_argument("--triton-layers", type=int, default=2, help="layers the reference-Triton leg builds and times")
    ap.add_argument("--triton-timeout", type=int, default=300)
    ap.add_argument("--no-parity-check", action="store_true")
    ap.add_argument("--seq-transport", default="p2p", choices=["p2p", "nccl"],
                    help="exchange of the sequence-sharded workload: peer-memory stores or one NCCL all-gather")
    ap.add_argument("--no-seqshard", action="store_true", help="at N > 1, skip the sequence-sharded leg")
    ap.add_argument("--per-layer-graphs", action="store_true",
                    help="replay one CUDA graph per layer (append_and_attend) instead of one graph per decode step")
    ap.add_argument("--eager-step", action="store_true",
                    help="launch the step's kernels one by one instead of replaying a graph (for profiler launch lists)")
    ap.add_argument("--traffic-key", action="store_true",
                    help="print the hash of the decode kernel sources that a record in profiles/dram_traffic.json carries")
    args = ap.parse_args()
    if args.traffic_key:
        print(json.dumps({"sources": TRAFFIC_SOURCES, "sources_sha16": sources_key(TRAFFIC_SOURCES)}))
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, args.workload, rank, world)
        return
    if args.impl == "triton":
        if rank == 0:
            run_triton(args, w, args.workload)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the package has no CPU path); use --impl reference for the CPU arm")
    import torch.distributed as dist
    from blockgtq_b200 import _lib
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))

    if w.get("mode") == "prefill":
        run_prefill(args, w, rank, world, dev)
        if world > 1:
            dist.destroy_process_group()
        return
    if w.get("mode") == "encode":
        run_encode(args, w, rank, world, dev)
        if world > 1:
            dist.destroy_process_group()
        return
    if w.get("mode") == "seq":
        run_seq_sharded(args, w, rank, world, dev)
        if world > 1:
            dist.destroy_process_group()
        return

    K, W = args.steps, args.warmup
    n_steps_total = 2 * (K + W) + min(K, 5) + 2
    # The cache is filled so that the LAST step of the run attends over the nominal context: every step sees a
    # cache of at most w["ctx"] tokens (ctx - n_steps_total + 1 ... ctx).
    ctx_start = max(64, w["ctx"] - n_steps_total)
    mgr, gen = build_manager(w, dev, seed=1234 + rank, extra_tokens=n_steps_total + 16, ctx=ctx_start)
    L, B, n_q, n_kv = w["layers"], w["batch"], w["n_q"], w["n_kv"]
    # one decode token per layer per step, pre-generated; device copies for `value`, pinned host for `e2e`
    qs = (torch.randn(n_steps_total, L, B, n_q, 1, HD, generator=gen, device=dev) * 2).half()
    ks = torch.stack([torch.stack([synth_keys(gen, (B * n_kv, 1), w["theta"], dev).reshape(B, n_kv, 1, HD)
                                   for _ in range(L)]) for _ in range(n_steps_total)])
    vs = torch.randn(n_steps_total, L, B, n_kv, 1, HD, generator=gen, device=dev).half()
    hqkv = torch.cat([qs, ks, vs], dim=3).cpu().pin_memory()       # (steps, L, B, n_q + 2 n_kv, 1, hd)
    hout = torch.empty(L, B, n_q, 1, HD, dtype=torch.float16).pin_memory()
    g_all = mgr.static_qkv_all()                                    # (L, B, n_q + 2 n_kv, 1, hd): per-layer step inputs
    g_in = [mgr.static_inputs(li) for li in range(L)]
    graph_outputs = mgr._use_graph                                 # results land in the manager's static output buffer
    step_no = [0]

    dqkv = torch.cat([qs, ks, vs], dim=3)                          # the same inputs, resident in HBM
    # One CUDA graph for the whole decode step (every layer's append + decode + combine), the way a serving
    # engine captures its model forward around these launches; --per-layer-graphs replays one graph per layer
    # through append_and_attend instead.
    step_graph = None
    if graph_outputs and not args.per_layer_graphs and not args.eager_step:
        for li in range(L):
            mgr.layer_step(li)                                      # eager once: kernel attributes, shapes
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            for li in range(L):
                mgr.layer_step(li)
    launches_per_step = 3 * L

    def run_layers():
        if step_graph is not None:
            step_graph.replay()
            _lib.count_launch(launches_per_step)
            return None
        if args.eager_step and graph_outputs:
            for li in range(L):
                mgr.layer_step(li)
            return None
        return [mgr.append_and_attend(li, *g_in[li]) for li in range(L)]

    def step_device():
        s = step_no[0]
        g_all.copy_(dqkv[s])                                        # the step's inputs into the layers' input buffers
        run_layers()
        mgr.increment_seq_len()
        step_no[0] += 1

    def step_e2e():
        s = step_no[0]
        g_all.copy_(hqkv[s], non_blocking=True)                     # H2D: every layer's q/k/v of this step
        outs = run_layers()
        if graph_outputs:                                           # D2H: every layer's attention output
            hout.copy_(mgr.static_outputs().unsqueeze(3), non_blocking=True)
        else:
            for li in range(L):
                hout[li].copy_(outs[li], non_blocking=True)
        mgr.increment_seq_len()
        torch.cuda.synchronize()
        step_no[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # clocks are sampled from the warm-up to the end of the end-to-end timing: warm-up, timed steps, kernel
    # timing and end-to-end steps all keep the GPU under the step's load, and 20 steps alone last only tens of
    # milliseconds
    sampler = clocks_sampler(local) if rank == 0 else None
    t_sampler = time.perf_counter()
    for _ in range(W):
        step_device()
    launches0 = _lib.launches
    ms_total = timed(step_device, K)
    launches = _lib.launches - launches0
    live_bytes = mgr.live_bytes_per_step()

    # per-launch duration of the dominant kernel (fused decode): the decode of every layer, launched as in the
    # step (programmatic dependent launches, the manager's flags and slot count) back to back, captured in a
    # CUDA graph so that no host launch time enters, and bracketed by CUDA events on the launching stream; each
    # layer's cache is a different 60+ MB and a pass over all layers exceeds L2, so no launch finds its input
    # in cache
    from blockgtq_b200.layer import decode as decode_op
    sink, n_packed, n_rec = mgr._region_sizes(mgr.seq_len)
    q_rot = torch.randn(B, n_q, HD, generator=gen, device=dev).half()
    dflags = mgr._dec_flags | (_lib.DEC_PROGRAMMATIC if mgr.programmatic else 0)

    def decode_all_layers():
        for li in range(L):
            decode_op(mgr._layers[li], q_rot, mgr._k_packed[li], mgr._k_norms[li], mgr._v_packed[li],
                      mgr._v_norms[li], 0, n_packed, n_splits=mgr._n_splits, scale=mgr.scale,
                      part_o=mgr._part_o, part_lse=mgr._part_lse, flags=dflags)

    decode_all_layers()
    n_prof = max(3, min(20, 240 // L))
    torch.cuda.synchronize()
    dec_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(dec_graph):
        decode_all_layers()
    dec_graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_prof):
        dec_graph.replay()
    e1.record()
    torch.cuda.synchronize()
    dec_avg_ms = e0.elapsed_time(e1) / (n_prof * L)
    # a short run ends before the clock sampler has written a handful of lines: keep the decode launches going
    # (untimed; they append nothing) until it has had half a second of this load
    while time.perf_counter() - t_sampler < 0.5:
        dec_graph.replay()
        torch.cuda.synchronize()
    del dec_graph
    packed_bytes_per_launch = (live_bytes - (sink + n_rec) * HD * 4 * n_kv * B * L) / L

    for _ in range(W):
        step_e2e()
    ms_e2e = timed(step_e2e, K)
    clocks = clocks_summary(sampler)

    parity = None
    if rank == 0 and not args.no_parity_check:
        # one more step of the timed path, then sampled (layer, batch, KV head) pairs of its outputs and of the
        # rows it appended against the CPU oracle on the same packed cache
        t_before = mgr.seq_len
        s_idx = step_no[0]
        step_device()
        torch.cuda.synchronize()
        mgr.check_status()
        parity = parity_check(mgr, w, dqkv[s_idx], t_before,
                              [mgr.static_outputs()[li] for li in range(L)] if graph_outputs else None)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = packed_bytes_per_launch / (dec_avg_ms * 1e-3) / 1e9
        ms_step = ms_total / K
        line = {
            "metric": "decode_tokens_per_s", "value": world * B / (ms_step * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args.workload, w, world) | {
                       "l2": "inputs larger than L2 (packed cache bytes per step >> 126 MB), no flush",
                       "graphs": "one per decode step" if step_graph is not None else
                                 ("none (eager launches)" if args.eager_step or not graph_outputs else "one per layer"),
                       "cache_lengths": [ctx_start + 1, int(mgr.seq_len)],      # first step's .. after the last one
                       "decode_item_ranges": "cost-balanced table (bgtq_decode_partition)",
                       "decode_us_per_layer": dec_avg_ms * 1e3, "step_hbm_gbs": live_bytes / (ms_step * 1e-3) / 1e9,
                       "step_frac_of_8tbs": live_bytes / (ms_step * 1e-3) / 8e12,
                       "decode_kernel": "specialised per layer at run time (NVRTC)"
                                        if not os.environ.get("BGTQ_DEC_NO_JIT") else "general (ahead of time)"},
            "roofline": {"bound": "hbm", "kernel": "bgtq_decode_jit" if not os.environ.get("BGTQ_DEC_NO_JIT") else "decode_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": dram_traffic(args.workload),
                         "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback",
                         "algorithmic_bytes_per_launch": packed_bytes_per_launch, "launch_ms": dec_avg_ms},
            "e2e": {"value": world * B / (ms_e2e / K * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": int(L * hqkv[0, 0].numel() * 2),
                    "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": ms_e2e / K},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if parity is not None:
            line["parity_check"] = parity
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(w)
        if not args.no_triton and world == 1:
            line["config"]["reference_triton"] = triton_leg(args, args.workload)
    seq = None
    if world > 1 and not args.no_seqshard and args.workload == DEFAULT:
        del mgr, dqkv, hqkv, qs, ks, vs, step_graph
        torch.cuda.empty_cache()
        # A failure that every rank meets the same way (a missing feature, memory) must not cost the main line
        try:
            seq = seqshard_leg(args, rank, world, dev)
        except Exception as e:                                     # noqa: BLE001
            seq = {"unavailable": f"{type(e).__name__}: {e}".splitlines()[0][:300]}
    if rank == 0:
        if seq is not None:
            line["seqshard"] = seq
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
