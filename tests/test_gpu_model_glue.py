"""GPU: the model-level glue (calibration helpers, production cache, prefill + decode step, manager
decode_step) on a tiny random Llama-architecture model, against the model's own fp16 forward.  The
packed cache is lossy, so logits are compared by cosine similarity; thresholds leave a wide margin
around the values measured for these bit widths (0.9995 at K6V4, 0.997 at K3V3)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny_model():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                      num_hidden_layers=2, intermediate_size=256, vocab_size=128, max_position_embeddings=512,
                      rope_theta=10000.0)
    return LlamaForCausalLM(cfg).to(DEV).half().eval()


@pytest.mark.parametrize("k_bits,v_bits,min_cos", [(6.0, 4, 0.998), (3.0, 3, 0.99)])
def test_production_prefill_and_decode_steps_track_the_fp16_model(k_bits, v_bits, min_cos):
    from blockgtq_b200 import (BlockGTQProductionCache, build_quantizers, collect_qk_activations,
                               production_decode_step, production_prefill)
    model = _tiny_model()
    L, nkv, nq, hd = 2, 1, 2, 128
    ids = torch.randint(0, 128, (1, 96), device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    data = collect_qk_activations(model, ids, DEV, n_calib_tokens=64)
    assert data[0]["q"].shape == (nkv, (nq // nkv) * 64, hd) and data[0]["k"].shape == (nkv, 64, hd)
    quantizers, batched, kernel_args = build_quantizers(data, L, nkv, hd, k_avg_bits=k_bits, v_bits=v_bits, device=DEV)
    cache = BlockGTQProductionCache(quantizers, batched, kernel_args, L, nkv, nq, hd, 256, v_bits=v_bits, device=DEV)
    with torch.no_grad():
        full = model(ids).logits
    prompt_logits = production_prefill(model, ids[:, :64], cache)
    assert torch.equal(prompt_logits, full[:, :64]) or (prompt_logits - full[:, :64]).abs().max() < 2e-2
    assert cache.seq_len == 64
    for t in range(64, 72):
        logits = production_decode_step(model, ids[:, t:t + 1], torch.tensor([[t]], device=DEV), cache)
        assert logits.shape == (1, 1, 128) and torch.isfinite(logits).all()
        cos = torch.nn.functional.cosine_similarity(logits[:, 0].float(), full[:, t].float()).item()
        assert cos >= min_cos, (t, cos)
    assert cache.seq_len == 72
    assert 0 < cache.cache_memory_bytes() < cache.fp16_cache_bytes()


def test_manager_decode_step_tracks_the_fp16_model():
    from blockgtq_b200 import BlockGTQKVManager, collect_qk_activations
    from blockgtq_b200.packed_kv_manager import decode_step
    from transformers import DynamicCache
    model = _tiny_model()
    L, nkv, nq, hd = 2, 1, 2, 128
    ids = torch.randint(0, 128, (1, 80), device=DEV, generator=torch.Generator(device=DEV).manual_seed(2))
    data = collect_qk_activations(model, ids, DEV, n_calib_tokens=64)
    mgr = BlockGTQKVManager(L, nq, nkv, hd, max_seq_len=128, batch_size=1, k_avg_bits=6.0, v_bits=4, device=DEV)
    for li in range(L):
        mgr.calibrate(li, data[li]["q"], data[li]["k"])
    with torch.no_grad():
        full = model(ids).logits
        pkv = DynamicCache()
        model(ids[:, :64], past_key_values=pkv, use_cache=True)
    mgr.init_from_cache(pkv)
    assert mgr.seq_len == 64
    for t in range(64, 70):
        logits = decode_step(model, ids[:, t:t + 1], torch.tensor([[t]], device=DEV), mgr)
        cos = torch.nn.functional.cosine_similarity(logits[:, 0].float(), full[:, t].float()).item()
        assert cos >= 0.998, (t, cos)
    assert mgr.seq_len == 70


def test_layer_major_prefill_then_decode_tracks_the_fp16_model():
    """Layer-major prefill (encode + packed prefill attention per layer, no fp16 KV cache) followed by
    decode steps; the cache it leaves must equal what the chunked prefill writes for layer 0 (same K/V
    inputs there) and the decode logits must stay close to the fp16 model (looser than after an fp16
    prefill: here every prompt position of layer 1 already saw layer 0's quantised attention; measured
    0.9935 at K6V4)."""
    from blockgtq_b200 import (BlockGTQProductionCache, build_quantizers, collect_qk_activations,
                               layer_major_prefill, production_decode_step, production_prefill)
    model = _tiny_model()
    L, nkv, nq, hd = 2, 1, 2, 128
    ids = torch.randint(0, 128, (1, 96), device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    data = collect_qk_activations(model, ids, DEV, n_calib_tokens=64)
    quantizers, batched, kernel_args = build_quantizers(data, L, nkv, hd, k_avg_bits=6.0, v_bits=4, device=DEV)
    cache = BlockGTQProductionCache(quantizers, batched, kernel_args, L, nkv, nq, hd, 256, v_bits=4, device=DEV)
    other = BlockGTQProductionCache(quantizers, batched, kernel_args, L, nkv, nq, hd, 256, v_bits=4, device=DEV)
    hidden = layer_major_prefill(model, cache, ids[:, :70])
    production_prefill(model, ids[:, :70], other)
    assert cache.seq_len == 70 and hidden.shape == (1, 70, 256)
    assert torch.equal(cache.k_packed[0, :, :, :70], other.k_packed[0, :, :, :70])
    assert torch.equal(cache.v_packed[0, :, :, :70], other.v_packed[0, :, :, :70])
    with torch.no_grad():
        full = model(ids).logits
    for t in range(70, 76):
        logits = production_decode_step(model, ids[:, t:t + 1], torch.tensor([[t]], device=DEV), cache)
        cos = torch.nn.functional.cosine_similarity(logits[:, 0].float(), full[:, t].float()).item()
        assert cos >= 0.985, (t, cos)


def test_captured_step_replayed_past_the_capacity_stores_nothing():
    """A step captured in the caller's own graph reads its position on the device; replaying it once more than
    the cache has room for must not write anywhere: the append kernel reports status 2 and stores nothing (the
    first row of the next (batch, head) pair, which an unchecked append would hit, stays as it was)."""
    import torch
    from blockgtq_b200 import BlockGTQKVManager
    from helpers import HD, synth_head
    dev = "cuda:0"
    gen = torch.Generator().manual_seed(5)
    B, n_kv, gqa, cap = 2, 2, 2, 64            # 64 = the allocation's own granularity: no spare rows behind max_T
    n_q = n_kv * gqa
    mgr = BlockGTQKVManager(1, n_q, n_kv, HD, max_seq_len=cap, batch_size=B, device=dev)
    cal = [synth_head(gen, 256, gqa) for _ in range(n_kv)]
    mgr.calibrate(0, torch.stack([c[0] for c in cal]).float(), torch.stack([c[1] for c in cal]).float())
    k0 = torch.randn(B, n_kv, cap - 1, HD, generator=gen).half().to(dev)
    mgr._encode_kv(0, k0, k0.clone(), 0, cap - 1)
    mgr.seq_len = cap - 1
    gq, gk, gv = mgr.static_inputs(0)
    gq.copy_(torch.randn(gq.shape, generator=gen).half())
    gk.copy_(torch.randn(gk.shape, generator=gen).half())
    gv.copy_(torch.randn(gv.shape, generator=gen).half())
    mgr.layer_step(0)                          # fills the last slot (eager, sets kernel attributes)
    mgr.increment_seq_len()
    torch.cuda.synchronize()
    mgr.check_status()
    with pytest.raises(ValueError):
        mgr.layer_step(0)                      # the host-side check
    # the device-side check: launch the step kernels with the position one past the end, as a replayed graph would
    snap = [t.clone() for t in (mgr._k_packed, mgr._k_norms, mgr._v_packed, mgr._v_norms)]
    mgr._sync_pos()
    mgr._layer_step(0)
    torch.cuda.synchronize()
    for a, b in zip(snap, (mgr._k_packed, mgr._k_norms, mgr._v_packed, mgr._v_norms)):
        assert torch.equal(a, b)
    assert int(mgr._status.item()) == 2
    with pytest.raises(RuntimeError):
        mgr.check_status()
