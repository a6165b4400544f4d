"""Calibration helpers with the reference's names (blockgtq/calibration.py:34-188): collect per-(layer,
KV-head) Q/K activations from an HF Llama-style model, build quantizers, bake query rotations."""
from __future__ import annotations

import torch

from .quantizer import BlockGTQQuantizer, build_batched_encode_args

__all__ = ["collect_qk_activations", "build_quantizers", "bake_q_rotations", "save_calib_cache", "load_calib_cache"]


@torch.no_grad()
def collect_qk_activations(model, enc, device, n_calib_tokens=256, post_rope=True, effective_len=None):
    """One forward over the first ``n_calib_tokens`` ids with hooks on every q_proj/k_proj.
    Returns ``{layer: {'q': (nkv, gqa*T, hd), 'k': (nkv, T, hd)}}`` (every query head of a KV group is kept
    as its own sample).  ``post_rope`` applies RoPE at positions 0..T-1 (stretched to ``effective_len``)."""
    ids = enc[:, :n_calib_tokens].to(device)
    cfg = model.config
    hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    nq = cfg.num_attention_heads
    nkv = getattr(cfg, "num_key_value_heads", nq)
    gqa = nq // nkv
    T = ids.size(1)
    pos = None
    if effective_len is not None:
        if effective_len < T:
            raise ValueError(f"effective_len ({effective_len}) must be >= n_calib_tokens ({T})")
        pos = torch.arange(0, T * (effective_len // T), effective_len // T, device=device).unsqueeze(0)
    data, handles = {}, []
    for li, layer in enumerate(model.model.layers):
        data[li] = {}

        def k_hook(_m, _i, out, li=li):
            data[li]["k"] = out.detach().reshape(-1, nkv, hd).permute(1, 0, 2)

        def q_hook(_m, _i, out, li=li):
            data[li]["q"] = out.detach().reshape(-1, nkv, gqa, hd).permute(1, 2, 0, 3).reshape(nkv, -1, hd)

        handles += [layer.self_attn.k_proj.register_forward_hook(k_hook),
                    layer.self_attn.q_proj.register_forward_hook(q_hook)]
    model(ids, position_ids=pos) if pos is not None else model(ids)
    for h in handles:
        h.remove()
    if post_rope:
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        rope = getattr(model.model.layers[0].self_attn, "rotary_emb", None) or model.model.rotary_emb
        p = pos if pos is not None else torch.arange(T, device=device).unsqueeze(0)
        cos, sin = rope(torch.zeros(1, 1, T, hd, device=device, dtype=torch.float16), p)
        for li in data:
            k, q = data[li]["k"], data[li]["q"]
            q3 = q.reshape(-1, k.shape[1], hd).unsqueeze(0).to(cos.dtype)
            q_r, _ = apply_rotary_pos_emb(q3, q3, cos, sin)
            k4 = k.unsqueeze(0).to(cos.dtype)
            _, k_r = apply_rotary_pos_emb(k4, k4, cos, sin)
            data[li]["q"] = q_r[0].reshape(nkv, -1, hd).to(q.dtype)
            data[li]["k"] = k_r[0].to(k.dtype)
    return data


def build_quantizers(layer_data, n_layers, nkv, hd, k_avg_bits=3.0, v_bits=3, k_nibble=True, device="cuda"):
    """-> (quantizers[li][hi], batched_args[li], kernel_args[li][hi])."""
    quantizers = [[None] * nkv for _ in range(n_layers)]
    kernel_args = [[None] * nkv for _ in range(n_layers)]
    batched = [None] * n_layers
    for li in range(n_layers):
        for hi in range(nkv):
            qz = BlockGTQQuantizer(head_dim=hd, avg_bits=k_avg_bits, device=device)
            qz.calibrate(layer_data[li]["q"][hi].contiguous(), layer_data[li]["k"][hi].contiguous())
            qz.init_v_quantizer(v_bits=v_bits, seed=42 + hi)
            quantizers[li][hi] = qz
            kernel_args[li][hi] = qz.build_kernel_args()
        batched[li] = build_batched_encode_args(quantizers[li], device=device)
    return quantizers, batched, kernel_args


def bake_q_rotations(model, quantizers, n_layers, nkv, nq):
    """Fold each head's permutation + rotation into q_proj in place; decode then skips the rotation."""
    for li in range(n_layers):
        attn = model.model.layers[li].self_attn
        for hi in range(nkv):
            quantizers[li][hi].bake_permutation_into_qproj(
                attn.q_proj.weight.data, kv_head_idx=hi, n_kv_heads=nkv, n_q_heads=nq,
                q_proj_bias=getattr(attn.q_proj, "bias", None))


def save_calib_cache(path, layer_data, model_name="", arch="llama", source="", score="energy"):
    """Write the collected activations in the reference's calib-cache layout
    (examples/build_calib_cache.py:282-298): one ``torch.save`` payload with ``calib_k``
    (n_layer, n_kv, T, hd), ``calib_q`` (n_layer, n_kv, gqa*T, hd) and the shape metadata."""
    n_layer = len(layer_data)
    k0, q0 = layer_data[0]["k"], layer_data[0]["q"]
    n_kv, T, hd = k0.shape
    calib_k = torch.stack([layer_data[li]["k"].detach().cpu() for li in range(n_layer)])
    calib_q = torch.stack([layer_data[li]["q"].detach().cpu() for li in range(n_layer)])
    q_per_kv = q0.shape[1] // T
    payload = {"calib_k": calib_k, "calib_q": calib_q, "model": model_name, "arch": arch, "n_tokens": T,
               "head_dim": hd, "n_kv": n_kv, "n_q": n_kv * q_per_kv, "n_layer": n_layer, "q_per_kv": q_per_kv,
               "n_samples_q": q0.shape[1], "q_convention": "all_heads_per_kv_group", "source": source, "score": score}
    torch.save(payload, path)
    return payload


def load_calib_cache(path, device="cpu"):
    """Read a calib cache (this module's or the reference's) back into the ``layer_data`` form
    :func:`build_quantizers` takes: ``{layer: {'q': (n_kv, gqa*T, hd), 'k': (n_kv, T, hd)}}``."""
    ck = torch.load(path, map_location="cpu", weights_only=False)
    ks, qs = ck["calib_k"], ck["calib_q"]
    if ks.dim() != 4 or qs.dim() != 4 or ks.shape[:2] != qs.shape[:2] or ks.shape[3] != qs.shape[3]:
        raise ValueError(f"not a calib cache: calib_k {tuple(ks.shape)}, calib_q {tuple(qs.shape)}")
    return {li: {"k": ks[li].to(device), "q": qs[li].to(device)} for li in range(ks.shape[0])}
