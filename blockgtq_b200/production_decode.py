"""Model glue around the production cache for HF Llama-style models
(blockgtq/production_decode.py:11-99): one decode step and the online prefill."""
from __future__ import annotations

import torch

from .packed_kv_manager import _layer_kv

__all__ = ["production_decode_step", "production_prefill"]


@torch.no_grad()
def production_decode_step(model, input_ids, position_ids, cache):
    """embed -> per layer (norm, q/k/v projections, RoPE, packed-cache attention, MLP) -> norm + lm_head.
    input_ids / position_ids (B, 1) -> logits (B, 1, vocab)."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    hidden = model.model.embed_tokens(input_ids)
    for li, layer in enumerate(model.model.layers):
        resid = hidden
        hidden = layer.input_layernorm(hidden)
        attn = layer.self_attn
        B, S, _ = hidden.shape
        q = attn.q_proj(hidden).view(B, S, cache.nq, cache.hd).transpose(1, 2)
        k = attn.k_proj(hidden).view(B, S, cache.nkv, cache.hd).transpose(1, 2)
        v = attn.v_proj(hidden).view(B, S, cache.nkv, cache.hd).transpose(1, 2)
        rope = getattr(attn, "rotary_emb", None) or model.model.rotary_emb
        cos, sin = rope(v, position_ids)
        if S == 1 and q.dtype == torch.float16 and getattr(cache, "can_fuse_rope", False):
            out = cache.encode_and_attend(li, q, k, v, rope=(cos, sin))     # rotary embedding inside the append kernel
        else:
            q, k = apply_rotary_pos_emb(q, k, cos, sin)
            out = cache.encode_and_attend(li, q, k, v)
        out = out.transpose(1, 2).reshape(B, S, cache.nq * cache.hd).to(hidden.dtype)
        hidden = resid + attn.o_proj(out)
        resid = hidden
        hidden = resid + layer.mlp(layer.post_attention_layernorm(hidden))
    cache.increment_seq_len()
    return model.lm_head(model.model.norm(hidden))


@torch.no_grad()
def production_prefill(model, input_ids, cache, chunk_encode=64):
    """HF forward for the prompt, then bulk-encode the post-RoPE K/V of every layer into the packed
    cache in ``chunk_encode``-token pieces.  Works with the legacy ``key_cache`` lists and with the
    per-layer ``layers[i].keys/values`` cache objects of newer transformers.  Returns the prompt logits."""
    from transformers import DynamicCache
    prompt_len = input_ids.shape[1]
    position_ids = torch.arange(prompt_len, device=input_ids.device).unsqueeze(0)
    hf_cache = DynamicCache()
    out = model(input_ids, position_ids=position_ids, past_key_values=hf_cache, use_cache=True)
    for li in range(cache.n_layers):
        k, v = _layer_kv(hf_cache, li)
        for start in range(0, prompt_len, chunk_encode):
            end = min(start + chunk_encode, prompt_len)
            cache._encode_batched(li, k[:, :, start:end], v[:, :, start:end], start)
    cache.seq_len = prompt_len
    del hf_cache
    return out.logits
