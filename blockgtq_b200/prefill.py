"""Layer-major prefill into the production cache (blockgtq/prefill.py:25-125): every layer encodes the
whole prompt's K/V into the packed cache and then attends all prompt positions against it in ONE
prefill-attention launch covering every KV head, so no fp16 KV cache is ever materialised."""
from __future__ import annotations

import torch

from .layer import prefill_attention, rotate_q_bulk

__all__ = ["layer_major_prefill"]


@torch.no_grad()
def layer_major_prefill(model, cache, prompt_ids, block_q=32, block_t=128):
    """model: HF Llama-style; cache: :class:`BlockGTQProductionCache`; prompt_ids (1, T).
    Fills cache rows [0, T) of every layer and sets ``cache.seq_len = T``.  ``block_q`` / ``block_t``
    are the reference kernel's tile sizes and are ignored here.  Returns the final hidden states
    (1, T, hidden) (the reference returns nothing; callers that ignore the value are unaffected)."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    B, T = prompt_ids.shape
    assert B == 1, "layer_major_prefill supports B=1 only"
    mgr = cache._mgr
    hidden = model.model.embed_tokens(prompt_ids)
    pos = torch.arange(T, device=prompt_ids.device).unsqueeze(0)
    for li, layer in enumerate(model.model.layers):
        resid = hidden
        hidden = layer.input_layernorm(hidden)
        attn = layer.self_attn
        q = attn.q_proj(hidden).view(B, T, cache.nq, cache.hd).transpose(1, 2)
        k = attn.k_proj(hidden).view(B, T, cache.nkv, cache.hd).transpose(1, 2)
        v = attn.v_proj(hidden).view(B, T, cache.nkv, cache.hd).transpose(1, 2)
        rope = getattr(attn, "rotary_emb", None) or model.model.rotary_emb
        cos, sin = rope(v, pos)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        cache._encode_batched(li, k, v, 0)
        lt = mgr._layers[li]
        baked = all(cache.quantizers[li][h]._q_perm_baked for h in range(cache.nkv))
        q16 = q.to(torch.float16)
        q_rot = q16.contiguous() if baked else rotate_q_bulk(lt, q16)
        out = prefill_attention(lt, q_rot, mgr._k_packed[li], mgr._k_norms[li], mgr._v_packed[li], mgr._v_norms[li],
                                T, q_pos_offset=0, causal=True, scale=cache.scale, flags=mgr._dec_flags,
                                v_rot=lt.v_rot)
        out = out.transpose(1, 2).reshape(B, T, cache.nq * cache.hd).to(hidden.dtype)
        hidden = resid + attn.o_proj(out)
        resid = hidden
        hidden = resid + layer.mlp(layer.post_attention_layernorm(hidden))
    cache.seq_len = T
    return hidden
