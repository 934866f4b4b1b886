"""Attention entry points with the reference's names and signatures (attn_hub/polar_attn.py:8-62)."""
import torch
import torch.nn.functional as F


def polar_prefill_attn(query_states, key_states, value_states, causal):
    """Dense prefill attention, [bs, seq, heads, dim] in and out.  Prefill is outside the decode hot path;
    this uses torch's fused scaled-dot-product attention with the KV heads expanded for GQA."""
    q = query_states.transpose(1, 2)
    k = key_states.transpose(1, 2)
    v = value_states.transpose(1, 2)
    rep = q.shape[1] // k.shape[1]
    if rep > 1:
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    out = F.scaled_dot_product_attention(q, k, v, is_causal=bool(causal) and q.shape[2] > 1)
    return out.transpose(1, 2).contiguous()


def polar_decode_attn(query_states, key_states, value_states, layer_idx, kv_cache):
    """Decode attention through the cache's retrieval path; key/value arguments are unused (the new row was
    appended by decode_update_kv_cache), as in the reference."""
    if kv_cache is None or not callable(getattr(kv_cache, "compute", None)):
        raise TypeError("polar_decode_attn expects kv_cache to provide compute(query_states, layer_idx), got "
                        f"{type(kv_cache).__module__}.{type(kv_cache).__name__}")
    return kv_cache.compute(query_states.contiguous(), layer_idx)
