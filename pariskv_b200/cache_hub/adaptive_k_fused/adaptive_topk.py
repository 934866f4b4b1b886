"""Fused adaptive-k with the reference's surface (cache_hub/adaptive_k_fused/adaptive_topk.py:331-405 and the
extension function of adaptive_topk.cu:272-314)."""
from types import SimpleNamespace

import torch

from ... import ops, torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def _adaptive_topk(sl_logits, cand_logits, sl_vnorm, cand_indices, cand_vnorm, threshold, K_out, adaptive_k,
                   topk_indices):
    """Extension-module form (v1): fp32 logits that are already scaled; outputs are written in place."""
    ops.adaptive_topk(sl_logits, cand_logits, 1.0, sl_vnorm, cand_indices, cand_vnorm, float(threshold), int(K_out),
                      adaptive_k=adaptive_k, topk_indices=topk_indices)


def load_kernel_module(path="adaptive_topk.cu", name="adaptive_topk", **_):
    return SimpleNamespace(adaptive_topk=_adaptive_topk)


def adaptive_topk_cuda(query_avg, sink_local_keys, sl_vnorm, cand_scores, cand_indices, cand_vnorm, attn_scale,
                       threshold, topk_cap, kernel=None):
    """-> (adaptive_k i64 [bs,H], topk_indices i64 [bs,H,min(topk_cap, C)], benefit descending)."""
    assert query_avg.dtype == torch.bfloat16 and sink_local_keys.dtype == torch.bfloat16
    assert sl_vnorm.dtype == torch.float32 and cand_vnorm.dtype == torch.float32
    assert cand_scores.dtype == torch.bfloat16 and cand_indices.dtype == torch.int64
    assert 0.0 < threshold <= 1.0 and topk_cap > 0 and attn_scale > 0
    K_out = min(int(topk_cap), cand_scores.shape[-1])
    # the sink/local logits are a small dense product: left to the library, as the reference does
    sl_logits = torch.einsum("bhd,bhkd->bhk", query_avg, sink_local_keys).to(torch.float32) * attn_scale
    return torch.ops.pariskv.adaptive_k_fused(sl_logits.contiguous(), cand_scores, float(attn_scale), sl_vnorm, cand_indices,
                                              cand_vnorm, float(threshold), K_out)
