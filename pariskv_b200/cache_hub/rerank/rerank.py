"""4-bit RaBitQ rerank with the reference's surface (cache_hub/rerank/rerank.py:214-263 and the extension
function of cache_hub/rerank/rerank.cu:141-224).  fp32 accumulation, correct for any batch size."""
from types import SimpleNamespace

import torch

from ... import ops, torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def _partial_rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, B, m, approx_scores,
                    v4b):
    """Extension-module form: fills approx_scores (bf16 [bs,H,C]); v4b (bf16 [bs,H,16,C,8]) may be None."""
    assert B == 16 and m == 8, "only B = 16, m = 8 is supported"
    ops.rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, approx_scores=approx_scores,
               v4b=v4b)


def load_kernel_module(path="rerank.cu", name="rerank", **_):
    return SimpleNamespace(partial_rerank=_partial_rerank)


def partial_rerank_cuda(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, B, m, kernel=None,
                        want_v4b: bool = False) -> tuple:
    """-> (approx_scores bf16 [bs,H,C], v4b).  The unpacked-level tensor v4b is a debug output that the cache
    never reads; it is produced only when want_v4b is set (None otherwise)."""
    assert coarse_indices.dtype == torch.int64, f"coarse_indices must be int64, got {coarse_indices.dtype}"
    assert coarse_indices.is_contiguous() and q_blocks.is_contiguous() and q_norm.is_contiguous()
    assert key_4bit.stride(-1) == 1
    assert B == 16 and m == 8, "only B = 16, m = 8 is supported"
    bs, H, C = coarse_indices.shape
    if not want_v4b:
        return torch.ops.pariskv.rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers), None
    v4b = torch.empty(bs, H, B, C, m, dtype=torch.bfloat16, device=coarse_indices.device)
    scores, _ = ops.rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, v4b=v4b)
    return scores, v4b


def rerank_rabitq_fused(cache_cnt, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, candidate_ratio,
                        final_topk, B, m) -> tuple:
    """Candidate top-k by count, rerank, final top-k (cache_hub/rerank/rerank.py:266-294).
    Returns (final_indices ascending, approx_scores bf16, None)."""
    import math
    kv_len = cache_cnt.shape[-1]
    C = max(1, math.ceil(kv_len * candidate_ratio))
    cand = ops.topk(cache_cnt, C)
    if C <= final_topk:
        return cand[:, :, :final_topk], None, None
    sbf, s32 = ops.rerank(cand, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, want_f32=True)
    return ops.final_topk(s32, cand, final_topk), sbf, None
