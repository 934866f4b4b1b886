"""The seven ops of the retrieval path as torch custom ops (namespace ``pariskv``), a thin layer over the C ABI.

The reference binds its CUDA functions as pybind extension modules that it JIT-compiles at first use
(cache_hub/collision/collision.cu:279-281, cache_hub/collision_fused/collision.cu:395-416,
cache_hub/topk/radix_topk.cu:258-401, cache_hub/rerank/rerank.cu:222-224,
cache_hub/adaptive_k_fused/adaptive_topk.cu:272-314, cache_hub/gather/gather_cpu.cpp:116-174,
cache_hub/gather_trans/trans_h2d.cu:79-126).  Here every op is registered with ``torch.library`` so that the
dispatcher knows its schema, which arguments it writes, and (through the fake implementations) the shape and dtype
of what it returns; the mirror modules under ``cache_hub/`` call these ops.  Each implementation forwards to
``pariskv_b200.ops``, i.e. to ``libpariskv_b200.so``; there is no other backend and no CPU fallback (``gather`` is the
host-side row gather the reference also runs on the CPU).

    torch.ops.pariskv.collision(sorted_cluster_ids, topk_cluster_cnt, code_book) -> int32 [bs,H,N]
    torch.ops.pariskv.collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts) -> int32 [bs,H,N]
    torch.ops.pariskv.topk(input, k) -> int64 [..., k]
    torch.ops.pariskv.rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers) -> bf16 [bs,H,C]
    torch.ops.pariskv.adaptive_k_fused(sl_logits, cand_scores, cand_scale, sl_vnorm, cand_indices, cand_vnorm,
                                       threshold, topk_cap) -> (int64 [bs,H], int64 [bs,H,K_out])
    torch.ops.pariskv.gather(src, index, out) -> ()            (host memory; writes out)
    torch.ops.pariskv.gather_trans(src_k, src_v, selected_indices, dst_k, dst_v) -> ()   (writes dst_k, dst_v)
"""
from typing import List, Tuple

import torch

from . import ops

_lib = torch.library.Library("pariskv", "DEF")
_lib.define("collision(Tensor sorted_cluster_ids, Tensor topk_cluster_cnt, Tensor code_book) -> Tensor")
_lib.define("collision_fused(Tensor sorted_cluster_ids, Tensor cluster_key_counts, Tensor codebook, int[] tier_counts) -> Tensor")
_lib.define("topk(Tensor input, int k) -> Tensor")
_lib.define("rerank(Tensor coarse_indices, Tensor key_4bit, Tensor key_block_weight, Tensor q_blocks, Tensor q_norm, "
            "Tensor mag_centers) -> Tensor")
_lib.define("adaptive_k_fused(Tensor sl_logits, Tensor cand_scores, float cand_scale, Tensor sl_vnorm, Tensor cand_indices, "
            "Tensor cand_vnorm, float threshold, int topk_cap) -> (Tensor, Tensor)")
_lib.define("gather(Tensor src, Tensor index, Tensor(a!) out) -> ()")
_lib.define("gather_trans(Tensor src_k, Tensor src_v, Tensor selected_indices, Tensor(a!) dst_k, Tensor(b!) dst_v) -> ()")


# ---- implementations: the C ABI through pariskv_b200.ops ------------------------------------------------------------
def _collision(sorted_cluster_ids, topk_cluster_cnt, code_book):
    bs, H, N, B = code_book.shape
    out = torch.empty(bs, H, N, dtype=torch.int32, device=code_book.device)
    return ops.collision(sorted_cluster_ids.contiguous(), topk_cluster_cnt.contiguous(), code_book.contiguous(), out)


def _collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts: List[int]):
    return ops.collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, list(tier_counts))


def _topk(input, k: int):
    return ops.topk(input, int(k))


def _rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers):
    scores, _ = ops.rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers)
    return scores


def _adaptive_k_fused(sl_logits, cand_scores, cand_scale: float, sl_vnorm, cand_indices, cand_vnorm, threshold: float,
                      topk_cap: int) -> Tuple[torch.Tensor, torch.Tensor]:
    K_out = min(int(topk_cap), cand_scores.shape[-1])
    return ops.adaptive_topk(sl_logits.contiguous(), cand_scores, float(cand_scale), sl_vnorm, cand_indices, cand_vnorm,
                             float(threshold), K_out)


def _gather(src, index, out):
    ops.gather_kv_out_cpu(src, index, out)


def _gather_trans(src_k, src_v, selected_indices, dst_k, dst_v):
    ops.h2d_gather_kv(src_k, src_v, selected_indices, dst_k, dst_v)


_lib.impl("collision", _collision, "CUDA")
_lib.impl("collision_fused", _collision_fused, "CUDA")
_lib.impl("topk", _topk, "CUDA")
_lib.impl("rerank", _rerank, "CUDA")
_lib.impl("adaptive_k_fused", _adaptive_k_fused, "CUDA")
_lib.impl("gather", _gather, "CPU")
# the sources of gather_trans are pinned HOST tensors, the index and destinations CUDA tensors: mixed devices, so the
# op is registered for every dispatch key that such a call can land on
_lib.impl("gather_trans", _gather_trans, "CompositeExplicitAutograd")


# ---- fake (meta) implementations: shapes and dtypes only -------------------------------------------------------------
@torch.library.register_fake("pariskv::collision")
def _(sorted_cluster_ids, topk_cluster_cnt, code_book):
    bs, H, N, _ = code_book.shape
    return code_book.new_empty(bs, H, N, dtype=torch.int32)


@torch.library.register_fake("pariskv::collision_fused")
def _(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts):
    bs, H, _, N = codebook.shape
    return codebook.new_empty(bs, H, N, dtype=torch.int32)


@torch.library.register_fake("pariskv::topk")
def _(input, k):
    return input.new_empty(*input.shape[:-1], k, dtype=torch.int64)


@torch.library.register_fake("pariskv::rerank")
def _(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers):
    return coarse_indices.new_empty(coarse_indices.shape, dtype=torch.bfloat16)


@torch.library.register_fake("pariskv::adaptive_k_fused")
def _(sl_logits, cand_scores, cand_scale, sl_vnorm, cand_indices, cand_vnorm, threshold, topk_cap):
    bs, H, C = cand_scores.shape
    return (cand_indices.new_empty(bs, H, dtype=torch.int64), cand_indices.new_empty(bs, H, min(int(topk_cap), C), dtype=torch.int64))


@torch.library.register_fake("pariskv::gather")
def _(src, index, out):
    return None


@torch.library.register_fake("pariskv::gather_trans")
def _(src_k, src_v, selected_indices, dst_k, dst_v):
    return None


OPS = ("collision", "collision_fused", "topk", "rerank", "adaptive_k_fused", "gather", "gather_trans")
