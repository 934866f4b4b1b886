"""Fused multi-tier collision count, with the reference's Python surface
(cache_hub/collision_fused/collison_interface.py:60-86 and the extension module it loads)."""
from types import SimpleNamespace

import torch

from ... import ops, torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def _update_cache_cnt(sorted_cluster_ids, cluster_key_counts, code_book, tier_counts, cache_cnt):
    """Extension-module form: writes into `cache_cnt` (int32 [bs,H,N]); tier_counts has 1..8 entries."""
    ops.collision_fused(sorted_cluster_ids, cluster_key_counts, code_book, list(tier_counts), cache_cnt)


def load_kernel_module(path="collision.cu", name="update_cache_cnt", **_):
    """The reference JIT-compiles a .cu here; this build is ahead of time, so this only hands back an object
    with the extension's function."""
    return SimpleNamespace(update_cache_cnt=_update_cache_cnt)


def update_cache_cnt_cuda_interface(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts) -> torch.Tensor:
    """sorted_cluster_ids i64|i32 [bs,H,B,NC], cluster_key_counts i32 [bs,H,B,NC], codebook u8 [bs,H,B,N] (any
    strides), tier_counts list[int] -> cache_cnt i32 [bs,H,N]."""
    return torch.ops.pariskv.collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, [int(t) for t in tier_counts])
