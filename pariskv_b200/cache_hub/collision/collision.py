"""Single-tier (unfused) collision count with the reference's surface (cache_hub/collision/collision.py:87-98).
All tensors int32: sorted_cluster_ids [bs,H,B,NC], topk_cluster_cnt [bs,H,B], codebook [bs,H,B,N]."""
from types import SimpleNamespace

import torch

from ... import ops, torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def _update_cache_cnt(sorted_cluster_ids, topk_cluster_cnt, code_book, cache_cnt):
    """Extension-module form: code_book is the transposed layout [bs,H,N,B]."""
    ops.collision(sorted_cluster_ids, topk_cluster_cnt, code_book, cache_cnt)


def load_kernel_module(path="collision.cu", name="update_cache_cnt", **_):
    return SimpleNamespace(update_cache_cnt=_update_cache_cnt)


def update_cache_cnt_cuda(sorted_cluster_ids, topk_cluster_cnt, codebook) -> torch.Tensor:
    return torch.ops.pariskv.collision(sorted_cluster_ids, topk_cluster_cnt, codebook.transpose(-1, -2).contiguous())
