"""Top-k ops with the reference's surface (cache_hub/topk/__init__.py:23-155, extension functions of
cache_hub/topk/radix_topk.cu:258-401).  Both names run the same exact, deterministic selection: the set is the
first k of (value descending, index ascending) and the indices come back in ascending order, int64."""
from types import SimpleNamespace

import torch

from ... import torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def _topk_2d(input, k):
    assert input.dim() == 2, "input must be 2D [B, L]"
    return torch.ops.pariskv.topk(input, int(k))


def _topk_3d(input, k):
    assert input.dim() == 3, "input must be 3D [bs, kv_heads, kv_len]"
    return torch.ops.pariskv.topk(input, int(k))


def load_radix_topk_ext(verbose: bool = False):
    return SimpleNamespace(bucket_topk=_topk_2d, bucket_topk_3d=_topk_3d, radix_topk=_topk_2d, radix_topk_3d=_topk_3d)


def bucket_topk(input: torch.Tensor, k: int) -> torch.Tensor:
    assert input.is_cuda, "input must be on CUDA"
    assert k > 0, f"k must be positive, got {k}"
    if input.dim() not in (2, 3):
        raise ValueError(f"input must be 2D or 3D, got {input.dim()}D")
    return torch.ops.pariskv.topk(input, int(k))


radix_topk = bucket_topk


def fast_topk(input: torch.Tensor, k: int) -> torch.Tensor:
    return bucket_topk(input, k)


def fast_topk_with_ratio(input: torch.Tensor, ratio: float) -> torch.Tensor:
    if input.dim() not in (2, 3):
        raise ValueError(f"input must be 2D or 3D, got {input.dim()}D")
    return fast_topk(input, max(1, int(input.shape[-1] * ratio)))
