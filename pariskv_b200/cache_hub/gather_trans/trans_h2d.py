"""UVA gathers from pinned host memory with the reference's surface (cache_hub/gather_trans/trans_h2d.py:65-105;
the packed variant follows the call site cache_hub/polar_cache_adaptivek_varlen.py:1634-1644)."""
import torch

from ... import ops, torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def h2d_gather_kv(src_k_caches, src_v_caches, selected_indices, dst_k_caches, dst_v_caches) -> None:
    bs, heads, kv_len, dim = src_k_caches.shape
    assert src_k_caches.shape == src_v_caches.shape and dst_k_caches.shape == dst_v_caches.shape
    assert dst_k_caches.shape[-2] >= selected_indices.shape[-1] and dim == 128
    assert src_k_caches.is_cpu and src_v_caches.is_cpu and src_k_caches.is_pinned() and src_v_caches.is_pinned()
    assert dst_k_caches.is_cuda and dst_v_caches.is_cuda
    assert src_k_caches.dtype == src_v_caches.dtype == dst_k_caches.dtype == dst_v_caches.dtype == torch.bfloat16
    torch.ops.pariskv.gather_trans(src_k_caches, src_v_caches, selected_indices, dst_k_caches, dst_v_caches)


def h2d_gather_kv_packed(k_cpu, v_cpu, k_packed, v_packed, indices_packed, cu_seqlens_topk, cu_seqlens_k,
                         sink_local_end, global_k) -> None:
    ops.h2d_gather_kv_packed(k_cpu, v_cpu, k_packed, v_packed, indices_packed, cu_seqlens_topk, cu_seqlens_k,
                             int(sink_local_end), int(global_k))
