"""Multi-GPU forms of the retrieval path: one process per GPU, torch.distributed for the plumbing.

Two ways the path shards (the reference itself is single-GPU; `cache_hub/polar_cache.py:171` puts the whole
cache on one device):

* KV heads (tensor-parallel models): every stage is independent per (batch, KV head), so each rank builds its
  cache with `num_key_value_heads / world` heads and runs the unchanged single-GPU path.  No collective on the
  retrieval path; `head_shard()` gives the slice.
* The sequence (million-token contexts): the searchable zone is cut into equal contiguous chunks, one per
  rank, each with its codes / 4-bit records in its own HBM and its K/V rows in its own pinned host memory.
  Per layer and step every rank runs the local chain (collision -> candidates -> rerank -> local top-K) with
  GLOBAL tier thresholds and the GLOBAL cluster histogram, then `merge_local_topk` all-gathers
  (fp32 score, global key index) and every rank selects the same global top-K; each rank attends only the
  selected rows it owns (rank 0 also the window) and `merge_partial_attention` combines the partial results
  through their log-sum-exp.  Two small all-gathers per layer (K * 12 bytes and Hq * 260 bytes per rank).

The selection inside `merge_local_topk` is pluggable so that the exchange can be tested with gloo ranks on
CPU; on GPUs the default selector is the CUDA top-k of this library.
"""
import math

import torch
import torch.distributed as dist


def head_shard(num_kv_heads: int, rank: int, world: int) -> slice:
    """KV heads owned by `rank` when heads are split evenly over `world` ranks."""
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not split evenly over {world} ranks")
    per = num_kv_heads // world
    return slice(rank * per, (rank + 1) * per)


def sequence_shard(n_keys: int, rank: int, world: int):
    """(start, end) of the contiguous chunk of a zone of n_keys owned by `rank` (equal chunks, last may be short)."""
    per = (n_keys + world - 1) // world
    start = min(n_keys, rank * per)
    return start, min(n_keys, start + per)


def local_plan(n_total: int, world: int, collision_ratio: float, candidate_ratio: float, final_topk: int,
               tier_ratios=(0.05, 0.15, 0.30, 0.50, 0.75, 1.0)):
    """Launch parameters of one shard: tier thresholds from the GLOBAL zone length, a per-shard candidate budget of
    ceil(C_total / world) and a local top-K of min(K, C_local)."""
    tiers = [int(math.ceil(n_total * collision_ratio * r)) for r in tier_ratios]
    c_total = max(1, int(math.ceil(n_total * candidate_ratio)))
    c_local = max(1, (c_total + world - 1) // world)
    return tiers, c_local, min(final_topk, c_local)


def allreduce_cluster_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the per-shard code histograms into the global one (done at prefill and after every flush)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)
    return counts


def _default_select(scores, indices, k):
    from . import ops
    return ops.final_topk(scores.contiguous(), indices.contiguous(), k)


def merge_local_topk(local_scores: torch.Tensor, local_indices: torch.Tensor, k: int, group=None, select=None):
    """All-gather every rank's local top list and select the global top-k.

    local_scores  fp32 [bs,H,Kl]; local_indices int64 [bs,H,Kl] GLOBAL key indices, ascending per row (shards are
    ascending contiguous chunks, so the rank-major concatenation is ascending too and "lowest position first"
    is "lowest key index first").  Kl must be the same on every rank; pad with score -inf and any index.
    Returns int64 [bs,H,k] global key indices in ascending order, identical on every rank."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    select = select or _default_select
    if world == 1:
        return select(local_scores, local_indices, k)
    bs, H, Kl = local_scores.shape
    # one buffer, one collective: scores as raw bits next to the indices
    packed = torch.empty(bs, H, Kl, 2, dtype=torch.int64, device=local_scores.device)
    packed[..., 0] = local_scores.contiguous().view(torch.int32).to(torch.int64)
    packed[..., 1] = local_indices
    flat = torch.empty(world * bs, H, Kl, 2, dtype=torch.int64, device=local_scores.device)
    dist.all_gather_into_tensor(flat, packed, group=group)   # output = inputs concatenated along dim 0
    gathered = flat.view(world, bs, H, Kl, 2)
    g = gathered.permute(1, 2, 0, 3, 4).reshape(bs, H, world * Kl, 2)
    scores = g[..., 0].to(torch.int32).view(torch.float32)
    return select(scores.contiguous(), g[..., 1].contiguous(), k)


def owned_rows(global_indices: torch.Tensor, start: int, end: int):
    """Split the global selection into this rank's rows: returns (local_indices [bs,H,K] with the owned rows first,
    n_owned int32 [bs,H]).  Rows outside [start, end) are moved behind the owned ones (stable), so the attention
    kernel can take `n_sel = n_owned`."""
    mine = (global_indices >= start) & (global_indices < end)
    order = torch.sort((~mine).to(torch.int8), dim=-1, stable=True).indices
    local = torch.gather(global_indices, -1, order) - start
    return local.clamp_(0, max(end - start - 1, 0)).contiguous(), mine.sum(-1).to(torch.int32).contiguous()


def merge_partial_attention(out: torch.Tensor, lse: torch.Tensor, group=None) -> torch.Tensor:
    """Combine attention results computed over disjoint row sets.  out bf16/f32 [bs,1,Hq,128] (normalised over
    the local rows), lse fp32 [bs,Hq] = log2 of the local softmax denominator (-inf when the rank had no rows).
    Returns the exact softmax over the union, same dtype as out, identical on every rank."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return out
    bs, _, Hq, D = out.shape
    packed = torch.empty(bs, Hq, D + 1, dtype=torch.float32, device=out.device)
    packed[..., :D] = out[:, 0].float()
    packed[..., D] = lse
    flat = torch.empty(world * bs, Hq, D + 1, dtype=torch.float32, device=out.device)
    dist.all_gather_into_tensor(flat, packed, group=group)
    gathered = flat.view(world, bs, Hq, D + 1)
    l = gathered[..., D]                                        # [world,bs,Hq]
    m = l.max(dim=0, keepdim=True).values
    w = torch.where(torch.isinf(l) & (l < 0), torch.zeros_like(l), torch.exp2(l - torch.where(torch.isinf(m), torch.zeros_like(m), m)))
    denom = w.sum(0).clamp_min(1e-38)
    merged = (gathered[..., :D] * w.unsqueeze(-1)).sum(0) / denom.unsqueeze(-1)
    return merged.unsqueeze(1).to(out.dtype)


def sequence_sharded_attend(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, counts_global, store_k,
                            store_v, n_total, start, end, collision_ratio, candidate_ratio, final_topk,
                            window_k=None, window_v=None, n_window=0, group=None):
    """One layer, one decode step of the sequence-sharded form on this rank's shard [start, end) of a zone of
    n_total keys.  codebook / key_block_weight / key_4bit / store_* hold the shard only (local index = global -
    start); counts_global is the all-reduced cluster histogram.  The window rows are attended by the rank that
    passes them (rank 0).  Returns (attention output identical on every rank, global top-K indices)."""
    from . import ops
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    tiers, c_local, k_local = local_plan(n_total, world, collision_ratio, candidate_ratio, final_topk)
    fin_local, ex = ops.retrieve(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, counts_global,
                                 tiers, c_local, k_local, want=("cand", "scores_f32"))
    scores = torch.gather(ex["scores_f32"], 2, torch.searchsorted(ex["cand"], fin_local))
    final = merge_local_topk(scores, fin_local + start, min(final_topk, world * k_local), group)
    local, n_owned = owned_rows(final, start, end)
    bs, _, Hq, _ = queries.shape
    lse = torch.empty(bs, Hq, dtype=torch.float32, device=queries.device)
    out = ops.sparse_attention(queries, window_k, window_v, n_window, store_k, store_v, local, n_sel=n_owned, lse=lse)
    return merge_partial_attention(out, lse, group), final
