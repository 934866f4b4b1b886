"""Multi-GPU forms of the retrieval path: one process per GPU, torch.distributed for the plumbing.

Two ways the path shards (the reference itself is single-GPU; `cache_hub/polar_cache.py:171` puts the whole
cache on one device):

* KV heads (tensor-parallel models): every stage is independent per (batch, KV head), so each rank builds its
  cache with `num_key_value_heads / world` heads and runs the unchanged single-GPU path.  No collective on the
  retrieval path; `head_shard()` gives the slice.
* The sequence (million-token contexts): the searchable zone is cut into equal contiguous chunks, one per
  rank, each with its codes / 4-bit records in its own HBM and its K/V rows in its own HBM (when they fit) or
  pinned host memory.  Per layer and step every rank counts collisions over its chunk with GLOBAL tier thresholds
  and the GLOBAL cluster histogram; the ranks all-gather their count histograms, so every rank knows the global
  threshold count and its share of the ties and keeps exactly its part of the single-GPU candidate set; after the
  rerank the ranks exchange (fp32 score, global key index) of their local top-K lists and every rank selects the
  same global top-K - the single-GPU selection, bit for bit; each rank attends only the selected rows it owns
  (rank 0 also the window) and an exchange of (partial output, log2 denominator) gives every rank the exact softmax
  over the union.  `SequenceShardedCache` / `sequence_sharded_attend` run the
  exchanges either as two small NCCL all-gathers with CUDA packing / unpacking kernels around them, or as
  stores into peer memory with flag words (`PeerExchange`).

`merge_local_topk`, `owned_rows` and `merge_partial_attention` are the same exchanges written with torch ops and a
pluggable selector: they run on CPU tensors with gloo ranks and are what the host-side tests exercise; on GPUs
the CUDA entry points (`pk_shard_*`) do this work.
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


def global_plan(n_total: int, collision_ratio: float, candidate_ratio: float, final_topk: int,
                tier_ratios=(0.05, 0.15, 0.30, 0.50, 0.75, 1.0)):
    """Launch parameters shared by every shard: tier thresholds, candidate count and final K of the WHOLE zone,
    exactly as a single GPU would use them (cache_hub/polar_cache.py:1221-1222, :1239-1240, :1300)."""
    tiers = [int(math.ceil(n_total * collision_ratio * r)) for r in tier_ratios]
    c_total = max(1, int(math.ceil(n_total * candidate_ratio)))
    return tiers, c_total, min(final_topk, c_total)


def shard_candidate_plan(shard_hist: torch.Tensor, rank: int, c_total: int):
    """What the selection kernel derives from the all-gathered count histograms (host-side mirror, any device):
    shard_hist int [world,bs,H,256] = how many keys of every shard have each collision count.  Returns
    (T [bs,H], ties [bs,H], n_cand [bs,H]): shard `rank` takes every key with count > T, and the first `ties` of its
    keys with count == T in key order; the union over the shards is the single-GPU candidate set - the c_total keys
    with the highest counts, ties going to the lowest key index - because the shards are contiguous and in key order."""
    h = shard_hist.to(torch.int64)
    total = h.sum(0)                                                   # [bs,H,256]
    suffix = torch.flip(torch.cumsum(torch.flip(total, [-1]), -1), [-1])   # keys with count >= bin
    T = (suffix >= c_total).to(torch.int64).sum(-1) - 1                # highest bin whose suffix reaches c_total
    T = T.clamp_(min=0)
    above = torch.gather(suffix, -1, (T + 1).clamp(max=255).unsqueeze(-1)).squeeze(-1)
    above = torch.where(T >= 255, torch.zeros_like(above), above)
    quota = c_total - above                                            # ties of count T taken over the whole zone
    eq = torch.gather(h, -1, T.view(1, *T.shape, 1).expand(h.shape[0], *T.shape, 1)).squeeze(-1)   # [world,bs,H]
    before = eq[:rank].sum(0)
    ties = torch.minimum((quota - before).clamp(min=0), eq[rank])
    mine = h[rank]
    idx = torch.arange(256, device=h.device).view(1, 1, 256)
    gt = torch.where(idx > T.unsqueeze(-1), mine, torch.zeros_like(mine)).sum(-1)
    return T, ties, gt + ties


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
    return merge_gathered_partials(flat.view(world, bs, Hq, D + 1)).to(out.dtype)


def merge_gathered_partials(gathered: torch.Tensor) -> torch.Tensor:
    """gathered fp32 [world,bs,Hq,D+1] = (partial output, log2 denominator) of every rank -> fp32 [bs,1,Hq,D]."""
    D = gathered.shape[-1] - 1
    l = gathered[..., D]                                        # [world,bs,Hq]
    m = l.max(dim=0, keepdim=True).values
    w = torch.where(torch.isinf(l) & (l < 0), torch.zeros_like(l), torch.exp2(l - torch.where(torch.isinf(m), torch.zeros_like(m), m)))
    denom = w.sum(0).clamp_min(1e-38)
    merged = (gathered[..., :D] * w.unsqueeze(-1)).sum(0) / denom.unsqueeze(-1)
    return merged.unsqueeze(1)


def sequence_sharded_attend(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, counts_global, store_k,
                            store_v, n_total, start, end, collision_ratio, candidate_ratio, final_topk,
                            window_k=None, window_v=None, n_window=0, group=None, n_window_dev=None, n_window_add=0,
                            exchange=None, scratch=None, attn_scratch=None, hist_gather=None):
    """One layer, one decode step of the sequence-sharded form on this rank's shard [start, end) of a zone of
    n_total keys.  codebook / key_block_weight / key_4bit / store_* hold the shard only (local index = global -
    start); counts_global is the all-reduced cluster histogram.  The window rows are attended by the rank that
    passes them (rank 0).

    The selection is the single-GPU selection: every shard counts collisions with the global thresholds, the ranks
    all-gather their 256-bin count histograms, and each takes the keys above the GLOBAL threshold count plus its
    share of the ties in rank (= key) order, so the union of the shards' candidates is the single-GPU candidate set;
    the global top-K of the shards' local top-K lists is then the single-GPU final selection.  Three small exchanges
    per layer: histograms (1 KB per head), local top lists (16 B x K per head), partial attention results.
    exchange (a PeerExchange) turns the two larger exchanges into stores into peer memory, hist_gather (a TPReducer in
    peer mode with room for bs*H*512 elements) the histogram all-gather too; without them they are NCCL collectives.
    Returns (attention output identical on every rank, global top-K indices)."""
    from . import ops
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    tiers, c_total, k_final = global_plan(n_total, collision_ratio, candidate_ratio, final_topk)
    if world == 1:   # the whole zone is local: the plain chain, nothing to exchange
        final, _ = ops.retrieve(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, counts_global,
                                tiers, c_total, k_final, scratch=scratch)
        return ops.sparse_attention(queries, window_k, window_v, n_window, store_k, store_v, final,
                                    n_window_dev=n_window_dev, n_window_add=n_window_add, scratch=attn_scratch), final
    bs, _, Hq, _ = queries.shape
    H, dev = codebook.shape[1], queries.device
    n_local = codebook.shape[3]
    row = min(c_total, n_local)
    bufs = {"cand": torch.empty(bs, H, row, dtype=torch.int64, device=dev),
            "scores_f32": torch.empty(bs, H, row, dtype=torch.float32, device=dev)}
    args = (queries, signs, mag_centers, codebook, key_block_weight, key_4bit, counts_global, c_total, k_final)
    # phase 1: collision counts of the shard, and how many of its keys have each count
    _, _, ex = ops.retrieve_ex(*args, tier_counts=tiers, phase=1, outputs=bufs, scratch=scratch)
    if hist_gather is not None:   # over peer memory: the gather kernel moves 32-bit words, whatever they hold
        hist_all = hist_gather.all_gather(ex["local_hist"].view(torch.bfloat16).view(1, -1)).view(torch.int32)
    else:
        hist_all = torch.empty(world * bs, H, 256, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(hist_all, ex["local_hist"], group=group)
    # phase 2: candidates by the global threshold, rerank, local top-K
    fin_local, n_sel, ex = ops.retrieve_ex(*args, tier_counts=tiers, phase=2, shard_hist=hist_all.view(world, bs, H, 256),
                                           world=world, rank=rank, outputs=bufs, scratch=scratch)
    n_cand = ex["n_cand"]
    if exchange is not None:   # the two larger exchanges as stores into peer memory (no collective launch)
        ops.shard_exchange_topk(ex["cand"], ex["scores_f32"], fin_local, start, exchange, n_sel=n_sel, n_cand=n_cand)
        scores, indices = ops.shard_collect_topk(exchange, bs, H, k_final)
    else:
        packed = ops.shard_pack_topk(ex["cand"], ex["scores_f32"], fin_local, start, n_sel=n_sel, n_cand=n_cand)
        flat = torch.empty(world * bs, H, k_final, 2, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(flat, packed, group=group)          # output = inputs concatenated along dim 0
        scores, indices = ops.shard_unpack_topk(flat.view(world, bs, H, k_final, 2))
    final = ops.final_topk(scores, indices, k_final)
    local, n_owned = ops.shard_owned_rows(final, start, end)
    lse = torch.empty(bs, Hq, dtype=torch.float32, device=dev)
    out = ops.sparse_attention(queries, window_k, window_v, n_window, store_k, store_v, local, n_sel=n_owned, lse=lse,
                               n_window_dev=n_window_dev, n_window_add=n_window_add, scratch=attn_scratch)
    if exchange is not None:
        ops.shard_exchange_partial(out, lse, exchange)
        return ops.shard_collect_partial(exchange, bs, Hq), final
    part = ops.shard_pack_partial(out, lse)
    flat2 = torch.empty(world * bs, Hq, 129, dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(flat2, part, group=group)
    return ops.shard_merge_partial(flat2.view(world, bs, Hq, 129)), final


class TPReducer:
    """The reduction of a tensor-parallel model's row-parallel projections at decode time: out = residual + sum over
    ranks of partial, for bf16 vectors of n elements.  With KV heads split over ranks (head_shard) this is the only
    exchange the model needs; the retrieval path itself has none.

    mode "peer": one launch over peer memory (pk_tp_allreduce): every data word goes into every peer's symmetric
    buffer together with the exchange number in one 8-byte store, the receiver polls its slots (bounded), fp32 sum in
    rank order, bit-identical on every rank; no NVLink multicast objects are created.
    mode "nccl": torch.distributed.all_reduce followed by the residual add.  A single rank needs neither."""

    def __init__(self, n, device, group=None, mode="peer"):
        self.n, self.device = int(n), device
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        if mode not in ("peer", "nccl"):
            raise ValueError("mode must be 'peer' or 'nccl'")
        self.mode = mode if self.world > 1 else "none"
        if self.mode == "peer":
            import os
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            from . import _lib
            if self.world > 16:
                raise ValueError("at most 16 ranks")
            self.area_bytes = (self.world * self.n * 4 + 255) // 256 * 256    # 8-byte slots: {two bf16, exchange number}
            self.flags_off = 2 * self.area_bytes
            self.buf = symm.empty(self.flags_off + 256, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm.rendezvous(self.buf, self.group.group_name)
            self.peer_array = _lib.u64_array([int(p) for p in self.handle.buffer_ptrs])
            self.ctl = torch.zeros(4, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)        # every rank's flags are zero before any store

    def reduce(self, partial, residual):
        """partial, residual: bf16 [1, n] -> bf16 [1, n], identical on every rank."""
        if self.mode == "none":
            return residual + partial
        if self.mode == "nccl":
            dist.all_reduce(partial, group=self.group)
            return residual + partial
        from . import ops
        return ops.tp_allreduce(partial.contiguous(), residual.contiguous(), self)

    def reduce_norm(self, partial, residual, weight, eps=1e-6):
        """(h, x): h = residual + sum over ranks of partial, x = RMS-norm(h) * weight.  In peer mode one launch does
        the exchange, the sum and the norm; otherwise the collective is followed by one add + norm launch."""
        from . import ops
        if self.mode == "peer":
            return ops.tp_allreduce(partial.contiguous(), residual.contiguous(), self, norm_weight=weight, eps=eps)
        if self.mode == "nccl":
            dist.all_reduce(partial, group=self.group)
        return ops.add_rmsnorm(partial, residual, weight, eps)

    def all_gather(self, part):
        """part: bf16 [1, m] (m <= n) -> bf16 [1, world * m], the ranks' parts in rank order."""
        if self.mode == "none":
            return part
        if part.numel() > self.n:
            raise ValueError("a rank's part must fit the reducer's row length")
        if self.mode == "nccl":
            out = torch.empty(1, self.world * part.numel(), dtype=part.dtype, device=part.device)
            dist.all_gather_into_tensor(out.view(self.world, -1), part.contiguous(), group=self.group)
            return out
        from . import ops
        return ops.tp_allgather(part.contiguous(), self)

    def check(self):
        """Raise if a bounded wait ran out (host synchronisation: call it outside the decode loop)."""
        if self.mode == "peer" and int(self.ctl.cpu()[2]):
            raise RuntimeError("tensor-parallel reduce: a peer's data did not arrive within the wait limit")


class PeerExchange:
    """Symmetric buffers for the two per-layer exchanges of the sequence-sharded form, so that they run as stores
    into peer memory plus flag words instead of two collectives (pk_shard_exchange_* / pk_shard_collect_*).

    One buffer per rank from torch's symmetric-memory allocator (same layout everywhere, every peer's copy mapped
    into this process): [gather 1 | gather 2 | flags 1 | flags 2].  NVLink multicast is not used and is switched
    off for the allocator (TORCH_SYMM_MEM_DISABLE_MULTICAST=1 must be in the environment before the first
    allocation; this constructor sets it if absent).  All ranks of `group` must construct it together."""

    def __init__(self, bs, H, Hq, Kl, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 16:
            raise ValueError("at most 16 ranks")
        self.device, self.bs, self.H, self.Hq, self.Kl = device, bs, H, Hq, Kl
        al = lambda n: (n + 255) // 256 * 256
        self.gather1_off = 0
        self.gather2_off = al(self.world * bs * H * Kl * 16)
        self.flags1_off = self.gather2_off + al(self.world * bs * Hq * 129 * 4)
        self.flags2_off = self.flags1_off + 256
        total = self.flags2_off + 256
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.local_base = ptrs[self.rank]
        self.peer_array = _lib.u64_array(ptrs)
        self.ctl = torch.zeros(8, dtype=torch.int32, device=device)    # two 16-byte control blocks, local
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)                                  # every rank's flags are zero before any store

    def check(self):
        """Raise if a bounded wait ran out (host synchronisation: call it outside the decode loop)."""
        st = self.ctl.cpu()
        if int(st[2]) or int(st[6]):
            raise RuntimeError("sequence-sharded exchange: a peer's data did not arrive within the wait limit")


class SequenceShardedCache:
    """Decode-side cache of the sequence-sharded form: this rank holds one contiguous chunk of every layer's
    zone (codes / 4-bit records / weights in HBM, K/V rows in HBM or pinned host memory) plus a full copy of the
    small GPU window; rank 0 attends the window.  It exposes the calls a decode loop makes on the single-GPU cache
    (`decode_update_kv_cache`, `compute`, `context`, and the hooks for replaying a captured step).

    Flush: when the update buffer fills, every rank drops the oldest `interval` window rows (the windows are
    replicas), the LAST rank codes them and appends them to its chunk — the zone grows at its end — and the
    histogram of the new codes is all-reduced into every rank's global cluster histogram."""

    def __init__(self, layer_num, num_kv_heads, num_heads, n_total, sink_size, local_size, interval, final_topk,
                 device, rank, world, group=None, collision_ratio=0.2, candidate_ratio=0.1, srht_sign_vector=None,
                 store="host", exchange="nccl", max_new_length=0):
        from .cache_hub.polar_cache import srht_signs
        self.layer_num, self.kv_head, self.num_heads = layer_num, num_kv_heads, num_heads
        self.sink_size, self.local_size, self.interval = sink_size, local_size, interval
        self.dynamic_update_interval = interval
        self.steady_size = sink_size + local_size
        self.final_topk, self.device, self.rank, self.world, self.group = final_topk, device, rank, world, group
        self.collision_ratio, self.candidate_ratio = collision_ratio, candidate_ratio
        self.start, end0 = sequence_shard(n_total, rank, world)
        self._n_total = [n_total] * layer_num               # zone keys per head, all ranks together
        self._n_local = [end0 - self.start] * layer_num     # zone keys per head held by this rank
        self.last = rank == world - 1
        # room for the keys that flushes append (they all go to the last rank)
        self.growth = ((max_new_length + interval - 1) // interval * interval + interval) if self.last else 0
        self.signs = (srht_sign_vector.to(device, torch.bfloat16).contiguous() if srht_sign_vector is not None
                      else srht_signs(device))
        self.centers = torch.tensor([0.0420, 0.1266, 0.2130, 0.3025, 0.3973, 0.5001, 0.6169, 0.7633],
                                    device=device, dtype=torch.bfloat16)
        cap = sink_size + local_size + interval
        self.window_capacity = cap
        self.window_k = [torch.zeros(1, num_kv_heads, cap, 128, dtype=torch.bfloat16, device=device) for _ in range(layer_num)]
        self.window_v = [torch.zeros(1, num_kv_heads, cap, 128, dtype=torch.bfloat16, device=device) for _ in range(layer_num)]
        self._window_len = [0] * layer_num
        self.meta = [None] * layer_num
        self.counts = [None] * layer_num
        self.store_kv = [None] * layer_num
        self._pinned = []                 # page-locked host tensors; their registrations end with this object
        from . import hostmem
        hostmem.release_on_collect(self, self._pinned)
        self.context = 0
        self.last_topk_indices = None
        if store not in ("host", "hbm", "auto"):
            raise ValueError("store must be 'host', 'hbm' or 'auto'")
        if store == "auto":   # keep the shard's K/V rows in HBM when they fit beside the codes, else pinned host memory
            need = layer_num * num_kv_heads * (self._n_local[0] + self.growth) * (512 + 112)
            free, _ = torch.cuda.mem_get_info(device)
            store = "hbm" if need + (16 << 30) < free else "host"
        self.store = store
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.px, self.hist_gather = None, None
        if exchange == "peer" and world > 1:   # the two larger per-layer exchanges as stores into peer memory
            _, _, k_final = global_plan(n_total, collision_ratio, candidate_ratio, final_topk)
            self.px = PeerExchange(1, num_kv_heads, num_heads, k_final, device, group)
            # the count histograms ([H,256] i32 per rank) travel through the short-row gather kernel as raw words
            self.hist_gather = TPReducer(num_kv_heads * 512, device, group, mode="peer")
        self.device_positions = False     # window length read from a device word (captured steps)
        self._dev_state = torch.zeros(1, dtype=torch.int32, device=device)
        # scratch of the chain and of the attention kernel, sized once for everything this shard can grow to: the
        # addresses stay fixed, so captured decode steps remain valid
        from . import ops
        n_cap = max(self._n_local[0] + self.growth, 1)
        n_all = n_total + ((max_new_length + interval - 1) // interval * interval + interval)
        c_cap = min(n_cap, max(1, int(math.ceil(n_all * candidate_ratio))))
        self._retrieve_scratch = ops.Scratch(device, ops.retrieve_scratch_bytes(1, num_kv_heads, n_cap, c_cap))
        self._attn_scratch = ops.Scratch(device, ops.attention_scratch_bytes(1, num_heads, cap + final_topk))

    # the names the single-GPU cache uses for the same quantities
    @property
    def n_total(self):
        return self._n_total[0]

    @property
    def cpu_valid_end(self):
        return self._n_total

    @property
    def end(self):
        return self.start + self._n_local[0]

    def load_layer(self, layer, shard_keys, shard_values, window_keys, window_values):
        """shard_keys / shard_values: bf16 [1,H,n_local,128] on the device (this rank's chunk of the zone);
        window_*: bf16 [1,H,sink+local,128] (sink rows then the last `local` rows of the prompt)."""
        from . import ops
        n_local = shard_keys.shape[2]
        assert n_local == self._n_local[layer], "shard length differs from sequence_shard()"
        cap = max(n_local + self.growth, 1)
        cb, w, pk = ops.alloc_key_metadata(1, self.kv_head, cap, self.device)
        counts = torch.zeros(1, self.kv_head, 16, 256, dtype=torch.int32, device=self.device)
        ops.encode_keys(shard_keys, self.signs, cb[:, :, :, :n_local], w[:, :, :, :n_local], pk[:, :, :, :n_local, :],
                        cluster_counts=counts)
        self.meta[layer] = (cb, w, pk)
        self.counts[layer] = allreduce_cluster_counts(counts, self.group)
        # K and V row of a key next to each other: one host address translation per selected key instead of two
        kv = torch.stack((shard_keys, shard_values), dim=3)          # [1,H,n,2,128] on the device
        if self.store == "hbm":
            skv = torch.empty(1, self.kv_head, cap, 2, 128, dtype=torch.bfloat16, device=self.device)
        else:
            from . import hostmem   # page-locked without the pinned allocator's power-of-two rounding
            skv = hostmem.pinned_empty(1, self.kv_head, cap, 2, 128, dtype=torch.bfloat16)
            self._pinned.append(skv)
        skv[:, :, :n_local].copy_(kv, non_blocking=True)
        self.store_kv[layer] = skv
        n = window_keys.shape[2]
        self.window_k[layer][:, :, :n] = window_keys
        self.window_v[layer][:, :, :n] = window_values
        self._window_len[layer] = n
        if layer == self.layer_num - 1:
            self.context = self.sink_size + self._n_total[layer] + self.local_size

    def decode_update_kv_cache(self, key_states, value_states, layer_idx):
        from . import ops
        pos = self._window_len[layer_idx]
        ops.append_kv(key_states, value_states, self.window_k[layer_idx], self.window_v[layer_idx], pos,
                      self._dev_state[0:1] if self.device_positions else None, 0)
        self._window_len[layer_idx] = pos + 1
        if layer_idx == 0:
            self.context += 1
        if self._window_len[layer_idx] == self.window_capacity:
            self._flush(layer_idx)
        return None, None

    def _flush(self, layer):
        """Move the oldest `interval` rows behind the sink out of the window and into the zone (last rank's chunk)."""
        from . import ops
        if self.device_positions:
            raise RuntimeError("a flush cannot be part of a captured step: run the step that flushes eagerly")
        I, sink, local = self.interval, self.sink_size, self.local_size
        wk, wv = self.window_k[layer], self.window_v[layer]
        delta = torch.zeros(1, self.kv_head, 16, 256, dtype=torch.int32, device=self.device)
        if self.last:
            n = self._n_local[layer]
            cb, w, pk = self.meta[layer]
            if n + I > cb.shape[3]:
                raise RuntimeError("zone capacity exhausted: construct the cache with a larger max_new_length")
            zk, zv = wk[:, :, sink:sink + I], wv[:, :, sink:sink + I]
            ops.encode_keys(zk, self.signs, cb[:, :, :, n:n + I], w[:, :, :, n:n + I], pk[:, :, :, n:n + I, :],
                            cluster_counts=delta)
            self.store_kv[layer][:, :, n:n + I].copy_(torch.stack((zk, zv), dim=3), non_blocking=True)
            self._n_local[layer] = n + I
        self.counts[layer] += allreduce_cluster_counts(delta, self.group)
        self._n_total[layer] += I
        wk[:, :, sink:sink + local] = wk[:, :, sink + I:sink + I + local].clone()
        wv[:, :, sink:sink + local] = wv[:, :, sink + I:sink + I + local].clone()
        self._window_len[layer] = sink + local

    def compute(self, queries, layer_idx):
        cb, w, pk = self.meta[layer_idx]
        n = self._n_local[layer_idx]
        skv = self.store_kv[layer_idx]
        first = self.rank == 0
        out, final = sequence_sharded_attend(
            queries.contiguous(), self.signs, self.centers, cb[:, :, :, :n], w[:, :, :, :n], pk[:, :, :, :n, :],
            self.counts[layer_idx], skv[:, :, :, 0], skv[:, :, :, 1], self._n_total[layer_idx], self.start,
            self.start + n, self.collision_ratio, self.candidate_ratio,
            self.final_topk, window_k=self.window_k[layer_idx] if first else None,
            window_v=self.window_v[layer_idx] if first else None,
            n_window=(self.window_capacity if self.device_positions else self._window_len[layer_idx]) if first else 0,
            group=self.group, n_window_dev=self._dev_state[0:1] if (first and self.device_positions) else None,
            n_window_add=1 if (first and self.device_positions) else 0, exchange=self.px,
            scratch=self._retrieve_scratch, attn_scratch=self._attn_scratch, hist_gather=self.hist_gather)
        self.last_topk_indices = final
        return out

    # ---- support for replaying a captured decode step (same calls as the single-GPU cache) ----
    def next_step_flushes(self) -> bool:
        return self._window_len[0] + 1 >= self.window_capacity

    def sync_device_state(self):
        self._dev_state[0] = self._window_len[0]

    def advance_device_step(self):
        self._dev_state[0:1] += 1

    def host_state(self):
        return (list(self._window_len), list(self._n_local), self.context, list(self._n_total))

    def set_host_state(self, st):
        self._window_len, self._n_local, self.context, self._n_total = list(st[0]), list(st[1]), st[2], list(st[3])

    def host_state_after_flushes(self, j):
        """The host state right after the j-th flush from now (None when the zone cannot grow that far)."""
        add = j * self.interval
        n_local = [n + (add if self.last else 0) for n in self._n_local]
        if self.last and self.meta[0] is not None and n_local[0] > self.meta[0][0].shape[3]:
            return None
        return ([self.steady_size] * self.layer_num, n_local, self.context, [n + add for n in self._n_total])

    def note_replayed_step(self):
        self._window_len = [n + 1 for n in self._window_len]
        self.context += 1
