"""Python entry points of the CUDA ops: thin wrappers that validate, allocate outputs and scratch with
torch, and call the C ABI on torch's current stream.  No op has a CPU or PyTorch fallback.

Storage convention: tensors are passed in the reference's LOGICAL shapes (codebook ``[bs,H,16,N]``,
block weights ``[bs,H,16,N]``, packed 4-bit ``[bs,H,16,N,4]``) with any strides.  Outputs allocated
here are key-major in memory (``[bs,H,N,16(,4)]``) and returned as permuted views with those shapes;
that layout turns a rerank candidate into one 64-byte plus one 32-byte record.
"""
import ctypes
import math

import torch

from . import _lib as L

_WS = {}


def workspace(device, nbytes, tag="default"):
    """A cached scratch buffer per (device, tag) for eager calls that do not bring their own.  It grows by
    replacement, so it must not grow while a CUDA graph is being captured (a graph captured earlier would keep
    the address of the buffer that was dropped): callers that capture pass a Scratch they own instead."""
    key = (torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device(), tag)
    buf = _WS.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"the shared '{tag}' scratch buffer would have to grow to {int(nbytes)} bytes during a "
                               "stream capture; give the op a Scratch sized before the capture")
        # zero-filled: the attention kernel keeps arrival counters in its workspace header
        buf = torch.zeros(max(int(nbytes), 1 << 16), dtype=torch.uint8, device=device)
        _WS[key] = buf
    return buf


class Scratch:
    """A fixed scratch buffer that its owner sizes once (for the largest problem it will run) and passes to every
    call: its address never changes, so launches captured in a CUDA graph stay valid for the owner's lifetime.
    Zero-filled at allocation (the attention kernel's arrival counters live in its header)."""

    def __init__(self, device, nbytes):
        self.buf = torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)

    def take(self, nbytes, what):
        if self.buf.numel() < nbytes:
            raise RuntimeError(f"{what}: the owned scratch buffer holds {self.buf.numel()} bytes, {int(nbytes)} needed")
        return self.buf


def _scratch(device, nbytes, tag, scratch):
    return scratch.take(nbytes, tag) if scratch is not None else workspace(device, nbytes, tag)


def retrieve_scratch_bytes(bs, H, N, C):
    return int(L.load().pk_retrieve_workspace_bytes(int(bs), int(H), int(N), int(C)))


def attention_scratch_bytes(bs, Hq, max_rows):
    return int(L.load().pk_attention_workspace_bytes(int(bs), int(Hq), int(max_rows)))


def attention_status(scratch_or_buf, bs, Hq):
    """The status word of an attention scratch buffer (a host synchronisation: call it outside the decode loop).
    Non-zero means that a block gave up waiting for its row copies; the results since then are invalid."""
    buf = scratch_or_buf.buf if isinstance(scratch_or_buf, Scratch) else scratch_or_buf
    return int(buf[: (bs * Hq + 1) * 4].view(torch.int32)[bs * Hq].item())


def check_attention_status(scratch_or_buf, bs, Hq):
    if attention_status(scratch_or_buf, bs, Hq) != 0:
        raise RuntimeError("sparse attention: a block gave up waiting for its K/V row copies (status word set); "
                           "the attention outputs since then are invalid")


def _call(name, *args):
    L.check(getattr(L.load(), name)(*args))


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("pariskv_b200 ops need CUDA tensors; there is no CPU fallback")


# --------------------------------------------------------------------------------------------------
# key coding
# --------------------------------------------------------------------------------------------------
def alloc_key_metadata(bs, H, cap, device):
    """Key-major metadata storage for `cap` keys per head, returned as reference-shaped views:
    (codebook u8 [bs,H,16,cap], block_weight bf16 [bs,H,16,cap], packed u8 [bs,H,16,cap,4])."""
    cb = torch.zeros(bs, H, cap, 16, dtype=torch.uint8, device=device)
    w = torch.zeros(bs, H, cap, 16, dtype=torch.bfloat16, device=device)
    pk = torch.zeros(bs, H, cap, 16, 4, dtype=torch.uint8, device=device)
    return cb.permute(0, 1, 3, 2), w.permute(0, 1, 3, 2), pk.permute(0, 1, 3, 2, 4)


def encode_keys(keys, signs, codebook=None, block_weight=None, packed_4bit=None, cluster_counts=None):
    """keys bf16 [bs,H,L,128] -> (codebook, block_weight, packed_4bit); see pk_encode_keys.
    When `cluster_counts` (i32 [bs,H,16,256]) is given, the code histogram of these keys is ADDED to it."""
    _require_cuda(keys, signs)
    bs, H, Lk, D = keys.shape
    if codebook is None:
        codebook, block_weight, packed_4bit = alloc_key_metadata(bs, H, Lk, keys.device)
    if keys.numel() == 0:
        return codebook, block_weight, packed_4bit
    d = [L.desc(t) for t in (keys, signs, codebook, block_weight, packed_4bit, cluster_counts)]
    _call("pk_encode_keys", *[L.ref(x) for x in d], L.stream_ptr(keys.device))
    return codebook, block_weight, packed_4bit


def count_clusters(codebook, counts=None, accumulate=False):
    _require_cuda(codebook)
    bs, H, B, N = codebook.shape
    if counts is None:
        counts = torch.empty(bs, H, B, 256, dtype=torch.int32, device=codebook.device)
        accumulate = False
    dc, dn = L.desc(codebook), L.desc(counts)
    _call("pk_count_clusters", L.ref(dc), L.ref(dn), int(bool(accumulate)), L.stream_ptr(codebook.device))
    return counts


def query_prep(queries, kv_heads, signs, want_avg=False):
    """queries bf16 [bs,1,Hq,128] -> q_blocks [bs,H,16,8], q_norm [bs,H,1] (, query_avg [bs,H,128])."""
    _require_cuda(queries, signs)
    bs = queries.shape[0]
    dev = queries.device
    qb = torch.empty(bs, kv_heads, 16, 8, dtype=torch.bfloat16, device=dev)
    qn = torch.empty(bs, kv_heads, 1, dtype=torch.bfloat16, device=dev)
    qa = torch.empty(bs, kv_heads, 128, dtype=torch.bfloat16, device=dev) if want_avg else None
    d = [L.desc(t) for t in (queries, signs, qb, qn, qa)]
    _call("pk_query_prep", *[L.ref(x) for x in d], L.stream_ptr(dev))
    return (qb, qn, qa) if want_avg else (qb, qn)


def rank_clusters(q_blocks):
    _require_cuda(q_blocks)
    bs, H = q_blocks.shape[:2]
    ids = torch.empty(bs, H, 16, 256, dtype=torch.int64, device=q_blocks.device)
    dq, di = L.desc(q_blocks), L.desc(ids)
    _call("pk_rank_clusters", L.ref(dq), L.ref(di), L.stream_ptr(q_blocks.device))
    return ids


# --------------------------------------------------------------------------------------------------
# collision
# --------------------------------------------------------------------------------------------------
def collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts, cache_cnt=None):
    _require_cuda(sorted_cluster_ids, cluster_key_counts, codebook)
    bs, H, B, N = codebook.shape
    dev = codebook.device
    if cache_cnt is None:
        cache_cnt = torch.empty(bs, H, N, dtype=torch.int32, device=dev)
    lib = L.load()
    nb = lib.pk_collision_workspace_bytes(bs, H, B, sorted_cluster_ids.shape[-1])
    ws = workspace(dev, nb, "collision")
    tiers = L.i64_array(list(tier_counts))
    d = [L.desc(t) for t in (sorted_cluster_ids, cluster_key_counts, codebook, cache_cnt)]
    _call("pk_collision_fused", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), tiers, len(tier_counts), L.ref(d[3]),
          ws.data_ptr(), ws.numel(), L.stream_ptr(dev))
    return cache_cnt


def collision_fused_static(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts, cache_cnt):
    """collision_fused for callers that must not allocate: the caller passes the output tensor, the tier table
    lives in a fixed 256 KB array inside the library (at most 1024 batch x head x subspace triples).  Calls
    share that array, so do not let two of them overlap on the GPU; make the first call on a device before any
    stream capture."""
    _require_cuda(sorted_cluster_ids, cluster_key_counts, codebook, cache_cnt)
    tiers = L.i64_array(list(tier_counts))
    d = [L.desc(t) for t in (sorted_cluster_ids, cluster_key_counts, codebook, cache_cnt)]
    _call("pk_collision_fused_static", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), tiers, len(tier_counts), L.ref(d[3]),
          L.stream_ptr(codebook.device))
    return cache_cnt


def collision(sorted_cluster_ids, topk_cluster_cnt, code_book, cache_cnt):
    """Unfused single-tier op; code_book is int32 [bs,H,N,B] (the kernel-side layout)."""
    _require_cuda(sorted_cluster_ids, topk_cluster_cnt, code_book, cache_cnt)
    bs, H, N, B = code_book.shape
    dev = code_book.device
    nb = L.load().pk_collision_workspace_bytes(bs, H, B, sorted_cluster_ids.shape[-1])
    ws = workspace(dev, nb, "collision")
    d = [L.desc(t) for t in (sorted_cluster_ids, topk_cluster_cnt, code_book, cache_cnt)]
    _call("pk_collision", *[L.ref(x) for x in d], ws.data_ptr(), ws.numel(), L.stream_ptr(dev))
    return cache_cnt


# --------------------------------------------------------------------------------------------------
# top-k
# --------------------------------------------------------------------------------------------------
def topk(x, k, order=0):
    """Exact top-k indices over the last dim of a 2-D or 3-D int32/float32 tensor -> int64.
    order 0: ascending index; order 1: value descending.  Ties go to the lower index."""
    _require_cuda(x)
    if x.dtype not in (torch.int32, torch.float32):
        x = x.to(torch.int32) if not x.dtype.is_floating_point else x.to(torch.float32)
    if x.stride(-1) != 1:
        x = x.contiguous()
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    out = torch.empty(x2.shape[0], k, dtype=torch.int64, device=x.device)
    dx, do = L.desc(x2), L.desc(out)
    _call("pk_topk", L.ref(dx), int(k), L.ref(do), int(order), L.stream_ptr(x.device))
    return out.view(*lead, k)


def final_topk(scores_f32, cand, K):
    _require_cuda(scores_f32, cand)
    bs, H, C = scores_f32.shape
    out = torch.empty(bs, H, K, dtype=torch.int64, device=scores_f32.device)
    d = [L.desc(t) for t in (scores_f32, cand, out)]
    _call("pk_final_topk", L.ref(d[0]), L.ref(d[1]), int(K), L.ref(d[2]), L.stream_ptr(scores_f32.device))
    return out


def adaptive_topk(sl_logits, cand_scores, cand_scale, sl_vnorm, cand_indices, cand_vnorm, threshold, K_out,
                  value_norm=None, sink_size=0, min_k=0, max_k=0, adaptive_k=None, topk_indices=None):
    _require_cuda(sl_logits, cand_scores, sl_vnorm, cand_indices)
    bs, H = sl_logits.shape[:2]
    dev = sl_logits.device
    if adaptive_k is None:
        adaptive_k = torch.empty(bs, H, dtype=torch.int64, device=dev)
    if topk_indices is None:
        topk_indices = torch.empty(bs, H, K_out, dtype=torch.int64, device=dev)
    d = [L.desc(t) for t in (sl_logits, cand_scores, sl_vnorm, cand_indices, cand_vnorm, value_norm, adaptive_k,
                             topk_indices)]
    _call("pk_adaptive_topk", L.ref(d[0]), L.ref(d[1]), float(cand_scale), L.ref(d[2]), L.ref(d[3]), L.ref(d[4]),
          L.ref(d[5]), int(sink_size), float(threshold), int(K_out), int(min_k), int(max_k), L.ref(d[6]),
          L.ref(d[7]), L.stream_ptr(dev))
    return adaptive_k, topk_indices


# --------------------------------------------------------------------------------------------------
# rerank
# --------------------------------------------------------------------------------------------------
def rerank(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers, approx_scores=None,
           scores_f32=None, v4b=None, want_f32=False):
    _require_cuda(coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers)
    bs, H, C = coarse_indices.shape
    dev = coarse_indices.device
    if approx_scores is None:
        approx_scores = torch.empty(bs, H, C, dtype=torch.bfloat16, device=dev)
    if scores_f32 is None and want_f32:
        scores_f32 = torch.empty(bs, H, C, dtype=torch.float32, device=dev)
    d = [L.desc(t) for t in (coarse_indices, key_4bit, key_block_weight, q_blocks, q_norm, mag_centers,
                             approx_scores, scores_f32, v4b)]
    _call("pk_rerank", *[L.ref(x) for x in d], L.stream_ptr(dev))
    return approx_scores, scores_f32


# --------------------------------------------------------------------------------------------------
# gather / attention
# --------------------------------------------------------------------------------------------------
def h2d_gather_kv(src_k, src_v, selected_indices, dst_k, dst_v):
    _require_cuda(selected_indices, dst_k, dst_v)
    d = [L.desc(t) for t in (src_k, src_v, selected_indices, dst_k, dst_v)]
    _call("pk_h2d_gather_kv", *[L.ref(x) for x in d], L.stream_ptr(dst_k.device))


def h2d_gather_kv_packed(src_k, src_v, k_packed, v_packed, indices_packed, cu_seqlens_topk, cu_seqlens_k,
                         sink_local_end, global_k):
    _require_cuda(k_packed, v_packed, indices_packed, cu_seqlens_topk, cu_seqlens_k)
    d = [L.desc(t) for t in (src_k, src_v, k_packed, v_packed, indices_packed, cu_seqlens_topk, cu_seqlens_k)]
    _call("pk_h2d_gather_kv_packed", *[L.ref(x) for x in d], int(sink_local_end), int(global_k),
          L.stream_ptr(k_packed.device))


def gather_kv_out_cpu(src, index, out, n_threads=0):
    for t in (src, index, out):
        if t.is_cuda:
            raise RuntimeError("gather_kv_out_cpu works on host tensors")
    d = [L.desc(t) for t in (src, index, out)]
    _call("pk_gather_kv_out_cpu", *[L.ref(x) for x in d], int(n_threads))


def append_kv(k_row, v_row, window_k, window_v, pos, pos_dev=None, pos_add=0):
    """Write the step's K/V row ([bs,1,H,128]) into window row `pos` (or pos_dev[0] + pos_add, read on device)."""
    _require_cuda(k_row, v_row, window_k, window_v)
    d = [L.desc(t) for t in (k_row, v_row, window_k, window_v, pos_dev)]
    _call("pk_append_kv", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), L.ref(d[3]), int(pos), L.ref(d[4]), int(pos_add),
          L.stream_ptr(window_k.device))


def append_encode(k_row, v_row, signs, window_k, window_v, win_codes, win_weight, win_4bit, win_vnorm, codebook,
                  block_weight, packed_4bit, value_norm, cluster_counts, store_kv, state, sink, interval):
    """One decode token into the cache: window row, key coding, and the flush of a full update buffer, all positions
    read from the device-side `state` words; see pk_append_encode."""
    _require_cuda(k_row, v_row, window_k, window_v, state)
    d = [L.desc(t) for t in (k_row, v_row, signs, window_k, window_v, win_codes, win_weight, win_4bit, win_vnorm, codebook,
                             block_weight, packed_4bit, value_norm, cluster_counts, store_kv, state)]
    _call("pk_append_encode", *[L.ref(x) for x in d], int(sink), int(interval), L.stream_ptr(window_k.device))


def sparse_attention(queries, window_k, window_v, n_window, store_k=None, store_v=None, selected=None, n_sel=None,
                     index_offset=0, scale=None, out=None, n_window_dev=None, n_window_add=0, lse=None, scratch=None):
    """Decode attention over window rows [0, n_window) plus the selected rows of the K/V store (device or
    pinned host memory); see pk_sparse_attention."""
    _require_cuda(queries, window_k, window_v, selected)
    bs, _, Hq, D = queries.shape
    dev = queries.device
    if out is None:
        out = torch.empty_like(queries)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    K = selected.shape[2] if selected is not None else 0
    nb = L.load().pk_attention_workspace_bytes(bs, Hq, n_window + K)
    ws = _scratch(dev, nb, "attention", scratch)
    d = [L.desc(t) for t in (queries, window_k, window_v, store_k, store_v, selected, n_sel, out, n_window_dev, lse)]
    _call("pk_sparse_attention", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), int(n_window), L.ref(d[8]), int(n_window_add),
          L.ref(d[3]), L.ref(d[4]), L.ref(d[5]), L.ref(d[6]), int(index_offset), float(scale), L.ref(d[7]), L.ref(d[9]),
          ws.data_ptr(), ws.numel(), L.stream_ptr(dev))
    return out


# --------------------------------------------------------------------------------------------------
# the fused retrieval chain
# --------------------------------------------------------------------------------------------------
def retrieve(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, cluster_key_counts, tier_counts,
             C, K, final_indices=None, want=(), scratch=None):
    """queries -> final top-K key indices (ascending) in one call.  `want` may name extra outputs among
    {"cand", "scores_f32", "q_blocks", "q_norm", "query_avg"}; returns (final_indices, extras dict)."""
    _require_cuda(queries, codebook, key_block_weight, key_4bit, cluster_key_counts)
    bs, H, B, N = codebook.shape
    dev = codebook.device
    if final_indices is None and K > 0:
        final_indices = torch.empty(bs, H, K, dtype=torch.int64, device=dev)
    extras = {}
    if "cand" in want:
        extras["cand"] = torch.empty(bs, H, C, dtype=torch.int64, device=dev)
    if "scores_f32" in want:
        extras["scores_f32"] = torch.empty(bs, H, C, dtype=torch.float32, device=dev)
    if "q_blocks" in want:
        extras["q_blocks"] = torch.empty(bs, H, 16, 8, dtype=torch.bfloat16, device=dev)
    if "q_norm" in want:
        extras["q_norm"] = torch.empty(bs, H, 1, dtype=torch.bfloat16, device=dev)
    if "query_avg" in want:
        extras["query_avg"] = torch.empty(bs, H, 128, dtype=torch.bfloat16, device=dev)
    nb = L.load().pk_retrieve_workspace_bytes(bs, H, N, C)
    ws = _scratch(dev, nb, "retrieve", scratch)
    tiers = L.i64_array(list(tier_counts))
    d = [L.desc(t) for t in (queries, signs, mag_centers, codebook, key_block_weight, key_4bit, cluster_key_counts,
                             final_indices, extras.get("cand"), extras.get("scores_f32"), extras.get("q_blocks"),
                             extras.get("q_norm"), extras.get("query_avg"))]
    _call("pk_retrieve", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), L.ref(d[3]), L.ref(d[4]), L.ref(d[5]), L.ref(d[6]),
          tiers, len(tier_counts), int(C), int(K), L.ref(d[7]), L.ref(d[8]), L.ref(d[9]), L.ref(d[10]),
          L.ref(d[11]), L.ref(d[12]), ws.data_ptr(), ws.numel(), L.stream_ptr(dev))
    return final_indices, extras


def retrieve_ex(queries, signs, mag_centers, codebook, key_block_weight, key_4bit, cluster_key_counts, C, K,
                tier_counts=None, kv_len=None, schedule=None, phase=0, local_hist=None, shard_hist=None, world=1,
                rank=0, final_indices=None, n_sel=None, n_cand=None, want=(), outputs=None, scratch=None,
                queries_settled=False):
    """The retrieval chain with per-sample zone lengths read on the device (`kv_len` i32 [bs] + `schedule`, a
    _lib.zone_schedule) or in its two-phase form for a zone sharded over ranks (phase 1 -> local_hist; phase 2 with
    the all-gathered shard_hist); see pk_retrieve_ex.  `outputs` may hold preallocated tensors for the names in
    `want` (reused between the two phases).  queries_settled: the queries were complete before the launch just before
    this call started (see pk_retrieve_args).  Returns (final_indices, n_sel, extras dict)."""
    _require_cuda(queries, codebook, key_block_weight, key_4bit, cluster_key_counts)
    bs, H, B, N = codebook.shape
    dev = codebook.device
    row = min(int(C), N) if phase else int(C)
    extras = dict(outputs or {})
    shapes = {"cand": ((bs, H, row), torch.int64), "scores_f32": ((bs, H, row), torch.float32),
              "q_blocks": ((bs, H, 16, 8), torch.bfloat16), "q_norm": ((bs, H, 1), torch.bfloat16),
              "query_avg": ((bs, H, 128), torch.bfloat16)}
    for name in want:
        if name not in extras:
            shape, dt = shapes[name]
            extras[name] = torch.empty(*shape, dtype=dt, device=dev)
    if phase != 1:
        if final_indices is None and K > 0:
            final_indices = torch.empty(bs, H, K, dtype=torch.int64, device=dev)
        if n_sel is None and K > 0:
            n_sel = torch.empty(bs, H, dtype=torch.int32, device=dev)
        if n_cand is None:
            n_cand = torch.empty(bs, H, dtype=torch.int32, device=dev)
    if phase == 1 and local_hist is None:
        local_hist = torch.empty(bs, H, 256, dtype=torch.int32, device=dev)
    nb = retrieve_scratch_bytes(bs, H, N, row)
    ws = _scratch(dev, nb, "retrieve", scratch)
    a = L.PkRetrieveArgs()
    keep = []

    def put(field, t):
        if t is not None:
            d = L.desc(t)
            keep.append(d)
            setattr(a, field, L.ptr(d))

    for field, t in (("queries", queries), ("signs", signs), ("mag_centers", mag_centers), ("codebook", codebook),
                     ("key_block_weight", key_block_weight), ("key_4bit", key_4bit),
                     ("cluster_key_counts", cluster_key_counts), ("kv_len", kv_len), ("local_hist", local_hist),
                     ("shard_hist", shard_hist), ("final_indices", final_indices), ("n_sel", n_sel),
                     ("cand", extras.get("cand")), ("n_cand", n_cand), ("scores_f32", extras.get("scores_f32")),
                     ("q_blocks", extras.get("q_blocks")), ("q_norm", extras.get("q_norm")),
                     ("query_avg", extras.get("query_avg"))):
        put(field, t)
    if tier_counts is not None:
        tiers = L.i64_array(list(tier_counts))
        a.tier_counts, a.n_tiers = tiers, len(tier_counts)
    if schedule is not None:
        a.schedule = ctypes.pointer(schedule)
    a.phase, a.C, a.K, a.world, a.rank = int(phase), int(C), int(K), int(world), int(rank)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.queries_settled = 1 if queries_settled else 0
    _call("pk_retrieve_ex", ctypes.byref(a), L.stream_ptr(dev))
    extras["n_cand"] = n_cand
    extras["local_hist"] = local_hist
    return final_indices, n_sel, extras


# --------------------------------------------------------------------------------------------------
# sequence-sharded form: packing / unpacking around the two all-gathers
# --------------------------------------------------------------------------------------------------
def shard_pack_topk(cand, scores, local_final, start, packed=None, n_sel=None, n_cand=None):
    """(cand, scores, local_final) -> packed i64 [bs,H,Kl,2]; n_sel / n_cand (i32 [bs,H]) give the valid entries of
    local_final / cand rows; see pk_shard_pack_topk."""
    _require_cuda(cand, scores, local_final)
    bs, H, Kl = local_final.shape
    if packed is None:
        packed = torch.empty(bs, H, Kl, 2, dtype=torch.int64, device=cand.device)
    d = [L.desc(t) for t in (cand, scores, local_final, n_sel, n_cand, packed)]
    _call("pk_shard_pack_topk", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), int(start), L.ref(d[3]), L.ref(d[4]), L.ref(d[5]),
          L.stream_ptr(cand.device))
    return packed


def shard_unpack_topk(gathered):
    """gathered i64 [world,bs,H,Kl,2] -> (scores f32, indices i64) [bs,H,world*Kl]; see pk_shard_unpack_topk."""
    _require_cuda(gathered)
    world, bs, H, Kl, _ = gathered.shape
    scores = torch.empty(bs, H, world * Kl, dtype=torch.float32, device=gathered.device)
    indices = torch.empty(bs, H, world * Kl, dtype=torch.int64, device=gathered.device)
    d = [L.desc(t) for t in (gathered, scores, indices)]
    _call("pk_shard_unpack_topk", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), L.stream_ptr(gathered.device))
    return scores, indices


def shard_owned_rows(final_indices, start, end):
    """final i64 [bs,H,K] -> (local i64 [bs,H,K], n_owned i32 [bs,H]); see pk_shard_owned_rows."""
    _require_cuda(final_indices)
    bs, H, K = final_indices.shape
    local = torch.empty_like(final_indices)
    n_owned = torch.empty(bs, H, dtype=torch.int32, device=final_indices.device)
    d = [L.desc(t) for t in (final_indices, local, n_owned)]
    _call("pk_shard_owned_rows", L.ref(d[0]), int(start), int(end), L.ref(d[1]), L.ref(d[2]),
          L.stream_ptr(final_indices.device))
    return local, n_owned


def shard_pack_partial(out, lse):
    """(out bf16 [bs,1,Hq,128], lse f32 [bs,Hq]) -> packed f32 [bs,Hq,129]; see pk_shard_pack_partial."""
    _require_cuda(out, lse)
    bs, _, Hq, _ = out.shape
    packed = torch.empty(bs, Hq, 129, dtype=torch.float32, device=out.device)
    d = [L.desc(t) for t in (out, lse, packed)]
    _call("pk_shard_pack_partial", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), L.stream_ptr(out.device))
    return packed


def shard_merge_partial(gathered):
    """gathered f32 [world,bs,Hq,129] -> out bf16 [bs,1,Hq,128]; see pk_shard_merge_partial."""
    _require_cuda(gathered)
    world, bs, Hq, _ = gathered.shape
    out = torch.empty(bs, 1, Hq, 128, dtype=torch.bfloat16, device=gathered.device)
    d = [L.desc(t) for t in (gathered, out)]
    _call("pk_shard_merge_partial", L.ref(d[0]), L.ref(d[1]), L.stream_ptr(gathered.device))
    return out


def shard_exchange_topk(cand, scores, local_final, start, px, n_sel=None, n_cand=None):
    """Pack this rank's local top list and store it into every peer's gather area; see pk_shard_exchange_topk.
    px: a dist.PeerExchange."""
    _require_cuda(cand, scores, local_final)
    d = [L.desc(t) for t in (cand, scores, local_final, n_sel, n_cand)]
    _call("pk_shard_exchange_topk", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), int(start), L.ref(d[3]), L.ref(d[4]),
          px.peer_array, px.world, px.rank, px.gather1_off, px.flags1_off, px.ctl.data_ptr(), L.stream_ptr(cand.device))


def shard_collect_topk(px, bs, H, Kl):
    """Wait for every rank's local top list, then unpack; see pk_shard_collect_topk."""
    scores = torch.empty(bs, H, px.world * Kl, dtype=torch.float32, device=px.device)
    indices = torch.empty(bs, H, px.world * Kl, dtype=torch.int64, device=px.device)
    d = [L.desc(t) for t in (scores, indices)]
    _call("pk_shard_collect_topk", px.local_base, px.gather1_off, px.flags1_off, px.ctl.data_ptr(), px.world, int(Kl),
          L.ref(d[0]), L.ref(d[1]), L.stream_ptr(px.device))
    return scores, indices


def shard_exchange_partial(out, lse, px):
    """Store this rank's partial attention result into every peer's gather area; see pk_shard_exchange_partial."""
    _require_cuda(out, lse)
    d = [L.desc(t) for t in (out, lse)]
    _call("pk_shard_exchange_partial", L.ref(d[0]), L.ref(d[1]), px.peer_array, px.world, px.rank, px.gather2_off,
          px.flags2_off, px.ctl.data_ptr() + 16, L.stream_ptr(out.device))


def shard_collect_partial(px, bs, Hq):
    """Wait for every rank's partial result, then merge; see pk_shard_collect_partial."""
    out = torch.empty(bs, 1, Hq, 128, dtype=torch.bfloat16, device=px.device)
    d = L.desc(out)
    _call("pk_shard_collect_partial", px.local_base, px.gather2_off, px.flags2_off, px.ctl.data_ptr() + 16, px.world,
          L.ref(d), L.stream_ptr(px.device))
    return out


def tp_allreduce(partial, residual, px, out=None, norm_weight=None, eps=1e-6):
    """out = residual + sum over ranks of partial, one launch over peer memory; px: a dist.TPReducer in peer mode.
    With norm_weight (bf16 [n]) the same launch also writes RMS-norm(out) * norm_weight and (out, normed) is
    returned.  See pk_tp_allreduce."""
    _require_cuda(partial, residual)
    if out is None:
        out = torch.empty_like(partial)
    d = [L.desc(t) for t in (partial, residual, out)]
    normed = torch.empty_like(partial) if norm_weight is not None else None
    dn = [L.desc(t) for t in (norm_weight, normed)] if norm_weight is not None else None
    _call("pk_tp_allreduce", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), px.peer_array, px.world, px.rank, 0, px.area_bytes,
          px.flags_off, px.ctl.data_ptr(), L.ref(dn[0]) if dn else None, L.ref(dn[1]) if dn else None, float(eps),
          L.stream_ptr(partial.device))
    return out if norm_weight is None else (out, normed)


def tp_allgather(part, px, out=None):
    """out [1, world*n] = every rank's part [1, n] in rank order, one launch over peer memory; px: a dist.TPReducer
    in peer mode.  See pk_tp_allgather."""
    _require_cuda(part)
    if out is None:
        out = torch.empty(1, px.world * part.numel(), dtype=torch.bfloat16, device=part.device)
    d = [L.desc(part), L.desc(out)]
    _call("pk_tp_allgather", L.ref(d[0]), L.ref(d[1]), px.peer_array, px.world, px.rank, 0, px.area_bytes, px.flags_off,
          px.ctl.data_ptr(), L.stream_ptr(part.device))
    return out


def qk_norm_rope(qkv, weight, cos, sin, eps=1e-6, out=None):
    """Per-head RMS-norm and rotate-half RoPE of the q and k heads of a fused q/k/v row in one launch.
    qkv bf16 [B, >= heads*128]; weight bf16 [heads,128]; cos / sin bf16 [1 or B,128] (sin = [-sin, sin]).
    Returns bf16 [B, heads, 128].  See pk_qk_norm_rope."""
    _require_cuda(qkv, weight, cos, sin)
    B, heads = qkv.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty(B, heads, 128, dtype=torch.bfloat16, device=qkv.device)
    d = [L.desc(t) for t in (qkv, weight, cos, sin, out)]
    _call("pk_qk_norm_rope", *[L.ref(x) for x in d], float(eps), L.stream_ptr(qkv.device))
    return out


def add_rmsnorm(a, residual, weight, eps=1e-6):
    """h = a + residual (residual may be None), x = RMS-norm(h) * weight, one launch.  Returns (h, x).
    See pk_add_rmsnorm."""
    _require_cuda(a, weight)
    h, x = torch.empty_like(a), torch.empty_like(a)
    d = [L.desc(t) if t is not None else None for t in (a, residual, weight, h, x)]
    _call("pk_add_rmsnorm", *[L.ref(t) if t is not None else None for t in d], float(eps), L.stream_ptr(a.device))
    return h, x


def silu_mul(gate_up):
    """silu(gate_up[:, :F]) * gate_up[:, F:], one launch.  See pk_silu_mul."""
    _require_cuda(gate_up)
    out = torch.empty(gate_up.shape[0], gate_up.shape[1] // 2, dtype=torch.bfloat16, device=gate_up.device)
    d = [L.desc(gate_up), L.desc(out)]
    _call("pk_silu_mul", L.ref(d[0]), L.ref(d[1]), L.stream_ptr(gate_up.device))
    return out


def gemv(weight, x, gated=False):
    """x [1, I] @ weight[O, I]^T -> [1, O] (bf16, fp32 accumulation) for one token; gated: weight = [gate; up] stacked,
    result [1, O/2] = silu(gate x) * (up x).  See pk_gemv."""
    _require_cuda(weight, x)
    O = weight.shape[0]
    out = torch.empty(1, O // 2 if gated else O, dtype=torch.bfloat16, device=x.device)
    d = [L.desc(weight), L.desc(x), L.desc(out)]
    _call("pk_gemv", L.ref(d[0]), L.ref(d[1]), L.ref(d[2]), int(bool(gated)), L.stream_ptr(x.device))
    return out
