"""ctypes front end of the CPU oracle (``pariskv_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module.  It is loaded by the tests, by the
smoke check and by the CPU-baseline / reference legs of the benchmark, always as the
checker or as the timed CPU baseline, never as a fallback of the CUDA path.

Tensors use the reference's logical shapes (``cache_hub/polar_cache.py:924-936``):
codebook ``[bs, H, 16, N]`` u8, block weights ``[bs, H, 16, N]`` bf16, packed 4-bit
``[bs, H, 16, N, 4]`` u8.  Outputs produced here are key-major in memory and returned
as permuted views with those logical shapes.
"""
import ctypes
import math
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

c_i64 = ctypes.c_int64
c_p = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to this file; returns the .so path."""
    so = os.path.join(_HERE, "libpariskv_oracle.so")
    src = os.path.join(_HERE, "pariskv_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libpariskv_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libpariskv_oracle.so")
        if not os.path.exists(so):
            build()
        _LIB = ctypes.CDLL(so)
        _LIB.pko_adaptive_topk.restype = c_i64
        _LIB.pko_expf.restype = ctypes.c_float
        _LIB.pko_expf.argtypes = [ctypes.c_float]
    return _LIB


def _p(t):
    return c_p(t.data_ptr())


def _cpu(t, dtype=None):
    t = t.detach().cpu()
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t


def constants():
    """(thresholds[7], centers[8]) as bf16 tensors: cache_hub/polar_cache.py:188-193."""
    thr = torch.empty(7, dtype=torch.float32)
    cen = torch.empty(8, dtype=torch.float32)
    lib().pko_constants(_p(thr), _p(cen))
    return thr.to(torch.bfloat16), cen.to(torch.bfloat16)


def encode(keys, signs):
    """keys [bs,H,L,128] bf16 -> (codebook, block_weight, packed_4bit) in reference shapes."""
    keys = _cpu(keys, torch.bfloat16).contiguous()
    signs = _cpu(signs, torch.bfloat16).contiguous()
    bs, H, L, D = keys.shape
    assert D == 128
    codes = torch.empty(bs, H, L, 16, dtype=torch.uint8)
    w = torch.empty(bs, H, L, 16, dtype=torch.bfloat16)
    pk = torch.empty(bs, H, L, 16, 4, dtype=torch.uint8)
    if L > 0:
        lib().pko_encode(_p(keys), c_i64(bs * H * L), _p(signs), _p(codes), _p(w), _p(pk))
    return codes.permute(0, 1, 3, 2), w.permute(0, 1, 3, 2), pk.permute(0, 1, 3, 2, 4)


def cluster_counts(codebook):
    """codebook [bs,H,16,N] u8 -> int32 [bs,H,16,256]."""
    cb = _cpu(codebook).permute(0, 1, 3, 2).contiguous()
    bs, H, N, B = cb.shape
    out = torch.zeros(bs, H, B, 256, dtype=torch.int32)
    for b in range(bs):
        for h in range(H):
            lib().pko_cluster_counts(_p(cb[b, h]), c_i64(N), _p(out[b, h]))
    return out


def query_prep(queries, kv_heads, signs):
    """queries [bs,1,Hq,128] bf16 -> (q_blocks [bs,H,16,8] bf16, q_norm [bs,H,1] bf16)."""
    q = _cpu(queries, torch.bfloat16).contiguous()
    signs = _cpu(signs, torch.bfloat16).contiguous()
    bs, one, Hq, D = q.shape
    G = Hq // kv_heads
    q = q.view(bs, kv_heads, G, D)
    qb = torch.empty(bs, kv_heads, 16, 8, dtype=torch.bfloat16)
    qn = torch.empty(bs, kv_heads, 1, dtype=torch.bfloat16)
    for b in range(bs):
        for h in range(kv_heads):
            lib().pko_query_prep(_p(q[b, h]), ctypes.c_int(G), _p(signs), _p(qb[b, h]), _p(qn[b, h]))
    return qb, qn


def cluster_rank(q_blocks):
    """q_blocks [bs,H,16,8] bf16 -> sorted_cluster_ids int64 [bs,H,16,256]."""
    qb = _cpu(q_blocks, torch.bfloat16).contiguous()
    bs, H = qb.shape[:2]
    out = torch.empty(bs, H, 16, 256, dtype=torch.int64)
    for b in range(bs):
        for h in range(H):
            lib().pko_cluster_rank(_p(qb[b, h]), _p(out[b, h]))
    return out


def tier_counts(kv_len, collision_ratio, tier_ratios=(0.05, 0.15, 0.30, 0.50, 0.75, 1.0)):
    """cache_hub/polar_cache.py:1221-1222 (Python floats, ceil)."""
    return [int(math.ceil(kv_len * collision_ratio * r)) for r in tier_ratios]


def candidate_len(kv_len, candidate_ratio):
    """cache_hub/polar_cache.py:1239-1240."""
    return max(1, int(math.ceil(kv_len * candidate_ratio)))


def adaptive_ratios(retrieval_len):
    """(candidate_ratio, collision_ratio): cache_hub/polar_cache.py:1113-1124."""
    if retrieval_len < 5000:
        return 0.5, 0.5
    if retrieval_len < 10000:
        return 0.25, 0.3
    if retrieval_len < 30000:
        return 0.2, 0.25
    return 0.1, 0.2


def collision(sorted_ids, cluster_key_counts, codebook, tiers):
    """Weighted multi-tier collision counts -> int32 [bs,H,N]."""
    ids = _cpu(sorted_ids, torch.int64).contiguous()
    ckc = _cpu(cluster_key_counts, torch.int32).contiguous()
    cb = _cpu(codebook, torch.uint8)
    bs, H, B, N = cb.shape
    NC = ids.shape[-1]
    tc = torch.tensor(list(tiers), dtype=torch.int64)
    out = torch.empty(bs, H, N, dtype=torch.int32)
    for b in range(bs):
        for h in range(H):
            v = cb[b, h]
            lib().pko_collision(_p(ids[b, h]), _p(ckc[b, h]), _p(v), c_i64(v.stride(1)),
                                c_i64(v.stride(0)), c_i64(N), ctypes.c_int(B), ctypes.c_int(NC),
                                _p(tc), ctypes.c_int(len(tiers)), _p(out[b, h]))
    return out


def collision_single(sorted_ids, topk_cluster_cnt, codebook):
    """Unfused single-tier count; codebook int32 [bs,H,B,N] (cache_hub/collision/collision.py:87-98)."""
    ids = _cpu(sorted_ids, torch.int32).contiguous()
    cnt = _cpu(topk_cluster_cnt, torch.int32).contiguous()
    cb = _cpu(codebook, torch.int32).transpose(-1, -2).contiguous()
    bs, H, N, B = cb.shape
    NC = ids.shape[-1]
    out = torch.empty(bs, H, N, dtype=torch.int32)
    for b in range(bs):
        for h in range(H):
            lib().pko_collision_single(_p(ids[b, h]), _p(cnt[b, h]), _p(cb[b, h]), c_i64(N),
                                       ctypes.c_int(B), ctypes.c_int(NC), _p(out[b, h]))
    return out


def topk(values, k, sorted_by_value=False):
    """Deterministic top-k over the last dim (value desc, index asc); int32 or float32 input.
    Output int64 [..., k]: ascending index, or in selection order when sorted_by_value."""
    v = _cpu(values)
    if v.dtype not in (torch.int32, torch.float32):
        v = v.to(torch.float32)
    v = v.contiguous()
    lead, n = v.shape[:-1], v.shape[-1]
    v2 = v.view(-1, n)
    out = torch.empty(v2.shape[0], k, dtype=torch.int64)
    fn = lib().pko_topk_i32 if v.dtype == torch.int32 else lib().pko_topk_f32
    for r in range(v2.shape[0]):
        fn(_p(v2[r]), c_i64(n), c_i64(k), _p(out[r]), ctypes.c_int(int(sorted_by_value)))
    return out.view(*lead, k)


def rerank(cand, key_4bit, key_block_weight, q_blocks, q_norm, centers):
    """-> (score fp32 [bs,H,C], score bf16 [bs,H,C])."""
    cand = _cpu(cand, torch.int64).contiguous()
    k4 = _cpu(key_4bit, torch.uint8)
    w = _cpu(key_block_weight, torch.bfloat16)
    qb = _cpu(q_blocks, torch.bfloat16).contiguous()
    qn = _cpu(q_norm, torch.bfloat16).contiguous()
    cen = _cpu(centers, torch.bfloat16).contiguous()
    bs, H, C = cand.shape
    assert k4.stride(-1) == 1
    s32 = torch.empty(bs, H, C, dtype=torch.float32)
    sbf = torch.empty(bs, H, C, dtype=torch.bfloat16)
    for b in range(bs):
        for h in range(H):
            a, ww = k4[b, h], w[b, h]
            qn_bits = int(qn[b, h].view(torch.int16).item()) & 0xFFFF
            lib().pko_rerank(_p(cand[b, h]), c_i64(C), _p(a), c_i64(a.stride(1)), c_i64(a.stride(0)),
                             _p(ww), c_i64(ww.stride(1)), c_i64(ww.stride(0)), _p(qb[b, h]),
                             ctypes.c_uint16(qn_bits), _p(cen), _p(s32[b, h]), _p(sbf[b, h]))
    return s32, sbf


def final_topk(score32, cand, K):
    s = _cpu(score32, torch.float32).contiguous()
    cand = _cpu(cand, torch.int64).contiguous()
    bs, H, C = s.shape
    out = torch.empty(bs, H, K, dtype=torch.int64)
    for b in range(bs):
        for h in range(H):
            lib().pko_final_topk(_p(s[b, h]), _p(cand[b, h]), c_i64(C), c_i64(K), _p(out[b, h]))
    return out


def adaptive_topk(sl_logits, sl_vnorm, cand_logits, cand_vnorm, cand_indices, threshold, K_out):
    """fp32 scaled logits in; -> (adaptive_k int64 [bs,H], topk_indices int64 [bs,H,K_out])."""
    sl = _cpu(sl_logits, torch.float32).contiguous()
    sv = _cpu(sl_vnorm, torch.float32).contiguous()
    cl = _cpu(cand_logits, torch.float32).contiguous()
    cv = _cpu(cand_vnorm, torch.float32).contiguous()
    ci = _cpu(cand_indices, torch.int64).contiguous()
    bs, H, S = sl.shape
    C = cl.shape[-1]
    ak = torch.empty(bs, H, dtype=torch.int64)
    out = torch.empty(bs, H, K_out, dtype=torch.int64)
    for b in range(bs):
        for h in range(H):
            ak[b, h] = lib().pko_adaptive_topk(_p(sl[b, h]), _p(sv[b, h]), c_i64(S), _p(cl[b, h]),
                                               _p(cv[b, h]), _p(ci[b, h]), c_i64(C),
                                               ctypes.c_float(threshold), c_i64(K_out), _p(out[b, h]))
    return ak, out


def gather(src, idx):
    """src [bs,H,N,D], idx int64 [bs,H,K] -> [bs,H,K,D]."""
    src = _cpu(src).contiguous()
    idx = _cpu(idx, torch.int64).contiguous()
    bs, H, N, D = src.shape
    K = idx.shape[-1]
    out = torch.empty(bs, H, K, D, dtype=src.dtype)
    rb = D * src.element_size()
    for b in range(bs):
        for h in range(H):
            lib().pko_gather_rows(_p(src[b, h]), _p(idx[b, h]), c_i64(K), c_i64(rb), _p(out[b, h]))
    return out


def attention(queries, keys, values, scale=None):
    """queries [bs,1,Hq,128] bf16; keys/values [bs,H,n,128] bf16 -> fp32 [bs,1,Hq,128]."""
    q = _cpu(queries, torch.bfloat16).contiguous()
    k = _cpu(keys, torch.bfloat16).contiguous()
    v = _cpu(values, torch.bfloat16).contiguous()
    bs, one, Hq, D = q.shape
    H, n = k.shape[1], k.shape[2]
    G = Hq // H
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.empty(bs, 1, Hq, D, dtype=torch.float32)
    PtrArr = ctypes.c_void_p * max(n, 1)
    for b in range(bs):
        for h in range(H):
            kp = PtrArr(*[k[b, h].data_ptr() + r * D * 2 for r in range(n)])
            vp = PtrArr(*[v[b, h].data_ptr() + r * D * 2 for r in range(n)])
            lib().pko_attention(_p(q[b, 0, h * G:(h + 1) * G]), ctypes.c_int(G), kp, vp, c_i64(n),
                                ctypes.c_float(scale), _p(out[b, 0, h * G:(h + 1) * G]))
    return out


def retrieve(queries, signs, codebook, key_block_weight, key_4bit, cluster_key_counts, centers,
             collision_ratio, C, K):
    """The whole retrieval chain of cache_hub/polar_cache.py:1126-1162 / :1207-1304 for one
    decode step.  Returns a dict with every intermediate so tests can compare stage by stage."""
    H = codebook.shape[1]
    N = codebook.shape[3]
    qb, qn = query_prep(queries, H, signs)
    ids = cluster_rank(qb)
    tiers = tier_counts(N, collision_ratio)
    cnt = collision(ids, cluster_key_counts, codebook, tiers)
    cand = topk(cnt, C)
    s32, sbf = rerank(cand, key_4bit, key_block_weight, qb, qn, centers)
    fin = final_topk(s32, cand, min(K, C))
    return dict(q_blocks=qb, q_norm=qn, sorted_ids=ids, tiers=tiers, cache_cnt=cnt, cand=cand,
                score32=s32, score_bf16=sbf, final=fin)
