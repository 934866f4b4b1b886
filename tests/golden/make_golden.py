"""Generates the golden fixtures in this folder by RUNNING THE REFERENCE'S OWN PYTHON CODE on CPU.

Run once, in a container that has a checkout of the reference project:

    python tests/golden/make_golden.py --ref <path of the ParisKV checkout>

The fixtures are committed; nothing else in the repository reads the reference checkout.

What is executed from the reference (imported, not restated):
  * cache_hub/polar_cache.py   polar_cache.batch_encode, _pack_4bit_codes, _count_cluster_keys,
                               _encode_query_blocks, get_cache_cnt_fused, the GQA query mean of
                               compute() (:1027-1031 is inlined there, so it is the one line
                               repeated here), _get_adaptive_ratios
  * cache_hub/collision_fused/collision_test.py   generate_test_input, update_cache_cnt_overall_ref,
                               update_cache_cnt_ref
  * cache_hub/collision/collision.py              update_cache_cnt_ref (single tier)
  * cache_hub/rerank/rerank.py                    rerank_rabitq_ref, _coarse_filter_truncate
  * cache_hub/adaptive_k_fused/adaptive_topk.py   generate_test_input, adaptive_topk_ref

Two stand-ins are unavoidable and are stated in every fixture's "note":
  * fast_hadamard_transform (a CUDA-only wheel that is not installed) is replaced by an fp32
    matrix product with the Sylvester Hadamard matrix, scale applied in fp32, one cast back;
  * the CUDA extension calls inside get_cache_cnt_fused are replaced by the reference's own torch
    reference for the same op (update_cache_cnt_ref per tier).
The SRHT sign vector is drawn on CPU (the reference draws it with the CUDA generator), so it is
stored in the fixture and passed explicitly to every implementation.
"""
import argparse
import importlib.util
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def hadamard_stub(x, scale=1.0):
    n = x.shape[-1]
    H = torch.ones(1, 1)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return ((x.float() @ H) * scale).to(x.dtype)


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t):
    """bf16 tensor -> uint16 numpy (bit pattern)."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def synth_keys(gen, bs, H, N, outliers=(7, 37, 71, 101)):
    """Keys with the distribution of the headline benchmark: N(0,1), four fixed channels x8,
    per-token lognormal(0, 0.5) norm factor, bf16."""
    z = torch.randn(bs, H, N, 128, generator=gen)
    z[..., list(outliers)] *= 8.0
    g = torch.exp(0.5 * torch.randn(bs, H, N, 1, generator=gen))
    return (z * g).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference (ParisKV) checkout")
    args = ap.parse_args()
    ref = args.ref
    sys.path.insert(0, ref)
    stub = types.ModuleType("fast_hadamard_transform")
    stub.hadamard_transform = hadamard_stub
    sys.modules["fast_hadamard_transform"] = stub
    import cache_hub  # noqa: F401  (executes the reference package)
    pc = sys.modules["cache_hub.polar_cache"]
    ctest = load_by_path("ref_collision_test", f"{ref}/cache_hub/collision_fused/collision_test.py")
    csingle = load_by_path("ref_collision_single", f"{ref}/cache_hub/collision/collision.py")
    rr = load_by_path("ref_rerank", f"{ref}/cache_hub/rerank/rerank.py")
    ak = load_by_path("ref_adaptive", f"{ref}/cache_hub/adaptive_k_fused/adaptive_topk.py")
    torch.set_num_threads(8)

    # ---- a fake `self` carrying exactly the attributes the reference methods read ----
    gen = torch.Generator().manual_seed(42)
    signs = (torch.randint(0, 2, (128,), generator=gen).to(torch.bfloat16) * 2 - 1)
    quant = types.SimpleNamespace(srht_diagonal_signs=[signs], B=16, m=8)
    fake = types.SimpleNamespace(
        quantizer=quant, _hadamard_scale=1.0 / math.sqrt(128), polar_B=16, polar_m=8, polar_K_omega=256,
        _bitpack_shifts=(1 << torch.arange(8, dtype=torch.uint8)),
        _mag_thresholds=torch.tensor([0.0843, 0.1698, 0.2578, 0.3499, 0.4487, 0.5585, 0.6901],
                                     dtype=torch.bfloat16),
        _mag_centers=torch.tensor([0.0420, 0.1266, 0.2130, 0.3025, 0.3973, 0.5001, 0.6169, 0.7633],
                                  dtype=torch.bfloat16),
    )
    cls = pc.polar_cache
    fake._pack_4bit_codes = types.MethodType(cls._pack_4bit_codes, fake)
    sign_table = torch.tensor([[1.0 if (c >> j) & 1 else -1.0 for j in range(8)] for c in range(256)],
                              dtype=torch.bfloat16)
    fake._V_omega_gpu_T = sign_table.T.contiguous()

    # ---- A. encode ----
    g = torch.Generator().manual_seed(0)
    keys = synth_keys(g, 1, 2, 384)
    keys[0, 0, 0] = 0                       # all-zero key (clamp paths)
    keys[0, 0, 1] = 0
    keys[0, 0, 1, 5] = 1.0                  # one-hot key: |y| all equal after the rotation
    keys[0, 0, 2] = keys[0, 0, 3] * 1e-30   # tiny norm
    cb, w, pk = cls.batch_encode(fake, keys, layer_idx=0, return_rabitq=True)
    counts = cls._count_cluster_keys(fake, cb, cb.device)
    np.savez_compressed(
        os.path.join(HERE, "encode.npz"), signs=bits(signs), keys=bits(keys), codebook=cb.numpy(),
        block_weight=bits(w), packed_4bit=pk.numpy(), cluster_counts=counts.numpy(),
        mag_thresholds=bits(fake._mag_thresholds), mag_centers=bits(fake._mag_centers),
        note="reference polar_cache.batch_encode/_count_cluster_keys on CPU; Hadamard stand-in fp32 matmul")

    # ---- B. query prep + cluster ranking + fused collision through the reference's own methods ----
    g = torch.Generator().manual_seed(1)
    bs, H, N = 2, 2, 1536
    keys_b = synth_keys(g, bs, H, N)
    cb_b, w_b, pk_b = cls.batch_encode(fake, keys_b, layer_idx=0, return_rabitq=True)
    counts_b = cls._count_cluster_keys(fake, cb_b, cb_b.device)
    pick = torch.randint(0, N, (bs, H, 4), generator=g)
    qs = torch.stack([torch.stack([keys_b[b, h, pick[b, h]].float() for h in range(H)]) for b in range(bs)])
    qs = 0.3 * qs / qs.norm(dim=-1, keepdim=True) + torch.randn(bs, H, 4, 128, generator=g) / math.sqrt(128)
    qs = (qs / qs.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    queries = qs.view(bs, 1, H * 4, 128).contiguous()
    fake.kv_head, fake.group_size, fake.head_dim = H, 4, 128
    query_avg = queries[:, 0].view(bs, H, 4, 128).mean(dim=2)      # polar_cache.compute :1028-1030
    q_blocks, q_norm = cls._encode_query_blocks(fake, query_avg)
    seen = {}

    def fused_stub(sorted_ids, ckc, codebook, tier_counts):
        seen["sorted_ids"] = sorted_ids.clone()
        seen["tier_counts"] = list(tier_counts)
        skc = torch.gather(ckc, -1, sorted_ids.long())
        before = torch.cumsum(skc, -1) - skc
        total = None
        for t in tier_counts:
            n_sel = (before < t).sum(-1)
            c = ctest.update_cache_cnt_ref(sorted_ids, n_sel, codebook)
            total = c if total is None else total + c
        return total.to(torch.int32)

    fake._update_cache_cnt_fused = fused_stub
    fake.cluster_key_counts_gpu = [counts_b]
    cand_ratio, coll_ratio = cls._get_adaptive_ratios(fake, N)
    cache_cnt = cls.get_cache_cnt_fused(fake, q_blocks, cb_b, coll_ratio, 0)
    scores = torch.matmul(q_blocks, fake._V_omega_gpu_T)            # only stored to check tie handling
    np.savez_compressed(
        os.path.join(HERE, "query_collision.npz"), signs=bits(signs), queries=bits(queries),
        query_avg=bits(query_avg), q_blocks=bits(q_blocks), q_norm=bits(q_norm),
        cluster_scores=bits(scores), sorted_ids=seen["sorted_ids"].numpy().astype(np.int16),
        tier_counts=np.array(seen["tier_counts"], dtype=np.int64), collision_ratio=coll_ratio,
        candidate_ratio=cand_ratio, keys=bits(keys_b), codebook=cb_b.numpy(), block_weight=bits(w_b),
        packed_4bit=pk_b.numpy(), cluster_counts=counts_b.numpy(), cache_cnt=cache_cnt.numpy(),
        note="reference _encode_query_blocks/get_cache_cnt_fused on CPU; CUDA collision op replaced by "
             "the reference's update_cache_cnt_ref per tier")

    # ---- C. the reference's own collision test generator (seed 42) ----
    out = {}
    for tag, kv_len in (("n2048", 2048), ("n1000", 1000)):
        ids, ckc, codebook, tier_ratios, kv_len, ratio = ctest.generate_test_input(kv_len=kv_len)
        ref = ctest.update_cache_cnt_overall_ref(ids, ckc, codebook, tier_ratios, kv_len, ratio)
        out[f"{tag}_sorted_ids"] = ids.numpy().astype(np.int16)
        out[f"{tag}_cluster_counts"] = ckc.numpy()
        out[f"{tag}_codebook"] = codebook.numpy().astype(np.uint8)
        out[f"{tag}_tier_counts"] = np.array([math.ceil(kv_len * ratio * r) for r in tier_ratios], dtype=np.int64)
        out[f"{tag}_cache_cnt"] = ref.numpy().astype(np.int32)
    ids1, cnt1, cb1 = None, None, None
    torch.manual_seed(42)
    ids1 = torch.stack([torch.stack([torch.stack([torch.randperm(64) for _ in range(16)]) for _ in range(2)])
                        for _ in range(1)]).to(torch.int32)
    cnt1 = torch.randint(1, 64, (1, 2, 16), dtype=torch.int32)
    cb1 = torch.randint(0, 64, (1, 2, 16, 777), dtype=torch.int32)
    out["single_sorted_ids"] = ids1.numpy()
    out["single_topk_cluster_cnt"] = cnt1.numpy()
    out["single_codebook"] = cb1.numpy()
    out["single_cache_cnt"] = csingle.update_cache_cnt_ref(ids1, cnt1, cb1).numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "collision.npz"), **out,
                        note="collision_test.generate_test_input(seed 42) + update_cache_cnt_overall_ref; "
                             "single_* = collision.py update_cache_cnt_ref")

    # ---- D. rerank: the reference's torch reference, evaluated in fp32 and in bf16 ----
    torch.manual_seed(42)
    bs, H, B, m, N = 1, 2, 16, 8, 4096
    cache_cnt_r = torch.randint(0, B + 1, (bs, H, N), dtype=torch.int32)
    sign = torch.randint(0, 2, (bs, H, B, N, m))
    mag = torch.randint(0, 8, (bs, H, B, N, m))
    v4 = (sign << 3) | mag
    key_4bit = ((v4[..., 1::2] << 4) | v4[..., 0::2]).to(torch.uint8)
    kbw = torch.randn(bs, H, B, N, dtype=torch.bfloat16).abs()
    qb = torch.randn(bs, H, B, m, dtype=torch.bfloat16)
    qn = torch.randn(bs, H, 1, dtype=torch.bfloat16).abs() + 0.1
    cen = fake._mag_centers
    ratio, K = 0.1, 100
    cand, C = rr._coarse_filter_truncate(cache_cnt_r, ratio)
    rec = {}
    orig_topk = torch.topk

    def spy(x, *a, **k):
        rec["last"] = x
        return orig_topk(x, *a, **k)

    # candidate_ratio=1.0 makes every key a candidate, so the recorded scores cover all N keys
    torch.topk = spy
    try:
        fin32 = rr.rerank_rabitq_ref(cache_cnt_r, key_4bit, kbw.float(), qb.float(), qn.float(), cen.float(),
                                     1.0, K, B, m)
        order32 = orig_topk(cache_cnt_r, k=N, dim=-1)[1]
        scores32_in_order = rec["last"].clone()
        finbf = rr.rerank_rabitq_ref(cache_cnt_r, key_4bit, kbw, qb, qn, cen, 1.0, K, B, m)
    finally:
        torch.topk = orig_topk
    scores32 = torch.empty_like(scores32_in_order)
    scores32.scatter_(2, order32, scores32_in_order)              # back to key order
    np.savez_compressed(
        os.path.join(HERE, "rerank.npz"), cache_cnt=cache_cnt_r.numpy(), key_4bit=key_4bit.numpy(),
        key_block_weight=bits(kbw), q_blocks=bits(qb), q_norm=bits(qn), mag_centers=bits(cen),
        scores_fp32=scores32.numpy(), final_fp32=fin32.numpy().astype(np.int32),
        final_bf16=finbf.numpy().astype(np.int32), candidate_ratio=ratio, final_topk=K,
        truncate_candidates=cand.numpy().astype(np.int32),
        note="rerank.rerank_rabitq_ref with every key a candidate; fp32 inputs for the score pin, "
             "bf16 inputs for the literal result")

    # ---- E. adaptive-k: the reference's four verification configs ----
    cfgs = [dict(bs=1, kv_heads=8, head_dim=128, sl_len=320, cand_len=12500, topk_cap=2048, threshold=0.95, seed=42),
            dict(bs=1, kv_heads=8, head_dim=128, sl_len=832, cand_len=5000, topk_cap=2048, threshold=0.95, seed=7),
            dict(bs=2, kv_heads=8, head_dim=128, sl_len=576, cand_len=8000, topk_cap=2048, threshold=0.85, seed=123),
            dict(bs=1, kv_heads=16, head_dim=128, sl_len=320, cand_len=15000, topk_cap=2048, threshold=0.95, seed=99)]
    out = {}
    for i, cfg in enumerate(cfgs):
        inp = ak.generate_test_input(device="cpu", **cfg)
        k_ref, idx_ref = ak.adaptive_topk_ref(
            inp["query_avg"], inp["sink_local_keys"], inp["sl_vnorm"], inp["cand_scores"], inp["cand_indices"],
            inp["cand_vnorm"], attn_scale=inp["attn_scale"], threshold=inp["threshold"], topk_cap=inp["topk_cap"])
        sl_logits = torch.einsum("bhd,bhkd->bhk", inp["query_avg"], inp["sink_local_keys"]).to(torch.float32) \
            * inp["attn_scale"]                                     # adaptive_topk.py:379-381
        # heads are independent: keep the first four of each config to keep the file small
        hs = slice(0, 4)
        out[f"c{i}_sl_logits"] = sl_logits[:, hs].numpy()
        out[f"c{i}_sl_vnorm"] = inp["sl_vnorm"][:, hs].numpy()
        out[f"c{i}_cand_scores"] = bits(inp["cand_scores"][:, hs])
        out[f"c{i}_cand_indices"] = inp["cand_indices"][:, hs].numpy().astype(np.int32)
        out[f"c{i}_cand_vnorm"] = inp["cand_vnorm"][:, hs].numpy()
        out[f"c{i}_attn_scale"] = inp["attn_scale"]
        out[f"c{i}_threshold"] = inp["threshold"]
        out[f"c{i}_topk_cap"] = inp["topk_cap"]
        out[f"c{i}_adaptive_k"] = k_ref[:, hs].numpy()
        out[f"c{i}_topk_indices"] = idx_ref[:, hs].numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "adaptive_topk.npz"), **out,
                        note="adaptive_topk.generate_test_input(device=cpu) + adaptive_topk_ref, heads 0-3")
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
