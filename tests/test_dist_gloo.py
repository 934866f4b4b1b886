"""World-size-2 tests of the multi-GPU plumbing with gloo ranks on CPU: the exchange of count histograms and local top
lists, the partial-attention merge and the histogram all-reduce of the sequence-sharded form.  The reference is the
oracle's SINGLE-GPU selection over the whole zone: the sharded form must reproduce it bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import srht_signs, synth_keys, synth_queries


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_select(scores, indices, k):
    from oracle import oracle as O
    return O.final_topk(scores, indices, k)


def _shard_counts(O, span, keys, q, signs, coll, counts_global):
    """Collision counts of one shard with the GLOBAL thresholds and cluster histogram, plus what the rerank needs."""
    start, end = span
    N, H = keys.shape[2], keys.shape[1]
    cb, w, pk = O.encode(keys[:, :, start:end].contiguous(), signs)
    qb, qn = O.query_prep(q, H, signs)
    cnt = O.collision(O.cluster_rank(qb), counts_global, cb, O.tier_counts(N, coll))
    return cnt, (pk, w, qb, qn)


def _count_hist(cnt):
    """int32 [bs,H,256]: how many keys of the shard have each collision count."""
    bs, H, n = cnt.shape
    h = torch.zeros(bs, H, 256, dtype=torch.int32)
    h.scatter_add_(2, cnt.long(), torch.ones(bs, H, n, dtype=torch.int32))
    return h


def _shard_result(O, rank, spans, keys, q, signs, cen, coll, cand_ratio, K, counts_global, hist_all=None):
    """One rank's part of the exact sharded selection on the CPU: candidates by the global threshold count and this
    shard's share of the ties, rerank, local top-K; lists padded to K entries with (-inf, -1).  hist_all
    [world,bs,H,256] is what the all-gather delivers; when None it is computed here from every shard."""
    from pariskv_b200 import dist as pkd
    N = keys.shape[2]
    _, c_total, k_final = pkd.global_plan(N, coll, cand_ratio, K)
    cnt, (pk, w, qb, qn) = _shard_counts(O, spans[rank], keys, q, signs, coll, counts_global)
    if hist_all is None:
        hist_all = torch.stack([_count_hist(_shard_counts(O, sp, keys, q, signs, coll, counts_global)[0]) for sp in spans])
    T, ties, n_cand = pkd.shard_candidate_plan(hist_all, rank, c_total)
    bs, H, n = cnt.shape
    start = spans[rank][0]
    sc_out = torch.full((bs, H, k_final), float("-inf"))
    idx_out = torch.full((bs, H, k_final), -1, dtype=torch.int64)
    for b in range(bs):
        for h in range(H):
            c = cnt[b, h]
            eq = torch.nonzero(c == T[b, h]).flatten()[: int(ties[b, h])]
            cand = torch.cat([torch.nonzero(c > T[b, h]).flatten(), eq]).sort().values
            assert cand.numel() == int(n_cand[b, h])
            if cand.numel() == 0:
                continue
            s32, _ = O.rerank(cand.view(1, 1, -1), pk[b:b + 1, h:h + 1], w[b:b + 1, h:h + 1], qb[b:b + 1, h:h + 1],
                              qn[b:b + 1, h:h + 1], cen)
            kl = min(k_final, cand.numel())
            loc = O.final_topk(s32, cand.view(1, 1, -1), kl)[0, 0]
            sc_out[b, h, :kl] = s32[0, 0][torch.searchsorted(cand, loc)]
            idx_out[b, h, :kl] = loc + start
    return sc_out, idx_out


def _single_gpu_final(O, keys, q, signs, cen, coll, cand_ratio, K, counts_global):
    """The reference: the whole zone on one device (cache_hub/polar_cache.py:1207-1304 restated by the oracle)."""
    from pariskv_b200 import dist as pkd
    N = keys.shape[2]
    _, c_total, k_final = pkd.global_plan(N, coll, cand_ratio, K)
    cb, w, pk = O.encode(keys, signs)
    return O.retrieve(q, signs, cb, w, pk, counts_global, cen, coll, c_total, k_final)["final"]


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from pariskv_b200 import dist as pkd
        g = torch.Generator().manual_seed(3)
        bs, H, N, K = 1, 2, 3001, 96
        keys = synth_keys(g, bs, H, N)
        vals = torch.randn(bs, H, N, 128, generator=g).to(torch.bfloat16)
        q = synth_queries(g, keys, 4) * 4
        signs = srht_signs()
        _, cen = O.constants()
        cand_ratio, coll = O.adaptive_ratios(N)
        start, end = pkd.sequence_shard(N, rank, world)
        # global histogram = all-reduce of the local ones
        cb_local, _, _ = O.encode(keys[:, :, start:end].contiguous(), signs)
        counts = O.cluster_counts(cb_local)
        pkd.allreduce_cluster_counts(counts)
        cb_all, _, _ = O.encode(keys, signs)
        assert torch.equal(counts, O.cluster_counts(cb_all))
        # local counts, exchange of the count histograms, candidates by the global threshold, exchange of the local
        # top lists, global selection
        spans = [pkd.sequence_shard(N, r, world) for r in range(world)]
        mine = _count_hist(_shard_counts(O, spans[rank], keys, q, signs, coll, counts)[0])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        hist_all = torch.stack(gathered)
        sc, gi = _shard_result(O, rank, spans, keys, q, signs, cen, coll, cand_ratio, K, counts, hist_all=hist_all)
        final = pkd.merge_local_topk(sc, gi, K, select=_oracle_select)
        # the reference: the single-GPU selection over the whole zone
        want = _single_gpu_final(O, keys, q, signs, cen, coll, cand_ratio, K, counts)
        assert torch.equal(final, want), "the sharded selection is not the single-GPU selection"
        T, ties, n_cand = pkd.shard_candidate_plan(hist_all, rank, pkd.global_plan(N, coll, cand_ratio, K)[1])
        tot = n_cand.clone()
        dist.all_reduce(tot)
        assert bool((tot == pkd.global_plan(N, coll, cand_ratio, K)[1]).all()), "shards' candidate counts must add up"
        assert bool((final[..., 1:] > final[..., :-1]).all())
        # every rank attends its own rows; partial results merge to attention over the union
        local, n_owned = pkd.owned_rows(final, start, end)
        assert int(n_owned.sum()) == int(((final >= start) & (final < end)).sum())
        outs, lses = [], []
        out = torch.zeros(bs, 1, 4 * H, 128)
        lse = torch.full((bs, 4 * H), float("-inf"))
        for h in range(H):
            n = int(n_owned[0, h])
            if n == 0:
                continue
            kk = O.gather(keys[:, h:h + 1, start:end].contiguous(), local[:, h:h + 1, :n])
            vv = O.gather(vals[:, h:h + 1, start:end].contiguous(), local[:, h:h + 1, :n])
            qq = q[:, :, 4 * h:4 * h + 4]
            out[:, :, 4 * h:4 * h + 4] = O.attention(qq, kk, vv)
            logits = torch.einsum("gd,nd->gn", qq[0, 0].float(), kk[0, 0].float()) / 128 ** 0.5
            lse[0, 4 * h:4 * h + 4] = torch.logsumexp(logits, -1) / 0.6931471805599453
        merged = pkd.merge_partial_attention(out, lse)
        ref = O.attention(q, O.gather(keys, final), O.gather(vals, final))
        assert (merged - ref).abs().max().item() < 1e-4
        torch.save(final, os.path.join(tmp, f"final_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_exchange_world2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = torch.load(os.path.join(tmp_path, "final_0.pt"))
    b = torch.load(os.path.join(tmp_path, "final_1.pt"))
    assert torch.equal(a, b), "ranks disagree on the global selection"


def test_head_and_sequence_shards():
    from pariskv_b200 import dist as pkd
    assert pkd.head_shard(8, 3, 4) == slice(6, 8)
    with pytest.raises(ValueError):
        pkd.head_shard(8, 0, 3)
    cover = [pkd.sequence_shard(1048508, r, 8) for r in range(8)]
    assert cover[0][0] == 0 and cover[-1][1] == 1048508
    assert all(cover[i][1] == cover[i + 1][0] for i in range(7))
    tiers, c_total, k_final = pkd.global_plan(1048508, 0.2, 0.1, 2048)
    assert c_total == 104851 and k_final == 2048 and tiers[-1] == 209702


def test_owned_rows_split():
    from pariskv_b200 import dist as pkd
    sel = torch.tensor([[[2, 5, 9, 14, 20]]])
    local, n = pkd.owned_rows(sel, 5, 15)
    assert n.tolist() == [[3]] and local[0, 0, :3].tolist() == [0, 4, 9]


def test_tier_thresholds_match_the_reference_arithmetic():
    """ceil(N * collision_ratio * rho) in Python floats, rho in (.05, .15, .30, .50, .75, 1): for N = 32768 and ratio
    0.2 the reference's own arithmetic (cache_hub/polar_cache.py:1221-1222) gives 328, 984, 1967, 3277, 4916, 6554."""
    from oracle import oracle as O
    from pariskv_b200 import dist as pkd
    want = [328, 984, 1967, 3277, 4916, 6554]
    assert list(O.tier_counts(32768, 0.2)) == want
    tiers, c_total, k_final = pkd.global_plan(32768, 0.2, 4096 / 32768, 256)
    assert tiers == want and c_total == 4096 and k_final == 256


def test_shard_candidate_plan_splits_ties_in_rank_order():
    """Three shards; 5 candidates wanted; counts: two keys at 9, then four keys at 7 spread over the shards: the two 9s
    are taken outright, three of the 7s in rank order (shard 0 has one, shard 1 two, shard 2 one -> 1, 2, 0)."""
    from pariskv_b200 import dist as pkd
    h = torch.zeros(3, 1, 1, 256, dtype=torch.int32)
    h[0, 0, 0, 9], h[0, 0, 0, 7], h[0, 0, 0, 2] = 1, 1, 10
    h[1, 0, 0, 7], h[1, 0, 0, 1] = 2, 10
    h[2, 0, 0, 9], h[2, 0, 0, 7], h[2, 0, 0, 0] = 1, 1, 10
    got = [pkd.shard_candidate_plan(h, r, 5) for r in range(3)]
    assert [int(g[0]) for g in got] == [7, 7, 7]
    assert [int(g[1]) for g in got] == [1, 2, 0]
    assert [int(g[2]) for g in got] == [2, 2, 1]
