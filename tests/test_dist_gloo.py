"""World-size-2 tests of the multi-GPU plumbing with gloo ranks on CPU: the exchange of local top lists, the
partial-attention merge and the histogram all-reduce of the sequence-sharded form, against the same sharded
formulation evaluated in one process by the oracle."""
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


def _shard_result(O, rank, world, keys, vals, q, signs, cen, coll, cand_ratio, K, counts_global, span=None):
    """One rank's part of the sharded formulation on the CPU; span = (start, end) when the chunks are not the equal
    split (after flushes the last chunk has grown)."""
    from pariskv_b200 import dist as pkd
    N = keys.shape[2]
    start, end = span if span is not None else pkd.sequence_shard(N, rank, world)
    tiers, c_local, k_local = pkd.local_plan(N, world, coll, cand_ratio, K)
    cb, w, pk = O.encode(keys[:, :, start:end].contiguous(), signs)
    H = keys.shape[1]
    qb, qn = O.query_prep(q, H, signs)
    ids = O.cluster_rank(qb)
    cnt = O.collision(ids, counts_global, cb, tiers)
    cand = O.topk(cnt, c_local)
    s32, _ = O.rerank(cand, pk, w, qb, qn, cen)
    loc = O.final_topk(s32, cand, k_local)
    sc = torch.gather(s32, 2, torch.searchsorted(cand, loc))
    return sc, loc + start, (start, end), (cb,)


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
        # local chain, exchange, global selection
        sc, gi, _, _ = _shard_result(O, rank, world, keys, vals, q, signs, cen, coll, cand_ratio, K, counts)
        final = pkd.merge_local_topk(sc, gi, K, select=_oracle_select)
        # the same formulation evaluated serially
        parts = [_shard_result(O, r, world, keys, vals, q, signs, cen, coll, cand_ratio, K, counts) for r in range(world)]
        want = O.final_topk(torch.cat([p[0] for p in parts], -1), torch.cat([p[1] for p in parts], -1), K)
        assert torch.equal(final, want)
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
    tiers, c_local, k_local = pkd.local_plan(1048508, 8, 0.2, 0.1, 2048)
    assert c_local == -(-104851 // 8) and k_local == 2048 and tiers[-1] == 209702


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
    tiers, c_local, k_local = pkd.local_plan(32768, 1, 0.2, 4096 / 32768, 256)
    assert tiers == want and c_local == 4096 and k_local == 256
    # per-shard budgets: ceil of the global candidate count over the ranks, the final K capped by it
    assert pkd.local_plan(32768, 4, 0.2, 4096 / 32768, 2048)[1:] == (1024, 1024)
