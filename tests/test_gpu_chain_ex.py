"""GPU parity of pk_retrieve_ex: per-sample zone lengths read on the device, and the two-phase form for a zone cut
into shards (run here as W serial "ranks" on one GPU).  Both must reproduce the single-sequence, single-GPU chain
(itself checked against the oracle) bit for bit."""
import math

import pytest
import torch

from conftest import srht_signs, synth_keys, synth_queries

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

BOUNDS = (5000, 10000, 30000)
ROWS = [(0.5, 0.5), (0.25, 0.3), (0.2, 0.25), (0.1, 0.2)]
TIER_RATIOS = (0.05, 0.15, 0.30, 0.50, 0.75, 1.0)


def plan(N):
    """The reference's arithmetic on the host (cache_hub/polar_cache.py:1113-1124, :1221-1222, :1239-1240)."""
    cand, coll = ROWS[-1]
    for b, r in zip(BOUNDS, ROWS):
        if N < b:
            cand, coll = r
            break
    tiers = [int(math.ceil(N * coll * r)) for r in TIER_RATIOS]
    return tiers, max(1, int(math.ceil(N * cand))), coll


@pytest.fixture(scope="module")
def ops():
    from pariskv_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def schedule():
    from pariskv_b200 import _lib
    return _lib.zone_schedule(BOUNDS, [r[0] for r in ROWS], [r[1] for r in ROWS], TIER_RATIOS)


def test_device_plan_matches_host_arithmetic(schedule):
    """pk_zone_max_candidates is the maximum of the host formula over all shorter zones."""
    import ctypes
    from pariskv_b200 import _lib
    lib = _lib.load()
    for N in (1, 17, 4999, 5000, 9999, 10000, 29999, 30000, 131004, 1048508):
        want = max(plan(n)[1] for n in set([N] + [b - 1 for b in BOUNDS if b - 1 <= N]))
        assert lib.pk_zone_max_candidates(ctypes.byref(schedule), N) == want


@pytest.mark.parametrize("lens,K", [((4099, 33000, 9000), 256), ((700, 120, 4999), 64), ((31000, 31000), 2048),
                                    ((200000, 90000), 2048)])   # the last: candidate rows long enough for the separate top-K
def test_varlen_batch_equals_single_sequences_and_oracle(ops, oracle, schedule, lens, K):
    """A batch whose samples have different zone lengths (device i32 [bs]) gives, per sample, exactly what a batch-1
    call on that sample gives with host-side thresholds — and what the oracle gives."""
    g = torch.Generator().manual_seed(sum(lens))
    bs, H, Nmax = len(lens), 2, max(lens)
    keys = synth_keys(g, bs, H, Nmax)
    q = synth_queries(g, keys, 4)
    signs = srht_signs()
    _, cen = oracle.constants()
    counts = torch.zeros(bs, H, 16, 256, dtype=torch.int32, device=DEV)
    cb, w, pk = ops.alloc_key_metadata(bs, H, Nmax, DEV)
    for b, n in enumerate(lens):   # only the first n keys of sample b are searchable; the rest of the view is junk
        ops.encode_keys(keys[b:b + 1, :, :n].to(DEV), signs.to(DEV), cb[b:b + 1, :, :, :n], w[b:b + 1, :, :, :n],
                        pk[b:b + 1, :, :, :n, :], cluster_counts=counts[b:b + 1])
        cb[b, :, :, n:] = 255
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    import ctypes
    from pariskv_b200 import _lib
    Cmax = int(_lib.load().pk_zone_max_candidates(ctypes.byref(schedule), Nmax))
    fin, n_sel, ex = ops.retrieve_ex(q.to(DEV), signs.to(DEV), cen.to(DEV), cb, w, pk, counts, Cmax, K, kv_len=kv_len,
                                     schedule=schedule, want=("cand", "scores_f32"))
    for b, n in enumerate(lens):
        tiers, C, coll = plan(n)
        Kb = min(K, C)
        assert int(ex["n_cand"][b, 0]) == C and int(n_sel[b, 0]) == Kb
        one, ex1 = ops.retrieve(q[b:b + 1].to(DEV), signs.to(DEV), cen.to(DEV), cb[b:b + 1, :, :, :n], w[b:b + 1, :, :, :n],
                                pk[b:b + 1, :, :, :n, :], counts[b:b + 1], tiers, C, Kb, want=("cand", "scores_f32"))
        assert torch.equal(ex["cand"][b, :, :C], ex1["cand"][0])
        assert torch.equal(ex["scores_f32"][b, :, :C], ex1["scores_f32"][0])
        assert torch.equal(fin[b, :, :Kb], one[0])
        kb = keys[b:b + 1, :, :n].contiguous()
        cb_o, w_o, pk_o = oracle.encode(kb, signs)
        ref = oracle.retrieve(q[b:b + 1], signs, cb_o, w_o, pk_o, oracle.cluster_counts(cb_o), cen, coll, C, Kb)
        assert torch.equal(fin[b, :, :Kb].cpu(), ref["final"][0])


@pytest.mark.parametrize("N,K,world", [(40000, 512, 4), (9001, 256, 3), (131004, 2048, 8), (400000, 2048, 2),
                                       (300000, 1024, 3)])   # the last two: shard rows beyond the in-block final stage
def test_sharded_phases_reproduce_single_gpu_selection(ops, oracle, N, K, world):
    """W contiguous shards, each run through phase 1 / phase 2 with the gathered histograms: the union of the shards'
    candidate lists IS the single-GPU candidate list, and the top-K of the shards' local top lists IS the single-GPU
    final selection."""
    g = torch.Generator().manual_seed(N + world)
    H = 2
    keys = synth_keys(g, 1, H, N)
    q = synth_queries(g, keys, 4).to(DEV)
    signs = srht_signs().to(DEV)
    _, cen = oracle.constants()
    cen = cen.to(DEV)
    counts = torch.zeros(1, H, 16, 256, dtype=torch.int32, device=DEV)
    cb, w, pk = ops.encode_keys(keys.to(DEV), signs, cluster_counts=counts)
    tiers, C, _ = plan(N)
    ref_fin, ref_ex = ops.retrieve(q, signs, cen, cb, w, pk, counts, tiers, C, K, want=("cand", "scores_f32"))
    per = (N + world - 1) // world
    shards = [(min(N, r * per), min(N, (r + 1) * per)) for r in range(world)]
    scratch, outs, hists = [], [], []
    for r, (s, e) in enumerate(shards):
        n = e - s
        scratch.append(ops.Scratch(DEV, ops.retrieve_scratch_bytes(1, H, n, min(C, n))))
        outs.append({"cand": torch.empty(1, H, min(C, n), dtype=torch.int64, device=DEV),
                     "scores_f32": torch.empty(1, H, min(C, n), dtype=torch.float32, device=DEV)})
        _, _, ex = ops.retrieve_ex(q, signs, cen, cb[:, :, :, s:e], w[:, :, :, s:e], pk[:, :, :, s:e, :], counts, C, K,
                                   tier_counts=tiers, phase=1, outputs=outs[r], scratch=scratch[r])
        hists.append(ex["local_hist"])
    shard_hist = torch.stack(hists).contiguous()      # what the all-gather delivers: [world,1,H,256]
    assert int(shard_hist.sum()) == H * N
    cand_all, score_all, top_idx, top_score = [[] for _ in range(H)], [[] for _ in range(H)], [[] for _ in range(H)], [[] for _ in range(H)]
    for r, (s, e) in enumerate(shards):
        fin, n_sel, ex = ops.retrieve_ex(q, signs, cen, cb[:, :, :, s:e], w[:, :, :, s:e], pk[:, :, :, s:e, :], counts, C, K,
                                         tier_counts=tiers, phase=2, shard_hist=shard_hist, world=world, rank=r,
                                         outputs=outs[r], scratch=scratch[r])
        for h in range(H):
            nc, ns = int(ex["n_cand"][0, h]), int(n_sel[0, h])
            assert ns == min(K, nc)
            cand_all[h].append(ex["cand"][0, h, :nc] + s)
            score_all[h].append(ex["scores_f32"][0, h, :nc])
            loc = fin[0, h, :ns]
            pos = torch.searchsorted(ex["cand"][0, h, :nc].contiguous(), loc)
            top_idx[h].append(loc + s)
            top_score[h].append(ex["scores_f32"][0, h, :nc][pos])
    for h in range(H):
        assert torch.equal(torch.cat(cand_all[h]), ref_ex["cand"][0, h]), "union of shard candidates != single-GPU set"
        assert torch.equal(torch.cat(score_all[h]), ref_ex["scores_f32"][0, h])
        idx, sc = torch.cat(top_idx[h]), torch.cat(top_score[h])
        merged = ops.final_topk(sc.view(1, 1, -1).contiguous(), idx.view(1, 1, -1).contiguous(), K)
        assert torch.equal(merged[0, 0], ref_fin[0, h]), "merged local top lists != single-GPU final selection"


def test_bench_shape_against_oracle(ops, oracle):
    """The exact shape of the headline benchmark: 8 KV heads x 131004 keys, C = 13101, K = 2048."""
    g = torch.Generator().manual_seed(77)
    H, N = 8, 131004
    keys = synth_keys(g, 1, H, N)
    q = synth_queries(g, keys, 4)
    signs = srht_signs()
    _, cen = oracle.constants()
    tiers, C, coll = plan(N)
    assert C == 13101
    cb_o, w_o, pk_o = oracle.encode(keys, signs)
    ref = oracle.retrieve(q, signs, cb_o, w_o, pk_o, oracle.cluster_counts(cb_o), cen, coll, C, 2048)
    counts = torch.zeros(1, H, 16, 256, dtype=torch.int32, device=DEV)
    cb, w, pk = ops.encode_keys(keys.to(DEV), signs.to(DEV), cluster_counts=counts)
    assert torch.equal(cb.cpu(), cb_o)
    fin, ex = ops.retrieve(q.to(DEV), signs.to(DEV), cen.to(DEV), cb, w, pk, counts, tiers, C, 2048,
                           want=("cand", "scores_f32"))
    assert torch.equal(ex["cand"].cpu(), ref["cand"])
    assert torch.equal(ex["scores_f32"].cpu(), ref["score32"])
    assert torch.equal(fin.cpu(), ref["final"])


def test_final_selection_with_ties_and_flat_scores(ops):
    """The fused final top-K on degenerate score rows: candidates whose records are identical get identical scores, so
    the selection is decided by position alone (lowest key index first)."""
    H, N, C, K = 1, 6000, 3000, 700
    signs = srht_signs().to(DEV)
    g = torch.Generator().manual_seed(5)
    one = synth_keys(g, 1, H, 1)
    keys = one.expand(1, H, N, 128).contiguous()          # every key the same: all counts and all scores tie
    q = synth_queries(g, keys, 4).to(DEV)
    cen = torch.tensor([0.0420, 0.1266, 0.2130, 0.3025, 0.3973, 0.5001, 0.6169, 0.7633], dtype=torch.bfloat16, device=DEV)
    counts = torch.zeros(1, H, 16, 256, dtype=torch.int32, device=DEV)
    cb, w, pk = ops.encode_keys(keys.to(DEV), signs, cluster_counts=counts)
    tiers, _, _ = plan(N)
    fin, ex = ops.retrieve(q, signs, cen, cb, w, pk, counts, tiers, C, K, want=("cand", "scores_f32"))
    assert torch.equal(ex["cand"][0, 0].cpu(), torch.arange(C))
    assert torch.equal(fin[0, 0].cpu(), torch.arange(K))
    assert float(ex["scores_f32"].max() - ex["scores_f32"].min()) == 0.0


def test_early_query_preparation_gives_the_same_chain(ops, schedule):
    """queries_settled only moves the query preparation and the cluster sort ahead of the kernel's dependency wait:
    candidates, scores and final indices are bit-identical, with dependent launch on or off."""
    from pariskv_b200 import _lib
    g = torch.Generator().manual_seed(404)
    lens = (33000, 12000)
    bs, H, Nmax = len(lens), 2, max(lens)
    keys = synth_keys(g, bs, H, Nmax)
    q = synth_queries(g, keys, 4).to(DEV)
    signs = srht_signs().to(DEV)
    cen = torch.tensor([0.0420, 0.1266, 0.2130, 0.3025, 0.3973, 0.5001, 0.6169, 0.7633], dtype=torch.bfloat16, device=DEV)
    counts = torch.zeros(bs, H, 16, 256, dtype=torch.int32, device=DEV)
    cb, w, pk = ops.alloc_key_metadata(bs, H, Nmax, DEV)
    for b, n in enumerate(lens):
        ops.encode_keys(keys[b:b + 1, :, :n].to(DEV), signs, cb[b:b + 1, :, :, :n], w[b:b + 1, :, :, :n],
                        pk[b:b + 1, :, :, :n, :], cluster_counts=counts[b:b + 1])
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    import ctypes
    Cmax = int(_lib.load().pk_zone_max_candidates(ctypes.byref(schedule), Nmax))
    outs = []
    try:
        for pdl in (False, True):
            _lib.set_pdl(pdl)
            for settled in (False, True):
                fin, n_sel, ex = ops.retrieve_ex(q, signs, cen, cb, w, pk, counts, Cmax, 512, kv_len=kv_len,
                                                 schedule=schedule, want=("cand", "scores_f32", "q_blocks", "q_norm"),
                                                 queries_settled=settled)
                outs.append((fin.clone(), n_sel.clone(), ex["cand"].clone(), ex["scores_f32"].clone(),
                             ex["q_blocks"].clone(), ex["q_norm"].clone()))
    finally:
        _lib.set_pdl(False)
    for o in outs[1:]:
        for a, b in zip(outs[0], o):
            assert torch.equal(a, b)
