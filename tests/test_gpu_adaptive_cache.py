"""The two adaptive-k cache variants against the oracle: the selection (adaptive_k, benefit-ordered indices)
must be bit-exact given the same logits and candidate scores; the attention output within bf16 tolerance."""
import pytest
import torch

from conftest import synth_keys

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(kind, P, bs, H, Hq, sink, local, I, **extra):
    if kind == "dense":
        from pariskv_b200.cache_hub.polar_cache_atten_value_indices_adaptive_k import polar_cache
    else:
        from pariskv_b200.cache_hub.polar_cache_adaptivek_varlen import polar_cache
    return polar_cache(valid_start=[0] * bs, layer_num=1, batch_size=bs, max_length=P + 64, num_key_value_heads=H,
                       num_heads=Hq, head_dim=128, dtype=torch.bfloat16, layer_mapping={"0": DEV}, max_new_length=64,
                       sink_size=sink, local_size=local, core=0, nprobe=0, cache_unit_size=0, cache_cluster_num=0,
                       num_gpus=1, model_size=8, final_topk=64, dynamic_update_interval=I, enable_offload=True, **extra)


@pytest.mark.parametrize("kind,extra", [("dense", dict(adaptive_topk_threshold=0.9, adaptive_topk_max_k=256)),
                                        ("varlen", dict(adaptive_topk_threshold=0.85, adaptive_topk_min_k=20,
                                                        adaptive_topk_max_k=200))])
@pytest.mark.parametrize("bs", [1, 3])
def test_adaptive_cache_matches_oracle(oracle, kind, extra, bs):
    g = torch.Generator().manual_seed(5 + bs)
    H, Hq, sink, local, I, P, steps = 2, 8, 4, 16, 8, 2400, 11
    cache = _make(kind, P, bs, H, Hq, sink, local, I, **extra)
    K = synth_keys(g, bs, H, P)
    V = (torch.randn(bs, H, P, 128, generator=g) * torch.exp(0.5 * torch.randn(bs, H, P, 1, generator=g))).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    for t in range(steps):
        nk = synth_keys(g, bs, H, 1)
        nv = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
        K, V = torch.cat([K, nk], 2), torch.cat([V, nv], 2)
        cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), 0)
        # queries aligned with a few cached keys so the benefit mass is concentrated
        pick = torch.randint(sink, P - local, (bs, H), generator=g)
        qk = torch.stack([torch.stack([K[b, h, pick[b, h]].float() for h in range(H)]) for b in range(bs)])
        q = (qk / qk.norm(dim=-1, keepdim=True) * 6.0).unsqueeze(2).expand(bs, H, Hq // H, 128)
        q = (q + 0.3 * torch.randn(bs, H, Hq // H, 128, generator=g)).reshape(bs, 1, Hq, 128).to(torch.bfloat16)
        out = cache.compute(q.to(DEV), 0)
        ak, topk, n_sel, sl_logits, cand, cand_scores = cache.last_adaptive
        f = (t + 1) // I
        zone_end = P - local + f * I
        N = zone_end - sink
        assert cache.cpu_valid_end[0] == N
        # value norms tracked by the cache equal the norms of the tokens in the zone / window
        vn = torch.linalg.vector_norm(V.float(), dim=-1)
        assert torch.allclose(cache.value_norm_gpu[0][:, :, :N].cpu(), vn[:, :, sink:zone_end], rtol=1e-6)
        win_idx = list(range(sink)) + list(range(zone_end, K.shape[2]))
        n_win = len(win_idx)
        assert torch.allclose(cache._sl_vnorm_cache[0][:, :, :n_win].cpu(), vn[:, :, win_idx], rtol=1e-6)
        # the candidate stage equals the oracle's
        zk, zv = K[:, :, sink:zone_end].contiguous(), V[:, :, sink:zone_end].contiguous()
        signs = cache.srht_diagonal_signs.cpu()
        cb, w, pk = oracle.encode(zk, signs)
        tiers, C, _ = cache.retrieval_plan(N)
        _, coll = cache._get_adaptive_ratios(N)
        r = oracle.retrieve(q, signs, cb, w, pk, oracle.cluster_counts(cb), cache._mag_centers.cpu(), coll, C, 1)
        assert torch.equal(cand.cpu(), r["cand"])
        assert torch.equal(cand_scores.cpu().view(torch.int16), r["score_bf16"].view(torch.int16))
        # adaptive selection: same inputs into the oracle -> same k and same order
        K_out = min(cache._max_k, C)
        scale = cache._attn_scale
        cl = (cand_scores.float().cpu().numpy() * torch.tensor(scale, dtype=torch.float32).numpy())
        cvn = torch.gather(vn[:, :, sink:zone_end], 2, r["cand"])
        k_o, idx_o = oracle.adaptive_topk(sl_logits.cpu(), vn[:, :, win_idx].float(), torch.from_numpy(cl), cvn,
                                          r["cand"], cache.adaptive_topk_threshold, K_out)
        k_o = k_o.clamp(max(1, min(cache._min_k, K_out)), K_out)
        assert torch.equal(ak.cpu(), k_o), (t, ak.cpu().tolist(), k_o.tolist())
        assert torch.equal(topk.cpu(), idx_o)
        want_n = k_o if kind == "varlen" else k_o.max().expand_as(k_o)
        assert torch.equal(n_sel.cpu().long(), want_n)
        # attention over window + the per-head prefixes
        for b in range(bs):
            for h in range(H):
                n = int(want_n[b, h])
                sb, sh = slice(b, b + 1), slice(h, h + 1)
                kk = torch.cat([K[sb, sh][:, :, win_idx], oracle.gather(zk[sb, sh], idx_o[sb, sh, :n])], 2)
                vv = torch.cat([V[sb, sh][:, :, win_idx], oracle.gather(zv[sb, sh], idx_o[sb, sh, :n])], 2)
                g0, g1 = h * (Hq // H), (h + 1) * (Hq // H)
                ref = oracle.attention(q[sb, :, g0:g1], kk, vv)
                # bf16 output: 2e-2 absolute for outputs of order one; the values here carry a lognormal scale, so
                # allow half a bf16 step (2^-8 relative) of the largest output as well
                tol = max(2e-2, ref.abs().max().item() * 2.0 ** -8)
                assert (out[sb, :, g0:g1].float().cpu() - ref).abs().max().item() <= tol, (t, b, h)
    assert cache.cpu_valid_end[0] == P - sink - local + I


@pytest.mark.parametrize("kind,extra", [("dense", dict(adaptive_topk_threshold=0.9, adaptive_topk_max_k=256)),
                                        ("varlen", dict(adaptive_topk_threshold=0.85, adaptive_topk_min_k=20,
                                                        adaptive_topk_max_k=200))])
def test_adaptive_cache_replays_under_one_graph(kind, extra):
    """Append + adaptive compute captured ONCE and replayed over a flush of the update buffer gives, step for step, the
    rows (per-head counts, benefit order) and the attention output of eager stepping on a twin cache: inside a capture
    every shape is a capacity and the lengths act through device words only."""
    g = torch.Generator().manual_seed(11)
    bs, H, Hq, sink, local, I, P, steps = 2, 2, 8, 4, 16, 8, 2400, 19
    twins = [_make(kind, P, bs, H, Hq, sink, local, I, **extra) for _ in range(2)]
    K = synth_keys(g, bs, H, P)
    V = (torch.randn(bs, H, P, 128, generator=g) * torch.exp(0.5 * torch.randn(bs, H, P, 1, generator=g))).to(torch.bfloat16)
    for c in twins:
        c.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    eager, graphed = twins
    k_in = torch.zeros(bs, 1, H, 128, dtype=torch.bfloat16, device=DEV)
    v_in = torch.zeros_like(k_in)
    q_in = torch.zeros(bs, 1, Hq, 128, dtype=torch.bfloat16, device=DEV)
    graph, out_g, captured = None, None, 0
    for t in range(steps):
        nk = synth_keys(g, bs, H, 1).transpose(1, 2).contiguous()
        nv = torch.randn(bs, 1, H, 128, generator=g).to(torch.bfloat16)
        pick = torch.randint(sink, P - local, (bs, H), generator=g)
        qk = torch.stack([torch.stack([K[b, h, pick[b, h]].float() for h in range(H)]) for b in range(bs)])
        q = (qk / qk.norm(dim=-1, keepdim=True) * 6.0).unsqueeze(2).expand(bs, H, Hq // H, 128)
        q = (q + 0.3 * torch.randn(bs, H, Hq // H, 128, generator=g)).reshape(bs, 1, Hq, 128).to(torch.bfloat16)
        k_in.copy_(nk), v_in.copy_(nv), q_in.copy_(q)
        eager.decode_update_kv_cache(k_in, v_in, 0)
        want = eager.compute(q_in, 0).clone()
        ak_e, topk_e, nsel_e = (x.clone() for x in eager.last_adaptive[:3])
        if t < 2:      # first steps eagerly on both (first-use set-up outside the capture)
            graphed.decode_update_kv_cache(k_in, v_in, 0)
            got = graphed.compute(q_in, 0)
        else:
            if graph is None:
                torch.cuda.synchronize()
                saved = graphed.host_state()
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    graph.capture_begin()
                    graphed.decode_update_kv_cache(k_in, v_in, 0)
                    out_g = graphed.compute(q_in, 0)
                    graph.capture_end()
                torch.cuda.current_stream().wait_stream(side)
                graphed.set_host_state(saved)   # the capture ran the host bookkeeping of one step without executing it
                captured += 1
            graph.replay()
            graphed.note_replayed_step()
            got = out_g
        ak_g, topk_g, nsel_g = graphed.last_adaptive[:3]
        assert torch.equal(nsel_g, nsel_e), t
        for b in range(bs):
            for h in range(H):
                n = int(nsel_e[b, h])
                assert torch.equal(topk_g[b, h, :n], topk_e[b, h, :n]), (t, b, h)
        assert torch.equal(got, want), t
    assert captured == 1 and eager.cpu_valid_end[0] > P - local - sink      # at least one flush was replayed
