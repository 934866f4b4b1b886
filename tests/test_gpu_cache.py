"""The cache class (prefill, append, flush, retrieval, attention) against a plain state machine built from
the oracle: the searchable zone is token positions [sink, P - local + f*I), the window is the sink rows plus
everything newer (reference invariants: cache_hub/polar_cache.py:645-699, :743-881, :1002-1107)."""
import pytest
import torch

from conftest import synth_keys

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make_cache(P, max_new, bs, H, Hq, sink, local, I, topk, offload, layers=2, thr=2000):
    from pariskv_b200.cache_hub.polar_cache import polar_cache
    return polar_cache(valid_start=[0] * bs, layer_num=layers, batch_size=bs, max_length=P + max_new,
                       num_key_value_heads=H, num_heads=Hq, head_dim=128, dtype=torch.bfloat16,
                       layer_mapping={str(i): DEV for i in range(layers)}, max_new_length=max_new, sink_size=sink,
                       local_size=local, core=0, nprobe=0, cache_unit_size=0, cache_cluster_num=0, num_gpus=1,
                       model_size=8, final_topk=topk, dynamic_update_interval=I, full_attention_threshold=thr,
                       enable_offload=offload)


def _oracle_step(oracle, cache, q, K_all, V_all, zone_end, layer):
    """K_all / V_all: every token so far [bs,H,T,128] (CPU).  Returns (attention fp32, final indices or None)."""
    sink = cache.sink_size
    T = K_all.shape[2]
    N = max(0, zone_end - sink)
    signs = cache.srht_diagonal_signs.cpu()
    win_idx = list(range(min(sink, T))) + list(range(max(zone_end, sink), T)) if N > 0 else list(range(T))
    wk, wv = K_all[:, :, win_idx], V_all[:, :, win_idx]
    full = T < max(cache.FULL_ATTENTION_THRESHOLD, cache.steady_size + 2 * cache.final_topk) or N <= 0
    if full:
        if N > 0:
            wk = torch.cat([wk, K_all[:, :, sink:zone_end]], 2)
            wv = torch.cat([wv, V_all[:, :, sink:zone_end]], 2)
        return oracle.attention(q, wk, wv), None
    zk, zv = K_all[:, :, sink:zone_end].contiguous(), V_all[:, :, sink:zone_end].contiguous()
    cb, w, pk = oracle.encode(zk, signs)
    tiers, C, K = cache.retrieval_plan(N)
    _, coll = cache._get_adaptive_ratios(N)
    assert tiers == oracle.tier_counts(N, coll)
    r = oracle.retrieve(q, signs, cb, w, pk, oracle.cluster_counts(cb), cache._mag_centers.cpu(), coll, C, K)
    att = oracle.attention(q, torch.cat([wk, oracle.gather(zk, r["final"])], 2),
                           torch.cat([wv, oracle.gather(zv, r["final"])], 2))
    return att, r["final"]


@pytest.mark.parametrize("offload", [True, False])
def test_cache_decode_matches_state_machine(oracle, offload):
    g = torch.Generator().manual_seed(7)
    bs, H, Hq, sink, local, I, topk, P, steps, layers = 2, 2, 8, 4, 16, 8, 32, 2100, 19, 2
    cache = _make_cache(P, 64, bs, H, Hq, sink, local, I, topk, offload, layers)
    Ks = [synth_keys(g, bs, H, P) for _ in range(layers)]
    Vs = [torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16) for _ in range(layers)]
    for l in range(layers):  # lockstep prefill: [bs, seq, H, 128]
        k_in, v_in = Ks[l].transpose(1, 2).contiguous().to(DEV), Vs[l].transpose(1, 2).contiguous().to(DEV)
        rk, rv = cache.prefill_update_kv_cache(None, k_in, v_in, l, 0)
        assert rk.shape == k_in.shape
    assert cache.context == P and cache.cpu_valid_end == [P - sink - local] * layers
    flushed = 0
    for t in range(steps):
        for l in range(layers):
            nk = synth_keys(g, bs, H, 1)
            nv = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
            Ks[l] = torch.cat([Ks[l], nk], 2)
            Vs[l] = torch.cat([Vs[l], nv], 2)
            cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), l)
            q = (torch.randn(bs, 1, Hq, 128, generator=g) * 0.5).to(torch.bfloat16)
            out = cache.compute(q.to(DEV), l)
            f = (t + 1) // I
            zone_end = P - local + f * I
            ref, fin = _oracle_step(oracle, cache, q, Ks[l], Vs[l], zone_end, l)
            assert cache.cpu_valid_end[l] == zone_end - sink
            assert torch.equal(cache.last_topk_indices.cpu(), fin), f"step {t} layer {l}: retrieved set differs"
            err = (out.float().cpu() - ref).abs().max().item()
            assert err <= 2e-2, (t, l, err)
        flushed = (t + 1) // I
    assert flushed == 2 and cache.context == P + steps
    # metadata of the flushed keys equals a fresh encode of the same token positions
    zone = Ks[0][:, :, sink:P - local + 2 * I].contiguous()
    cb, w, pk = oracle.encode(zone, cache.srht_diagonal_signs.cpu())
    N = zone.shape[2]
    assert torch.equal(cache.codebook_gpu[0][:, :, :, :N].cpu(), cb)
    assert torch.equal(cache.key_4bit_packed_gpu[0][:, :, :, :N].cpu(), pk)
    assert torch.equal(cache.cluster_key_counts_gpu[0].cpu(), oracle.cluster_counts(cb))


def test_cache_short_prompt_dense_path(oracle):
    g = torch.Generator().manual_seed(3)
    bs, H, Hq, sink, local, I, topk = 1, 2, 8, 4, 8, 4, 16
    cache = _make_cache(10, 40, bs, H, Hq, sink, local, I, topk, True, layers=1)
    K = synth_keys(g, bs, H, 10)
    V = torch.randn(bs, H, 10, 128, generator=g).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    for t in range(14):  # crosses steady (12) and two flushes of 4
        nk, nv = synth_keys(g, bs, H, 1), torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
        K, V = torch.cat([K, nk], 2), torch.cat([V, nv], 2)
        cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), 0)
        q = torch.randn(bs, 1, Hq, 128, generator=g).to(torch.bfloat16)
        out = cache.compute(q.to(DEV), 0)
        ref = oracle.attention(q, K, V)  # short context: dense attention over every token
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2, t
    assert cache.cpu_valid_end[0] == 12 and cache._window_len[0] == 12


def test_dropin_names_resolve():
    import pariskv_b200.dropin as dropin
    dropin.install(force=True)
    from attn_hub import polar_decode_attn, polar_prefill_attn  # noqa: F401
    from cache_hub.polar_cache import polar_cache
    assert polar_cache.__module__ == "pariskv_b200.cache_hub.polar_cache"
    from cache_hub.topk import load_radix_topk_ext
    x = torch.randint(0, 97, (1, 2, 500), dtype=torch.int32, device=DEV)
    idx = load_radix_topk_ext().radix_topk_3d(x, 50)
    assert idx.shape == (1, 2, 50) and idx.dtype == torch.int64
    q = torch.randn(1, 5, 8, 128, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(1, 5, 2, 128, device=DEV, dtype=torch.bfloat16)
    out = polar_prefill_attn(q, k, k, causal=True)
    assert out.shape == q.shape


def test_cache_step_replayed_as_cuda_graph_matches_eager(oracle):
    """The append + retrieval + attention of a layer captured once and replayed: the window position is read
    on the device, so every replay must give the bits of the eager run."""
    g = torch.Generator().manual_seed(21)
    bs, H, Hq, sink, local, I, topk, P, layers = 1, 2, 8, 4, 16, 16, 32, 2300, 1
    K0 = synth_keys(g, bs, H, P)
    V0 = torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16)
    caches = [_make_cache(P, 64, bs, H, Hq, sink, local, I, topk, True, layers) for _ in range(2)]
    for c in caches:
        c.prefill_update_kv_cache(None, K0.transpose(1, 2).contiguous().to(DEV), V0.transpose(1, 2).contiguous().to(DEV), 0, 0)
    eager, graphed = caches
    k_s = torch.zeros(bs, 1, H, 128, dtype=torch.bfloat16, device=DEV)
    v_s = torch.zeros_like(k_s)
    q_s = torch.zeros(bs, 1, Hq, 128, dtype=torch.bfloat16, device=DEV)
    out_s = torch.zeros_like(q_s)
    # one eager step on both first (creates workspaces outside the capture)
    steps = []
    for t in range(10):
        steps.append((synth_keys(g, bs, H, 1).transpose(1, 2).contiguous(),
                      torch.randn(bs, 1, H, 128, generator=g).to(torch.bfloat16),
                      (torch.randn(bs, 1, Hq, 128, generator=g) * 0.5).to(torch.bfloat16)))
    refs = []
    for k, v, q in steps:
        eager.decode_update_kv_cache(k.to(DEV), v.to(DEV), 0)
        refs.append(eager.compute(q.to(DEV), 0).clone())
    k, v, q = steps[0]
    graphed.decode_update_kv_cache(k.to(DEV), v.to(DEV), 0)
    assert torch.equal(graphed.compute(q.to(DEV), 0), refs[0])
    graphed.device_positions = True
    graphed.sync_device_state()
    saved = graphed.host_state()
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        graphed.decode_update_kv_cache(k_s, v_s, 0)
        out_s.copy_(graphed.compute(q_s, 0))
        graphed.advance_device_step()
    graphed.set_host_state(saved)
    for t in range(1, 10):
        assert not graphed.next_step_flushes()
        k, v, q = steps[t]
        k_s.copy_(k)
        v_s.copy_(v)
        q_s.copy_(q)
        gr.replay()
        graphed.note_replayed_step()
        torch.cuda.synchronize()
        assert torch.equal(out_s, refs[t]), f"replay {t} differs from the eager step"
    assert graphed.host_state() == eager.host_state()


def test_bulk_offload_on_copy_stream(oracle):
    """A prompt long enough for the copy-stream offload: the store holds exactly the zone rows (K and V interleaved),
    and a decode step issued right after the prefill (no host synchronisation) sees them."""
    g = torch.Generator().manual_seed(17)
    bs, H, Hq, sink, local, I, topk, P, layers = 1, 2, 8, 4, 16, 8, 32, 6000, 2
    cache = _make_cache(P, 32, bs, H, Hq, sink, local, I, topk, True, layers)
    assert cache.BULK_OFFLOAD_ROWS <= P - sink - local
    Ks = [synth_keys(g, bs, H, P) for _ in range(layers)]
    Vs = [torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16) for _ in range(layers)]
    for l in range(layers):
        cache.prefill_update_kv_cache(None, Ks[l].transpose(1, 2).contiguous().to(DEV),
                                      Vs[l].transpose(1, 2).contiguous().to(DEV), l, 0)
        assert cache._offload_event[l] is not None
    outs, fins = [], []
    qs = [torch.randn(bs, 1, Hq, 128, generator=g).to(torch.bfloat16) for _ in range(layers)]
    nk = torch.randn(bs, 1, H, 128, generator=g).to(torch.bfloat16)
    nv = torch.randn(bs, 1, H, 128, generator=g).to(torch.bfloat16)
    for l in range(layers):           # straight after the prefill: ordering comes from the layer's event
        cache.decode_update_kv_cache(nk.to(DEV), nv.to(DEV), l)
        outs.append(cache.compute(qs[l].to(DEV), l))
        fins.append(cache.last_topk_indices)
        assert cache._offload_event[l] is None
    torch.cuda.synchronize()
    N = P - sink - local
    for l in range(layers):
        assert torch.equal(cache.unified_keys_cpu[l][:, :, :N], Ks[l][:, :, sink:sink + N])
        assert torch.equal(cache.unified_values_cpu[l][:, :, :N], Vs[l][:, :, sink:sink + N])
        K_all = torch.cat([Ks[l], nk.transpose(1, 2)], 2)
        V_all = torch.cat([Vs[l], nv.transpose(1, 2)], 2)
        att, fin = _oracle_step(oracle, cache, qs[l], K_all, V_all, P - local, l)
        assert torch.equal(fins[l].cpu(), fin)
        assert (outs[l].float().cpu() - att).abs().max().item() <= 2e-2


def test_long_generation_with_drifting_keys_one_kv_head(oracle):
    """One KV head per rank (the tensor-parallel split of an 8-KV-head model over 8 GPUs needs no collective on this
    path), batch 2, a generation that crosses six flushes, appended keys drawn around a mean direction that rotates:
    every step's retrieved set and attention output against the oracle's state machine, and at the end the coded
    zone against a fresh encode of the same token positions."""
    from pariskv_b200 import dist as pkd
    assert pkd.head_shard(8, 3, 8) == slice(3, 4)
    g = torch.Generator().manual_seed(23)
    bs, H, Hq, sink, local, I, topk, P, steps = 2, 1, 8, 4, 16, 8, 32, 2300, 50
    cache = _make_cache(P, 64, bs, H, Hq, sink, local, I, topk, True, 1)
    Ks = synth_keys(g, bs, H, P)
    Vs = torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, Ks.transpose(1, 2).contiguous().to(DEV), Vs.transpose(1, 2).contiguous().to(DEV), 0, 0)
    a = torch.randn(128, generator=g)
    b = torch.randn(128, generator=g)
    a, b = a / a.norm(), b - (b @ a) * a / (a @ a)
    b = b / b.norm()
    for t in range(steps):
        theta = 0.05 * t                         # the mean direction turns in the (a, b) plane
        mean = (torch.cos(torch.tensor(theta)) * a + torch.sin(torch.tensor(theta)) * b) * 12.0
        nk = (mean + torch.randn(bs, H, 1, 128, generator=g)).to(torch.bfloat16)
        nv = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
        Ks, Vs = torch.cat([Ks, nk], 2), torch.cat([Vs, nv], 2)
        cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), 0)
        q = ((mean / 12.0) * 0.5 + torch.randn(bs, 1, Hq, 128, generator=g) * 0.3).to(torch.bfloat16)
        out = cache.compute(q.to(DEV), 0)
        zone_end = P - local + ((t + 1) // I) * I
        ref, fin = _oracle_step(oracle, cache, q, Ks, Vs, zone_end, 0)
        assert torch.equal(cache.last_topk_indices.cpu(), fin), f"step {t}: retrieved set differs"
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2, t
    assert cache.cpu_valid_end[0] == P - sink - local + 6 * I and cache.context == P + steps
    zone = Ks[:, :, sink:P - local + 6 * I].contiguous()
    cb, w, pk = oracle.encode(zone, cache.srht_diagonal_signs.cpu())
    N = zone.shape[2]
    assert torch.equal(cache.codebook_gpu[0][:, :, :, :N].cpu(), cb)
    assert torch.equal(cache.key_4bit_packed_gpu[0][:, :, :, :N].cpu(), pk)
    assert torch.equal(cache.cluster_key_counts_gpu[0].cpu(), oracle.cluster_counts(cb))


@pytest.mark.parametrize("pdl", [False, True])
def test_graphed_decoder_with_precaptured_graphs_matches_eager(pdl):
    """bench.GraphedDecoder: ONE captured graph replayed across three flushes of the update buffer (the flush runs
    inside the append launch, all positions are device words) must produce the same tokens as plain eager stepping
    (same weights, same cache content).  With programmatic dependent launch on, every kernel of the step may start
    under the tail of its predecessor, captured and eager alike; the tokens must not change."""
    import bench
    from pariskv_b200 import _lib
    _lib.set_pdl(False)
    cfg = dict(layers=2, hidden=256, q_heads=8, kv_heads=2, head_dim=128, ffn=512, vocab=997, rope_theta=1.0e6,
               context=2600, sink=4, local=16, interval=8, topk=32)
    dev = torch.device(DEV)
    model = bench.DecoderHarness(cfg, dev, seed=5)
    steps = 30

    def fresh():
        return bench.build_cache(cfg, dev, steps + 40, seed=9)

    cache = fresh()
    tok = torch.tensor([3], device=dev)
    eager = []
    for _ in range(steps):
        tok = model.step(cache, tok)
        eager.append(int(tok))
    assert cache.cpu_valid_end[0] == 2600 - 20 + 3 * 8

    cache = fresh()
    _lib.set_pdl(pdl)
    if pdl:      # eager stepping with dependent launch as well
        tok, again = torch.tensor([3], device=dev), []
        for _ in range(steps):
            tok = model.step(cache, tok)
            again.append(int(tok))
        assert again == eager
        cache = fresh()
    runner = bench.GraphedDecoder(model, cache)
    tok = torch.tensor([3], device=dev)
    got = []
    for _ in range(2):                  # eager first, as the benchmark does
        tok = model.step(cache, tok)
        got.append(int(tok))
    runner.tok.copy_(tok)
    runner.precapture(3)
    captured = runner.captures
    assert captured == 1, "one graph must serve every zone length"
    for _ in range(steps - 2):
        runner.step()
        got.append(int(runner.nxt))
    _lib.set_pdl(False)
    assert got == eager
    assert runner.captures == captured, "a graph was captured inside the run although all lengths were prepared"
    assert cache.cpu_valid_end[0] == 2600 - 20 + 3 * 8 and cache.context == 2600 + steps


def test_first_captured_graph_survives_later_captures_and_unrelated_allocations():
    """Scratch owned by the cache: the graph captured FIRST is replayed after graphs for longer zones were captured
    and after a few hundred MB of unrelated tensors were allocated, filled and freed.  Its tokens must be those of
    eager stepping, and the scratch addresses must not have moved."""
    import bench
    cfg = dict(layers=2, hidden=256, q_heads=8, kv_heads=2, head_dim=128, ffn=512, vocab=997, rope_theta=1.0e6,
               context=2600, sink=4, local=16, interval=8, topk=32)
    dev = torch.device(DEV)
    model = bench.DecoderHarness(cfg, dev, seed=6)
    cache = bench.build_cache(cfg, dev, 80, seed=10)
    tok = torch.tensor([5], device=dev)
    eager = []
    for _ in range(6):
        tok = model.step(cache, tok)
        eager.append(int(tok))
    cache = bench.build_cache(cfg, dev, 80, seed=10)
    addr = (cache._retrieve_scratch.buf.data_ptr(), cache._attn_scratch.buf.data_ptr())
    runner = bench.GraphedDecoder(model, cache)
    tok = torch.tensor([5], device=dev)
    got = []
    for _ in range(2):
        tok = model.step(cache, tok)
        got.append(int(tok))
    runner.tok.copy_(tok)
    runner.precapture(4)                      # graph(N) first, then graph(N + I) ... graph(N + 4 I)
    junk = [torch.full((64 << 20,), 0x7f, dtype=torch.uint8, device=dev) for _ in range(5)]
    torch.cuda.synchronize()
    del junk
    junk = [torch.full((8 << 20,), 0x55, dtype=torch.uint8, device=dev) for _ in range(24)]
    torch.cuda.synchronize()
    del junk
    for _ in range(4):                        # still before the first flush: these replay the first graph
        runner.step()
        got.append(int(runner.nxt))
    assert got == eager
    assert addr == (cache._retrieve_scratch.buf.data_ptr(), cache._attn_scratch.buf.data_ptr())
    cache.check_status()


def test_shared_scratch_refuses_to_grow_inside_a_capture():
    from pariskv_b200 import ops
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        g.capture_begin()
        try:
            with pytest.raises(RuntimeError, match="during a stream capture"):
                ops.workspace(DEV, 1 << 30, "test-capture-growth")
        finally:
            g.capture_end()
    torch.cuda.current_stream().wait_stream(s)


def test_attention_status_word_is_read_and_raised(oracle):
    """The attention kernel reports a copy wait that ran out through a status word in its scratch header.  Nothing is
    made to time out here: the word is set by hand and the host-side reader must raise; with the word cleared the
    same cache goes on giving correct results (the arrival counters in the same header were left at zero)."""
    g = torch.Generator().manual_seed(31)
    bs, H, Hq, sink, local, I, topk, P = 1, 2, 8, 4, 16, 8, 32, 2300
    cache = _make_cache(P, 32, bs, H, Hq, sink, local, I, topk, True, 1)
    K = synth_keys(g, bs, H, P)
    V = torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    nk = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
    nv = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
    cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), 0)
    q = torch.randn(bs, 1, Hq, 128, generator=g).to(torch.bfloat16)
    out = cache.compute(q.to(DEV), 0)
    cache.check_status()                                          # clean run: no complaint
    header = cache._attn_scratch.buf[: (bs * Hq + 1) * 4].view(torch.int32)
    assert int(header[: bs * Hq].abs().sum()) == 0                # every call leaves the counters at zero
    header[bs * Hq] = 1
    with pytest.raises(RuntimeError, match="gave up waiting"):
        cache.check_status()
    header[bs * Hq] = 0
    out2 = cache.compute(q.to(DEV), 0)
    assert torch.equal(out, out2)
    cache.check_status()


def test_per_query_head_retrieval_option(oracle):
    """per_query_head_retrieval: every query head selects its own top-k from the keys of its KV head.  Oracle: the
    same chain run with one "KV head" per query head (the KV head's codes repeated over the group, group size one)."""
    g = torch.Generator().manual_seed(41)
    bs, H, Hq, sink, local, I, topk, P = 2, 2, 8, 4, 16, 8, 32, 2300
    G = Hq // H
    from pariskv_b200.cache_hub.polar_cache import polar_cache
    cache = polar_cache(valid_start=[0] * bs, layer_num=1, batch_size=bs, max_length=P + 32, num_key_value_heads=H, num_heads=Hq,
                        head_dim=128, dtype=torch.bfloat16, layer_mapping={"0": DEV}, max_new_length=32, sink_size=sink,
                        local_size=local, core=0, nprobe=0, cache_unit_size=0, cache_cluster_num=0, num_gpus=1, model_size=8,
                        final_topk=topk, dynamic_update_interval=I, enable_offload=True, per_query_head_retrieval=True)
    K = synth_keys(g, bs, H, P)
    V = torch.randn(bs, H, P, 128, generator=g).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    nk = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
    nv = torch.randn(bs, H, 1, 128, generator=g).to(torch.bfloat16)
    cache.decode_update_kv_cache(nk.transpose(1, 2).contiguous().to(DEV), nv.transpose(1, 2).contiguous().to(DEV), 0)
    q = (torch.randn(bs, 1, Hq, 128, generator=g) * 0.5).to(torch.bfloat16)
    out = cache.compute(q.to(DEV), 0)
    signs = cache.srht_diagonal_signs.cpu()
    rep = lambda t: t.repeat_interleave(G, dim=1)          # KV-head tensors repeated per query head
    zk, zv = K[:, :, sink:P - local].contiguous(), V[:, :, sink:P - local].contiguous()
    cb, w, pk = oracle.encode(zk, signs)
    N = zk.shape[2]
    _, C, Kf = cache.retrieval_plan(N)
    _, coll = cache._get_adaptive_ratios(N)
    r = oracle.retrieve(q, signs, rep(cb), rep(w), rep(pk), rep(oracle.cluster_counts(cb)), cache._mag_centers.cpu(), coll, C, Kf)
    assert torch.equal(cache.last_topk_indices.cpu(), r["final"]), "per-query-head selections differ from the oracle"
    sel = r["final"]                                        # [bs, Hq, Kf]
    heads_differ = any(not torch.equal(sel[0, 0], sel[0, j]) for j in range(1, G))
    assert heads_differ, "query heads of one group should not all retrieve the same rows"
    wk = torch.cat([rep(K[:, :, :sink]), rep(K[:, :, P - local:]), rep(nk), oracle.gather(rep(zk), sel)], 2)
    wv = torch.cat([rep(V[:, :, :sink]), rep(V[:, :, P - local:]), rep(nv), oracle.gather(rep(zv), sel)], 2)
    ref = oracle.attention(q, wk, wv)                      # Hq query heads over Hq "KV heads": group size one
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2


def test_batch_of_different_lengths_equals_single_sequences(oracle):
    """Three samples of different lengths decoded as ONE batch (left-padded lockstep prefill, per-sample zone lengths
    read on the device) across a flush: every step, every sample's retrieved indices and attention output must be
    exactly what a batch-1 cache of that sample gives, and the indices must be the oracle's."""
    g = torch.Generator().manual_seed(51)
    H, Hq, sink, local, I, topk = 2, 8, 4, 16, 8, 48
    lens = [2300, 3100, 2650]
    bs, Pmax, steps = len(lens), max(lens), 12
    Ks = [synth_keys(g, 1, H, n) for n in lens]
    Vs = [torch.randn(1, H, n, 128, generator=g).to(torch.bfloat16) for n in lens]

    def make(batch, starts):
        from pariskv_b200.cache_hub.polar_cache import polar_cache
        return polar_cache(valid_start=starts, layer_num=1, batch_size=batch, max_length=Pmax + 32, num_key_value_heads=H,
                           num_heads=Hq, head_dim=128, dtype=torch.bfloat16, layer_mapping={"0": DEV}, max_new_length=32,
                           sink_size=sink, local_size=local, core=0, nprobe=0, cache_unit_size=0, cache_cluster_num=0,
                           num_gpus=1, model_size=8, final_topk=topk, dynamic_update_interval=I, enable_offload=True)

    batched = make(bs, [Pmax - n for n in lens])
    kp = torch.zeros(bs, Pmax, H, 128, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    for b, n in enumerate(lens):                     # left padding: sample b starts at column Pmax - n
        kp[b, Pmax - n:] = Ks[b][0].transpose(0, 1)
        vp[b, Pmax - n:] = Vs[b][0].transpose(0, 1)
    batched.prefill_update_kv_cache(None, kp.to(DEV), vp.to(DEV), 0, 0)
    singles = []
    for b, n in enumerate(lens):
        c = make(1, [0])
        c.prefill_update_kv_cache(None, Ks[b].transpose(1, 2).contiguous().to(DEV), Vs[b].transpose(1, 2).contiguous().to(DEV), 0, 0)
        singles.append(c)
    assert batched.zone_len[0] == [n - sink - local for n in lens]
    signs = batched.srht_diagonal_signs.cpu()
    for t in range(steps):
        nk = synth_keys(g, bs, H, 1).transpose(1, 2).contiguous()      # [bs,1,H,128]
        nv = torch.randn(bs, 1, H, 128, generator=g).to(torch.bfloat16)
        q = (torch.randn(bs, 1, Hq, 128, generator=g) * 0.5).to(torch.bfloat16)
        batched.decode_update_kv_cache(nk.to(DEV), nv.to(DEV), 0)
        out = batched.compute(q.to(DEV), 0)
        for b, n in enumerate(lens):
            Ks[b] = torch.cat([Ks[b], nk[b:b + 1].transpose(1, 2)], 2)
            singles[b].decode_update_kv_cache(nk[b:b + 1].to(DEV), nv[b:b + 1].to(DEV), 0)
            one = singles[b].compute(q[b:b + 1].to(DEV), 0)
            assert torch.equal(out[b:b + 1], one), (t, b)
            kb = int(batched.last_n_sel[b, 0])
            assert kb == singles[b].last_topk_indices.shape[2] == topk
            assert torch.equal(batched.last_topk_indices[b, :, :kb], singles[b].last_topk_indices[0]), (t, b)
            if t in (0, steps - 1):                   # before and after the flush: the oracle on this sample's zone
                N = batched.zone_len[0][b]
                zk = Ks[b][:, :, sink:sink + N].contiguous()
                cb, w, pk = oracle.encode(zk, signs)
                _, C, Kf = batched.retrieval_plan(N)
                _, coll = batched._get_adaptive_ratios(N)
                r = oracle.retrieve(q[b:b + 1], signs, cb, w, pk, oracle.cluster_counts(cb), batched._mag_centers.cpu(), coll, C, Kf)
                assert torch.equal(batched.last_topk_indices[b:b + 1, :, :Kf].cpu(), r["final"]), (t, b)
    assert batched.zone_len[0] == [n - sink - local + I for n in lens], "one flush of the update buffer was expected"
    batched.check_status()


def test_append_reports_a_full_zone_through_its_status_word():
    """A flush that finds no room in the zone publishes nothing and raises the layer's error word; the host-side
    mirror refuses the step before it is launched.  Here the launch is forced through the op itself, with a state
    that claims a zone already at capacity: every address stays valid, nothing faults."""
    from pariskv_b200 import ops
    cache = _make_cache(2300, 8, 1, 2, 8, 4, 16, 8, 32, False, 1)
    g = torch.Generator().manual_seed(3)
    K = synth_keys(g, 1, 2, 2300)
    V = torch.randn(1, 2, 2300, 128, generator=g).to(torch.bfloat16)
    cache.prefill_update_kv_cache(None, K.transpose(1, 2).contiguous().to(DEV), V.transpose(1, 2).contiguous().to(DEV), 0, 0)
    st = cache._layer_state[0]
    st[0] = cache.window_capacity - 1            # the next row fills the window ...
    st[4] = cache.zone_capacity                  # ... and the zone claims to be full
    row = torch.zeros(1, 1, 2, 128, dtype=torch.bfloat16, device=DEV)
    ops.append_encode(row, row, cache.srht_diagonal_signs, cache.unified_keys_gpu[0], cache.unified_values_gpu[0],
                      cache._win_codes[0], cache._win_weight[0], cache._win_4bit[0], cache._win_vnorm[0], cache.codebook_gpu[0],
                      cache.key_block_weight_gpu[0], cache.key_4bit_packed_gpu[0], None, cache.cluster_key_counts_gpu[0],
                      cache._store_kv[0], st, cache.sink_size, cache.dynamic_update_interval)
    torch.cuda.synchronize()
    assert st.tolist()[3] == 1 and st.tolist()[4] == cache.zone_capacity
    with pytest.raises(RuntimeError, match="no room for a flush"):
        cache.check_status()
