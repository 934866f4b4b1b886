"""Sequence-sharded retrieval + attention on two GPUs (NCCL) against the same sharded formulation evaluated by
the oracle in one process.  Skipped on machines with fewer than two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import srht_signs, synth_keys, synth_queries
from test_dist_gloo import _free_port, _single_gpu_final

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import oracle as O
        from pariskv_b200 import dist as pkd, ops
        g = torch.Generator().manual_seed(3)
        bs, H, N, K = 1, 2, 9001, 128
        keys = synth_keys(g, bs, H, N)
        vals = torch.randn(bs, H, N, 128, generator=g).to(torch.bfloat16)
        q = synth_queries(g, keys, 4) * 4
        wk = torch.randn(bs, H, 40, 128, generator=g).to(torch.bfloat16)
        wv = torch.randn(bs, H, 40, 128, generator=g).to(torch.bfloat16)
        signs = srht_signs()
        _, cen = O.constants()
        cand_ratio, coll = O.adaptive_ratios(N)
        start, end = pkd.sequence_shard(N, rank, world)
        counts = torch.zeros(bs, H, 16, 256, dtype=torch.int32, device=dev)
        cb, w, pk = ops.encode_keys(keys[:, :, start:end].contiguous().to(dev), signs.to(dev), cluster_counts=counts)
        pkd.allreduce_cluster_counts(counts)
        cb_all, _, _ = O.encode(keys, signs)
        assert torch.equal(counts.cpu(), O.cluster_counts(cb_all))
        sk = keys[:, :, start:end].contiguous().pin_memory()
        sv = vals[:, :, start:end].contiguous().pin_memory()
        out, final = pkd.sequence_sharded_attend(
            q.to(dev), signs.to(dev), cen.to(dev), cb, w, pk, counts, sk, sv, N, start, end, coll, cand_ratio, K,
            window_k=wk.to(dev) if rank == 0 else None, window_v=wv.to(dev) if rank == 0 else None,
            n_window=40 if rank == 0 else 0)
        want = _single_gpu_final(O, keys, q, signs, cen, coll, cand_ratio, K, counts.cpu())
        assert torch.equal(final.cpu(), want), "the sharded selection is not the single-GPU selection"
        ref = O.attention(q, torch.cat([wk, O.gather(keys, want)], 2), torch.cat([wv, O.gather(vals, want)], 2))
        err = (out.float().cpu() - ref).abs().max().item()
        assert err <= 2e-2, err
        torch.save(out.cpu(), os.path.join(tmp, f"out_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _cache_check(rank, world, dev, exchange="nccl"):
    """SequenceShardedCache: load two layers, decode across one flush of the update buffer (the flushed rows go to the
    last rank's chunk, the histogram delta is all-reduced), attend; against the oracle's SINGLE-GPU selection over the
    whole zone."""
    from oracle import oracle as O
    from pariskv_b200 import dist as pkd
    g = torch.Generator().manual_seed(5)
    H, N0, K, sink, local, interval, steps = 2, 7003, 96, 4, 16, 4, 6
    signs = srht_signs()
    _, cen = O.constants()
    cache = pkd.SequenceShardedCache(2, H, 8, N0, sink, local, interval, K, dev, rank, world,
                                     srht_sign_vector=signs, exchange=exchange, max_new_length=steps)
    start, end = pkd.sequence_shard(N0, rank, world)
    spans0 = [pkd.sequence_shard(N0, r, world) for r in range(world)]
    data = []
    for l in range(2):
        keys = synth_keys(g, 1, H, N0)                      # the zone: token positions [sink, sink + N0)
        vals = torch.randn(1, H, N0, 128, generator=g).to(torch.bfloat16)
        wk = torch.randn(1, H, sink + local, 128, generator=g).to(torch.bfloat16)
        wv = torch.randn(1, H, sink + local, 128, generator=g).to(torch.bfloat16)
        cache.load_layer(l, keys[:, :, start:end].contiguous().to(dev), vals[:, :, start:end].contiguous().to(dev),
                         wk.to(dev), wv.to(dev))
        data.append([keys, vals, wk, wv])
    assert cache.context == sink + N0 + local
    for step in range(steps):
        for l in range(2):
            keys, vals, wk, wv = data[l]
            nk = torch.randn(1, 1, H, 128, generator=g).to(torch.bfloat16)
            nv = torch.randn(1, 1, H, 128, generator=g).to(torch.bfloat16)
            q = synth_queries(g, keys, 4) * 4
            cache.decode_update_kv_cache(nk.to(dev), nv.to(dev), l)
            qd = q.to(dev)
            if world > 1:   # the oracle work between steps skews the ranks by seconds; the peer waits are short
                torch.cuda.synchronize()
                dist.barrier()
            out = cache.compute(qd, l)
            wk = torch.cat([wk, nk.transpose(1, 2)], 2)
            wv = torch.cat([wv, nv.transpose(1, 2)], 2)
            if wk.shape[2] == sink + local + interval:      # the same flush on the oracle side
                keys = torch.cat([keys, wk[:, :, sink:sink + interval]], 2)
                vals = torch.cat([vals, wv[:, :, sink:sink + interval]], 2)
                wk = torch.cat([wk[:, :, :sink], wk[:, :, sink + interval:]], 2)
                wv = torch.cat([wv[:, :, :sink], wv[:, :, sink + interval:]], 2)
            data[l] = [keys, vals, wk, wv]
            N = keys.shape[2]
            assert cache.cpu_valid_end[l] == N
            counts = O.cluster_counts(O.encode(keys, signs)[0])
            assert torch.equal(cache.counts[l].cpu(), counts)
            want = _single_gpu_final(O, keys, q, signs, cen, 0.2, 0.1, K, counts)
            assert torch.equal(cache.last_topk_indices.cpu(), want), (step, l)
            ref = O.attention(q, torch.cat([wk, O.gather(keys, want)], 2), torch.cat([wv, O.gather(vals, want)], 2))
            err = (out.float().cpu() - ref).abs().max().item()
            assert err <= 2e-2, err
    assert cache.context == sink + N0 + local + steps and cache.cpu_valid_end == [N0 + interval] * 2
    if cache.px is not None:
        cache.px.check()


def _cache_worker(rank, world, port, exchange="nccl"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        _cache_check(rank, world, dev, exchange)
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_cache_single_rank():
    _cache_check(0, 1, torch.device("cuda", 0))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharded_cache_on_two_gpus():
    mp.spawn(_cache_worker, args=(2, _free_port()), nprocs=2, join=True)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharded_cache_peer_exchange_on_two_gpus():
    """The same check with both exchanges as stores into peer memory (bounded flag waits) instead of NCCL."""
    mp.spawn(_cache_worker, args=(2, _free_port(), "peer"), nprocs=2, join=True)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharded_on_two_gpus(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    a = torch.load(os.path.join(tmp_path, "out_0.pt"))
    b = torch.load(os.path.join(tmp_path, "out_1.pt"))
    assert torch.equal(a, b)


# ---- KV-head-sharded (tensor-parallel) form ------------------------------------------------------------------------
def test_head_sharded_caches_reproduce_the_full_cache():
    """Each of W caches built with H / W KV heads (the tensor-parallel split) must retrieve exactly the indices that
    the full-width cache retrieves for those heads, and produce the same attention output for their query heads."""
    from pariskv_b200 import dist as pkd
    from pariskv_b200.cache_hub.polar_cache import polar_cache
    dev = "cuda:0"
    g = torch.Generator().manual_seed(12)
    H, Hq, P, sink, local, I, K = 8, 32, 4200, 4, 16, 8, 64
    keys = synth_keys(g, 1, H, P)
    vals = torch.randn(1, H, P, 128, generator=g).to(torch.bfloat16)
    q = (torch.randn(1, 1, Hq, 128, generator=g) * 0.5).to(torch.bfloat16)

    def run(heads, qheads):
        c = polar_cache(valid_start=[0], layer_num=1, batch_size=1, max_length=P + 16, num_key_value_heads=heads.stop - heads.start,
                        num_heads=qheads.stop - qheads.start, head_dim=128, dtype=torch.bfloat16, layer_mapping={"0": dev},
                        max_new_length=16, sink_size=sink, local_size=local, core=0, nprobe=0, cache_unit_size=0,
                        cache_cluster_num=0, num_gpus=1, model_size=8, final_topk=K, dynamic_update_interval=I,
                        enable_offload=True)
        c.prefill_update_kv_cache(None, keys[:, heads].transpose(1, 2).contiguous().to(dev),
                                  vals[:, heads].transpose(1, 2).contiguous().to(dev), 0, 0)
        out = c.compute(q[:, :, qheads].contiguous().to(dev), 0)
        return c.last_topk_indices.cpu(), out.cpu()

    full_idx, full_out = run(slice(0, H), slice(0, Hq))
    for world in (2, 8):
        for r in range(world):
            hs = pkd.head_shard(H, r, world)
            qs = slice(hs.start * 4, hs.stop * 4)
            idx, out = run(hs, qs)
            assert torch.equal(idx, full_idx[:, hs]), (world, r)
            assert torch.equal(out, full_out[:, :, qs]), (world, r)


def _tp_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from pariskv_b200.dist import TPReducer
        for mode in ("peer", "nccl"):
            red = TPReducer(4096, dev, mode=mode)
            g = torch.Generator().manual_seed(7)
            for it in range(60):      # back to back: consecutive reductions alternate between the two gather areas
                parts = [torch.randn(1, 4096, generator=g).to(torch.bfloat16) for _ in range(world)]
                res = torch.randn(1, 4096, generator=g).to(torch.bfloat16)
                want = res.float()
                for p in parts:
                    want = want + p.float()
                got = red.reduce(parts[rank].clone().to(dev), res.to(dev)).float().cpu()
                if mode == "peer":
                    assert torch.equal(got, want.to(torch.bfloat16).float()), (mode, it)
                else:
                    assert (got - want).abs().max().item() <= 0.25, (mode, it)
                if it % 3 == 0:       # the same reduction with the RMS-norm of the result written by the same launch
                    wn = (1.0 + 0.1 * torch.randn(4096, generator=g)).to(torch.bfloat16)
                    h, x = red.reduce_norm(parts[rank].clone().to(dev), res.to(dev), wn.to(dev))
                    h, x = h.float().cpu(), x.float().cpu()
                    if mode == "peer":
                        assert torch.equal(h, got), (mode, it)
                    ref = h * torch.rsqrt((h * h).mean() + 1e-6) * wn.float()
                    assert (x - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item()), (mode, it)
            red.check()
            torch.cuda.synchronize()
            dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_reduce_on_two_gpus():
    mp.spawn(_tp_worker, args=(2, _free_port()), nprocs=2, join=True)


class _EchoCache:
    """Stands in for a cache that wants all heads on every rank: attention output = the (normed, rotated) queries."""
    context = 300

    def decode_update_kv_cache(self, k, v, layer):
        self.kv_shape = (tuple(k.shape), tuple(v.shape))

    def compute(self, q, layer):
        return q


def _hybrid_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bench
        from pariskv_b200.dist import TPReducer
        cfg = dict(layers=3, hidden=512, q_heads=8, kv_heads=4, head_dim=128, ffn=1024, vocab=2048, rope_theta=1e4)
        single = bench.DecoderHarness(cfg, dev, seed=21)
        tok = torch.tensor([17], device=dev)
        single.step(_EchoCache(), tok)
        want = single.last_logits.float()
        Vr = cfg["vocab"] // world
        for mode in ("peer", "nccl"):
            red = TPReducer((cfg["q_heads"] + 2 * cfg["kv_heads"]) * 128, dev, mode=mode)
            model = bench.DecoderHarness(cfg, dev, seed=21, rank=rank, world=world, reducer=red, gather_heads=True)
            cache = _EchoCache()
            nxt = model.step(cache, tok)
            got = model.last_logits.float()
            # the cache saw ALL heads; the logits are this rank's slice of the single-GPU logits (bf16 rounding of the
            # split sums aside); the arg-max over the ranks' slices is the same token on every rank
            assert cache.kv_shape == ((1, 1, 4, 128), (1, 1, 4, 128))
            ref = want[:, rank * Vr:(rank + 1) * Vr]
            assert (got - ref).abs().max().item() <= 0.05 * max(1.0, ref.abs().max().item()), mode
            toks = torch.empty(world, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(toks, nxt)
            assert bool((toks == toks[0]).all())
            red.check()
            torch.cuda.synchronize()
            dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_dense_layers_with_all_heads_gathered_on_two_gpus():
    """The harness form used with the sequence-sharded cache: q/k/v rows all-gathered (peer kernel or NCCL), output
    and MLP projections reduced; against the single-GPU harness with the same weights."""
    mp.spawn(_hybrid_worker, args=(2, _free_port()), nprocs=2, join=True)
