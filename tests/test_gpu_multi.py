"""Sequence-sharded retrieval + attention on two GPUs (NCCL) against the same sharded formulation evaluated by
the oracle in one process.  Skipped on machines with fewer than two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import srht_signs, synth_keys, synth_queries
from test_dist_gloo import _free_port, _shard_result

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
        parts = [_shard_result(O, r, world, keys, vals, q, signs, cen, coll, cand_ratio, K, counts.cpu()) for r in range(world)]
        want = O.final_topk(torch.cat([p[0] for p in parts], -1), torch.cat([p[1] for p in parts], -1), K)
        assert torch.equal(final.cpu(), want), "global selection differs from the sharded oracle"
        ref = O.attention(q, torch.cat([wk, O.gather(keys, want)], 2), torch.cat([wv, O.gather(vals, want)], 2))
        err = (out.float().cpu() - ref).abs().max().item()
        assert err <= 2e-2, err
        torch.save(out.cpu(), os.path.join(tmp, f"out_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _cache_check(rank, world, dev, exchange="nccl"):
    """SequenceShardedCache: load two layers, append two rows, attend; against the oracle on the whole zone."""
    from oracle import oracle as O
    from pariskv_b200 import dist as pkd
    g = torch.Generator().manual_seed(5)
    H, N, K, sink, local, interval = 2, 7003, 96, 4, 16, 8
    signs = srht_signs()
    _, cen = O.constants()
    cache = pkd.SequenceShardedCache(2, H, 8, N, sink, local, interval, K, dev, rank, world,
                                     srht_sign_vector=signs, exchange=exchange)
    start, end = pkd.sequence_shard(N, rank, world)
    data = []
    for l in range(2):
        keys = synth_keys(g, 1, H, N)
        vals = torch.randn(1, H, N, 128, generator=g).to(torch.bfloat16)
        wk = torch.randn(1, H, sink + local, 128, generator=g).to(torch.bfloat16)
        wv = torch.randn(1, H, sink + local, 128, generator=g).to(torch.bfloat16)
        cache.load_layer(l, keys[:, :, start:end].contiguous().to(dev), vals[:, :, start:end].contiguous().to(dev),
                         wk.to(dev), wv.to(dev))
        data.append((keys, vals, wk, wv))
    assert cache.context == sink + N + local
    for step in range(2):
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
            data[l] = (keys, vals, wk, wv)
            counts = O.cluster_counts(O.encode(keys, signs)[0])
            parts = [_shard_result(O, r, world, keys, vals, q, signs, cen, 0.2, 0.1, K, counts) for r in range(world)]
            want = O.final_topk(torch.cat([p[0] for p in parts], -1), torch.cat([p[1] for p in parts], -1), K)
            assert torch.equal(cache.last_topk_indices.cpu(), want)
            ref = O.attention(q, torch.cat([wk, O.gather(keys, want)], 2), torch.cat([wv, O.gather(vals, want)], 2))
            err = (out.float().cpu() - ref).abs().max().item()
            assert err <= 2e-2, err
    assert cache.context == sink + N + local + 2
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
