"""CPU-side tests: the oracle against the golden fixtures produced by the reference's own code, and the
C-ABI library's exported surface (no compute without a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, bf16_from_bits, bits_of


# ---- oracle vs golden fixtures ---------------------------------------------------------------------
def test_oracle_encode_matches_reference(oracle, golden):
    e = golden("encode")
    cb, w, pk = oracle.encode(bf16_from_bits(e["keys"]), bf16_from_bits(e["signs"]))
    assert torch.equal(cb, torch.from_numpy(e["codebook"]))
    assert torch.equal(pk, torch.from_numpy(e["packed_4bit"]))
    assert torch.equal(bits_of(w), bits_of(bf16_from_bits(e["block_weight"])))
    assert torch.equal(oracle.cluster_counts(cb), torch.from_numpy(e["cluster_counts"]))
    thr, cen = oracle.constants()
    assert torch.equal(bits_of(thr), bits_of(bf16_from_bits(e["mag_thresholds"])))
    assert torch.equal(bits_of(cen), bits_of(bf16_from_bits(e["mag_centers"])))


def test_oracle_query_rank_collision_match_reference(oracle, golden):
    q = golden("query_collision")
    qb, qn = oracle.query_prep(bf16_from_bits(q["queries"]), 2, bf16_from_bits(q["signs"]))
    assert torch.equal(bits_of(qb), bits_of(bf16_from_bits(q["q_blocks"])))
    assert torch.equal(bits_of(qn), bits_of(bf16_from_bits(q["q_norm"])))
    cb, w, pk = oracle.encode(bf16_from_bits(q["keys"]), bf16_from_bits(q["signs"]))
    assert torch.equal(cb, torch.from_numpy(q["codebook"]))
    assert torch.equal(bits_of(w), bits_of(bf16_from_bits(q["block_weight"])))
    # cluster order: the reference's argsort is not stable, so compare the score sequences
    ids = oracle.cluster_rank(qb)
    rid = torch.from_numpy(q["sorted_ids"].astype(np.int64))
    sc = bf16_from_bits(q["cluster_scores"]).float()
    assert torch.equal(torch.gather(sc, -1, ids), torch.gather(sc, -1, rid))
    so = torch.gather(sc, -1, ids)
    assert bool((so[..., 1:] <= so[..., :-1]).all())
    tie = so[..., 1:] == so[..., :-1]
    assert bool((ids[..., 1:][tie] > ids[..., :-1][tie]).all()), "ties must go to the lower cluster id"
    assert oracle.tier_counts(q["codebook"].shape[3], float(q["collision_ratio"])) == q["tier_counts"].tolist()
    cnt = oracle.collision(rid, torch.from_numpy(q["cluster_counts"]), torch.from_numpy(q["codebook"]),
                           q["tier_counts"].tolist())
    assert torch.equal(cnt, torch.from_numpy(q["cache_cnt"]))


def test_oracle_collision_matches_reference_generator(oracle, golden):
    c = golden("collision")
    for tag in ("n2048", "n1000"):
        out = oracle.collision(torch.from_numpy(c[tag + "_sorted_ids"].astype(np.int64)),
                               torch.from_numpy(c[tag + "_cluster_counts"]), torch.from_numpy(c[tag + "_codebook"]),
                               c[tag + "_tier_counts"].tolist())
        assert torch.equal(out, torch.from_numpy(c[tag + "_cache_cnt"]))
    out = oracle.collision_single(torch.from_numpy(c["single_sorted_ids"]), torch.from_numpy(c["single_topk_cluster_cnt"]),
                                  torch.from_numpy(c["single_codebook"]))
    assert torch.equal(out, torch.from_numpy(c["single_cache_cnt"]))


def test_oracle_rerank_matches_reference(oracle, golden):
    r = golden("rerank")
    N = r["key_4bit"].shape[3]
    cand = torch.arange(N).view(1, 1, N).expand(1, 2, N).contiguous()
    s32, sbf = oracle.rerank(cand, torch.from_numpy(r["key_4bit"]), bf16_from_bits(r["key_block_weight"]),
                             bf16_from_bits(r["q_blocks"]), bf16_from_bits(r["q_norm"]), bf16_from_bits(r["mag_centers"]))
    ref = torch.from_numpy(r["scores_fp32"])
    rel = ((s32 - ref).abs() / ref.abs().clamp(min=1e-3 * ref.abs().max())).max().item()
    assert rel <= 1e-3, rel
    fin = oracle.final_topk(s32, cand, int(r["final_topk"]))
    assert bool((fin[..., 1:] > fin[..., :-1]).all())
    for h in range(2):
        assert set(fin[0, h].tolist()) == set(r["final_fp32"][0, h].tolist())
        # the literal bf16 pipeline of the reference rounds five times; it still agrees on almost all keys
        assert len(set(fin[0, h].tolist()) & set(r["final_bf16"][0, h].tolist())) >= 95
    # candidate stage: same set as the reference's truncating filter up to ties at the threshold count
    cnt = torch.from_numpy(r["cache_cnt"])
    C = r["truncate_candidates"].shape[-1]
    mine = oracle.topk(cnt, C)
    for h in range(2):
        a, b = cnt[0, h][mine[0, h]], cnt[0, h][torch.from_numpy(r["truncate_candidates"][0, h].astype(np.int64))]
        assert sorted(a.tolist()) == sorted(b.tolist())


def test_oracle_adaptive_k_matches_reference(oracle, golden):
    a = golden("adaptive_topk")
    for i in range(4):
        cs = bf16_from_bits(a[f"c{i}_cand_scores"]).float() * float(a[f"c{i}_attn_scale"])
        K_out = min(int(a[f"c{i}_topk_cap"]), cs.shape[-1])
        k, idx = oracle.adaptive_topk(torch.from_numpy(a[f"c{i}_sl_logits"]), torch.from_numpy(a[f"c{i}_sl_vnorm"]), cs,
                                      torch.from_numpy(a[f"c{i}_cand_vnorm"]),
                                      torch.from_numpy(a[f"c{i}_cand_indices"].astype(np.int64)),
                                      float(a[f"c{i}_threshold"]), K_out)
        k_ref = torch.from_numpy(a[f"c{i}_adaptive_k"])
        idx_ref = torch.from_numpy(a[f"c{i}_topk_indices"].astype(np.int64))
        assert torch.equal(k, k_ref)
        for b in range(k.shape[0]):
            for h in range(k.shape[1]):
                kk = int(k_ref[b, h])
                assert set(idx[b, h, :kk].tolist()) == set(idx_ref[b, h, :kk].tolist())


def test_oracle_topk_contract(oracle):
    x = torch.tensor([[3, 7, 7, 1, 7, 3, 0]], dtype=torch.int32)
    assert oracle.topk(x, 2).tolist() == [[1, 2]]
    assert oracle.topk(x, 4).tolist() == [[0, 1, 2, 4]]
    assert oracle.topk(x, 4, sorted_by_value=True).tolist() == [[1, 2, 4, 0]]
    f = torch.tensor([[-0.0, 0.0, -1.5, 2.5, float("-inf")]])
    assert oracle.topk(f, 2, sorted_by_value=True).tolist() == [[3, 1]]


def test_oracle_expf_close_to_libm(oracle):
    xs = np.linspace(-87, 0, 20001, dtype=np.float32)
    got = np.array([oracle.lib().pko_expf(ctypes.c_float(float(x))) for x in xs[::40]], dtype=np.float64)
    ref = np.exp(xs[::40].astype(np.float64))
    assert np.max(np.abs(got - ref) / ref) < 4e-7


def test_oracle_attention_matches_torch(oracle):
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 8, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 2, 50, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(1, 2, 50, 128, generator=g).to(torch.bfloat16)
    out = oracle.attention(q, k, v)
    qq = q.float().view(1, 2, 4, 128)
    ref = torch.softmax(torch.einsum("bhgd,bhnd->bhgn", qq, k.float()) / 128 ** 0.5, -1) @ v.float()
    assert (out.view(1, 2, 4, 128) - ref).abs().max().item() < 1e-5


# ---- the C ABI ---------------------------------------------------------------------------------------
def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pariskv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from pariskv_b200 import _lib
    from pariskv_b200.build import build
    build()
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header declarations differ"
    assert lib.pk_version() == 1
    assert lib.pk_collision_workspace_bytes(1, 8, 16, 256) == 8 * 16 * 256
    assert lib.pk_attention_workspace_bytes(1, 32, 2244) == 256 + 32 * 36 * 132 * 4
    assert lib.pk_retrieve_workspace_bytes(1, 8, 131004, 13101) > 0


def test_public_header_is_plain_c():
    """include/pariskv_b200.h must compile on its own as C and as C++ (no torch types, no CUDA headers)."""
    import shutil
    import subprocess
    hdr = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "pariskv_b200.h")
    for cc, args in (("gcc", ["-x", "c", "-std=c11"]), ("g++", ["-x", "c++", "-std=c++17"])):
        if shutil.which(cc) is None:
            pytest.skip(f"{cc} not installed")
        r = subprocess.run([cc, "-fsyntax-only", "-Wall", *args, hdr], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_argument_errors_surface_as_exceptions():
    """Validation runs before any CUDA call, so it can be exercised without a GPU."""
    from pariskv_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(2, 10, dtype=torch.int32)
    out = torch.zeros(2, 11, dtype=torch.int64)
    dx, do = _lib.desc(x), _lib.desc(out)
    rc = lib.pk_topk(_lib.ref(dx), 11, _lib.ref(do), 0, None)
    assert rc == 1 and b"k must be" in lib.pk_last_error()
    with pytest.raises(RuntimeError, match="k must be"):
        _lib.check(rc)
    bad = torch.zeros(2, 10, dtype=torch.float64)
    with pytest.raises(TypeError):
        _lib.desc(bad)


def test_ops_refuse_cpu_tensors():
    from pariskv_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.topk(torch.zeros(2, 10, dtype=torch.int32), 3)


def test_host_gather_runs_on_cpu(oracle):
    from pariskv_b200 import ops
    g = torch.Generator().manual_seed(0)
    src = torch.randn(2, 3, 100, 128, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 100, (2, 3, 17), generator=g)
    out = torch.empty(2, 3, 17, 128, dtype=torch.bfloat16)
    ops.gather_kv_out_cpu(src, idx, out, n_threads=2)
    assert torch.equal(out, oracle.gather(src, idx))
    idx[1, 2, 3] = 100
    with pytest.raises(RuntimeError, match="out of bounds"):
        ops.gather_kv_out_cpu(src, idx, out)


def test_torch_ops_are_registered_with_schemas_and_shape_functions():
    """The seven ops are torch custom ops (namespace pariskv): the dispatcher knows their schemas and, through the
    fake implementations, their output shapes - checked here on meta tensors, no GPU involved."""
    from pariskv_b200 import torch_ops
    for name in torch_ops.OPS:
        assert hasattr(torch.ops.pariskv, name), name
    m = lambda *shape, dtype: torch.empty(*shape, dtype=dtype, device="meta")
    bs, H, B, NC, N, C = 2, 3, 16, 256, 1000, 100
    out = torch.ops.pariskv.collision_fused(m(bs, H, B, NC, dtype=torch.int64), m(bs, H, B, NC, dtype=torch.int32),
                                            m(bs, H, B, N, dtype=torch.uint8), [10, 20, 30, 40, 50, 60])
    assert out.shape == (bs, H, N) and out.dtype == torch.int32
    out = torch.ops.pariskv.collision(m(bs, H, B, NC, dtype=torch.int32), m(bs, H, B, dtype=torch.int32),
                                      m(bs, H, N, B, dtype=torch.int32))
    assert out.shape == (bs, H, N) and out.dtype == torch.int32
    out = torch.ops.pariskv.topk(m(bs, H, N, dtype=torch.int32), C)
    assert out.shape == (bs, H, C) and out.dtype == torch.int64
    out = torch.ops.pariskv.rerank(m(bs, H, C, dtype=torch.int64), m(bs, H, B, N, 4, dtype=torch.uint8),
                                   m(bs, H, B, N, dtype=torch.bfloat16), m(bs, H, B, 8, dtype=torch.bfloat16),
                                   m(bs, H, 1, dtype=torch.bfloat16), m(8, dtype=torch.bfloat16))
    assert out.shape == (bs, H, C) and out.dtype == torch.bfloat16
    k, idx = torch.ops.pariskv.adaptive_k_fused(m(bs, H, 68, dtype=torch.float32), m(bs, H, C, dtype=torch.bfloat16), 0.088,
                                                m(bs, H, 68, dtype=torch.float32), m(bs, H, C, dtype=torch.int64),
                                                m(bs, H, C, dtype=torch.float32), 0.9, 64)
    assert k.shape == (bs, H) and idx.shape == (bs, H, 64) and idx.dtype == torch.int64
    schema = str(torch.ops.pariskv.gather_trans.default._schema)
    assert "Tensor(a!) dst_k" in schema and "Tensor(b!) dst_v" in schema
    # the host-side gather runs through the registered op
    src = torch.randn(1, 2, 50, 128).to(torch.bfloat16)
    index = torch.randint(0, 50, (1, 2, 7))
    out = torch.empty(1, 2, 7, 128, dtype=torch.bfloat16)
    torch.ops.pariskv.gather(src, index, out)
    assert torch.equal(out, torch.gather(src, 2, index[..., None].expand(1, 2, 7, 128)))


def test_host_numa_helpers_without_a_gpu():
    """The CPU-list parser, and the store-placement scope as a no-op where the GPU's node cannot be told."""
    import os
    from pariskv_b200 import hostmem
    assert hostmem._cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert hostmem._cpulist("") == set()
    before = os.sched_getaffinity(0)
    import torch
    with hostmem.near_device(torch.device("cuda", 0)) as scope:
        assert scope.bound is None or scope.bound["cpus"] > 0
    assert os.sched_getaffinity(0) == before
