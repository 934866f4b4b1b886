"""The allocation-free collision entry point (pk_collision_fused_static) against the regular one.

Some users of the library cannot allocate device memory at all on the decode path - a plugin inside a
serving runtime that has taken the whole HBM pool, a latency-critical thread kept off the allocator - so this
entry point keeps its scratch table in a fixed array inside the library.  The test calls it through the C ABI
twice in a row on different inputs (the array is shared and keeps the previous call's table) and requires the
same bits as the regular entry point, no growth of the allocator's footprint, and a clear refusal beyond the
stated size limit.  It lives in its own file that pytest collects last.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, bs, H, N, B=16, NC=256):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.stack([torch.stack([torch.randperm(NC, generator=g) for _ in range(B)])
                                    for _ in range(H)]) for _ in range(bs)])
    ckc = torch.randint(1, max(2, N // 4), (bs, H, B, NC), generator=g, dtype=torch.int32)
    cb = torch.randint(0, NC, (bs, H, B, N), generator=g, dtype=torch.int32).to(torch.uint8)
    return ids.to(DEV), ckc.to(DEV), cb.to(DEV)


def test_static_scratch_entry_point_matches_regular_one_twice():
    from pariskv_b200 import _lib, ops
    lib = _lib.load()
    assert lib.pk_collision_fused_static_max_triples() == 1024
    cases = [(1, 2, 8, 5000, [40, 120, 300, 700, 1500, 2600]), (2, 1, 3, 777, [9, 30, 61, 100, 150, 200])]
    for seed, bs, H, N, tiers in cases:           # two calls in a row, second with other shapes and tiers
        ids, ckc, cb = _inputs(seed, bs, H, N)
        want = ops.collision_fused(ids, ckc, cb, tiers)
        out = torch.full((bs, H, N), -1, dtype=torch.int32, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        ops.collision_fused_static(ids, ckc, cb, tiers, out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, "the allocation-free entry point allocated"
        assert torch.equal(out, want)
    # same inputs as the first call again: the table left by the second call must not matter
    seed, bs, H, N, tiers = cases[0]
    ids, ckc, cb = _inputs(seed, bs, H, N)
    out = torch.empty(bs, H, N, dtype=torch.int32, device=DEV)
    ops.collision_fused_static(ids, ckc, cb, tiers, out)
    assert torch.equal(out, ops.collision_fused(ids, ckc, cb, tiers))


def test_static_scratch_entry_point_rejects_oversize():
    from pariskv_b200 import ops
    bs, H, B = 9, 8, 16                            # 1152 triples > 1024
    ids = torch.zeros(bs, H, B, 256, dtype=torch.int64, device=DEV)
    ckc = torch.zeros(bs, H, B, 256, dtype=torch.int32, device=DEV)
    cb = torch.zeros(bs, H, B, 64, dtype=torch.uint8, device=DEV)
    out = torch.zeros(bs, H, 64, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="at most 1024"):
        ops.collision_fused_static(ids, ckc, cb, [1, 2, 3, 4, 5, 6], out)
