"""ctypes binding of ``libpariskv_b200.so`` (the C ABI declared in ``include/pariskv_b200.h``).

There is no fallback: if the library cannot be loaded every op raises.  Tensors cross the boundary
as ``pk_tensor`` descriptors (data pointer, dtype tag, shape, strides); nothing torch-specific is
visible to the C side.
"""
import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpariskv_b200.so")

PK_MAX_DIMS = 6
PK_U8, PK_I32, PK_I64, PK_F32, PK_BF16 = range(5)
_DTYPES = {torch.uint8: PK_U8, torch.int32: PK_I32, torch.int64: PK_I64, torch.float32: PK_F32,
           torch.bfloat16: PK_BF16}


class PkTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * PK_MAX_DIMS), ("stride", ctypes.c_int64 * PK_MAX_DIMS)]


class PkZoneSchedule(ctypes.Structure):
    _fields_ = [("n_rows", ctypes.c_int32), ("n_tiers", ctypes.c_int32), ("bound", ctypes.c_int64 * 3),
                ("candidate_ratio", ctypes.c_double * 4), ("collision_ratio", ctypes.c_double * 4),
                ("tier_ratio", ctypes.c_double * 8)]


TP = ctypes.POINTER(PkTensor)


class PkRetrieveArgs(ctypes.Structure):
    _fields_ = [("queries", TP), ("signs", TP), ("mag_centers", TP), ("codebook", TP), ("key_block_weight", TP),
                ("key_4bit", TP), ("cluster_key_counts", TP), ("tier_counts", ctypes.POINTER(ctypes.c_int64)),
                ("n_tiers", ctypes.c_int32), ("phase", ctypes.c_int32), ("C", ctypes.c_int64), ("K", ctypes.c_int64),
                ("kv_len", TP), ("schedule", ctypes.POINTER(PkZoneSchedule)), ("local_hist", TP), ("shard_hist", TP),
                ("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("final_indices", TP), ("n_sel", TP),
                ("cand", TP), ("n_cand", TP), ("scores_f32", TP), ("q_blocks", TP), ("q_norm", TP),
                ("query_avg", TP), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
                ("queries_settled", ctypes.c_int32), ("reserved", ctypes.c_int32)]


_I64, _INT, _F32, _VP = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_I64P = ctypes.POINTER(ctypes.c_int64)
_U64 = ctypes.c_uint64
_U64P = ctypes.POINTER(ctypes.c_uint64)

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "pk_version": (_INT, []),
    "pk_last_error": (ctypes.c_char_p, []),
    "pk_launch_count": (_I64, []),
    "pk_set_pdl": (_INT, [_INT]),
    "pk_timing_enable": (_INT, [_INT]),
    "pk_timing_read": (_INT, [ctypes.POINTER(ctypes.c_double), _I64P, _INT]),
    "pk_timing_read_graph": (_INT, [ctypes.POINTER(ctypes.c_double), _I64P, _INT]),
    "pk_timing_clear_graph": (_INT, []),
    "pk_encode_keys": (_INT, [TP, TP, TP, TP, TP, TP, _VP]),
    "pk_count_clusters": (_INT, [TP, TP, _INT, _VP]),
    "pk_query_prep": (_INT, [TP, TP, TP, TP, TP, _VP]),
    "pk_rank_clusters": (_INT, [TP, TP, _VP]),
    "pk_collision_workspace_bytes": (_I64, [_I64, _I64, _I64, _I64]),
    "pk_collision_fused": (_INT, [TP, TP, TP, _I64P, _INT, TP, _VP, _I64, _VP]),
    "pk_collision": (_INT, [TP, TP, TP, TP, _VP, _I64, _VP]),
    "pk_collision_fused_static_max_triples": (_I64, []),
    "pk_collision_fused_static": (_INT, [TP, TP, TP, _I64P, _INT, TP, _VP]),
    "pk_topk": (_INT, [TP, _I64, TP, _INT, _VP]),
    "pk_final_topk": (_INT, [TP, TP, _I64, TP, _VP]),
    "pk_adaptive_topk": (_INT, [TP, TP, _F32, TP, TP, TP, TP, _I64, _F32, _I64, _I64, _I64, TP, TP, _VP]),
    "pk_rerank": (_INT, [TP, TP, TP, TP, TP, TP, TP, TP, TP, _VP]),
    "pk_h2d_gather_kv": (_INT, [TP, TP, TP, TP, TP, _VP]),
    "pk_h2d_gather_kv_packed": (_INT, [TP, TP, TP, TP, TP, TP, TP, _I64, _I64, _VP]),
    "pk_gather_kv_out_cpu": (_INT, [TP, TP, TP, _INT]),
    "pk_attention_workspace_bytes": (_I64, [_I64, _I64, _I64]),
    "pk_sparse_attention": (_INT, [TP, TP, TP, _I64, TP, _I64, TP, TP, TP, TP, _I64, _F32, TP, TP, _VP, _I64, _VP]),
    "pk_append_kv": (_INT, [TP, TP, TP, TP, _I64, TP, _I64, _VP]),
    "pk_append_encode": (_INT, [TP] * 16 + [_I64, _I64, _VP]),
    "pk_retrieve_workspace_bytes": (_I64, [_I64, _I64, _I64, _I64]),
    "pk_retrieve": (_INT, [TP, TP, TP, TP, TP, TP, TP, _I64P, _INT, _I64, _I64, TP, TP, TP, TP, TP, TP, _VP, _I64,
                           _VP]),
    "pk_retrieve_ex": (_INT, [ctypes.POINTER(PkRetrieveArgs), _VP]),
    "pk_zone_max_candidates": (_I64, [ctypes.POINTER(PkZoneSchedule), _I64]),
    "pk_shard_pack_topk": (_INT, [TP, TP, TP, _I64, TP, TP, TP, _VP]),
    "pk_shard_unpack_topk": (_INT, [TP, TP, TP, _VP]),
    "pk_shard_owned_rows": (_INT, [TP, _I64, _I64, TP, TP, _VP]),
    "pk_shard_pack_partial": (_INT, [TP, TP, TP, _VP]),
    "pk_shard_merge_partial": (_INT, [TP, TP, _VP]),
    "pk_shard_exchange_topk": (_INT, [TP, TP, TP, _I64, TP, TP, _U64P, _INT, _INT, _I64, _I64, _VP, _VP]),
    "pk_shard_collect_topk": (_INT, [_U64, _I64, _I64, _VP, _INT, _I64, TP, TP, _VP]),
    "pk_shard_exchange_partial": (_INT, [TP, TP, _U64P, _INT, _INT, _I64, _I64, _VP, _VP]),
    "pk_shard_collect_partial": (_INT, [_U64, _I64, _I64, _VP, _INT, TP, _VP]),
    "pk_tp_allreduce": (_INT, [TP, TP, TP, _U64P, _INT, _INT, _I64, _I64, _I64, _VP, TP, TP, ctypes.c_double, _VP]),
    "pk_tp_allgather": (_INT, [TP, TP, _U64P, _INT, _INT, _I64, _I64, _I64, _VP, _VP]),
    "pk_qk_norm_rope": (_INT, [TP, TP, TP, TP, TP, ctypes.c_double, _VP]),
    "pk_add_rmsnorm": (_INT, [TP, TP, TP, TP, TP, ctypes.c_double, _VP]),
    "pk_silu_mul": (_INT, [TP, TP, _VP]),
    "pk_gemv": (_INT, [TP, TP, TP, _INT, _VP]),
}

_lib = None


def load():
    """Load the library (once).  Raises RuntimeError with the build hint if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m pariskv_b200.build` "
                "(there is no fallback path for the CUDA kernels)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def desc(t):
    """torch.Tensor (or None) -> pk_tensor (or None).  Keep the tensor alive while the call runs."""
    if t is None:
        return None
    if t.dim() > PK_MAX_DIMS:
        raise ValueError("too many dimensions")
    if t.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {t.dtype}")
    d = PkTensor()
    d.data = t.data_ptr()
    d.dtype = _DTYPES[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def ref(d):
    return ctypes.byref(d) if d is not None else None


def ptr(d):
    """pk_tensor (or None) -> a typed pointer for a structure field (NULL for None)."""
    return ctypes.pointer(d) if d is not None else None


def zone_schedule(bounds, candidate_ratios, collision_ratios, tier_ratios):
    """The ratio schedule as the C structure: row i applies to zones shorter than bounds[i], the last row to the rest."""
    s = PkZoneSchedule()
    s.n_rows, s.n_tiers = len(candidate_ratios), len(tier_ratios)
    if len(bounds) != s.n_rows - 1 or len(collision_ratios) != s.n_rows or not 1 <= s.n_rows <= 4 or not 1 <= s.n_tiers <= 8:
        raise ValueError("schedule: need n-1 bounds for n <= 4 rows and 1..8 tier ratios")
    for i, b in enumerate(bounds):
        s.bound[i] = int(b)
    for i in range(s.n_rows):
        s.candidate_ratio[i], s.collision_ratio[i] = float(candidate_ratios[i]), float(collision_ratios[i])
    for i, r in enumerate(tier_ratios):
        s.tier_ratio[i] = float(r)
    return s


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check(rc):
    if rc != 0:
        msg = load().pk_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"pariskv_b200 error {rc}: {msg}")


def u64_array(values):
    return (ctypes.c_uint64 * len(values))(*[int(v) for v in values])


def i64_array(values):
    arr = (ctypes.c_int64 * len(values))(*[int(v) for v in values])
    return arr


def launch_count() -> int:
    return int(load().pk_launch_count())


STAGES = ["query_prep", "rank_table", "collision", "select_rerank", "final_topk", "attention", "attention_merge",
          "encode", "topk", "rerank", "uva_gather", "count_clusters", "append", "glue", "tp_reduce",
          "shard_send", "shard_recv", "shard_owned", "hist_reduce", "gemv", "adaptive_topk"]


def set_pdl(on: bool):
    """Launch the kernels of a decode step with programmatic dependent launch (see pk_set_pdl)."""
    check(load().pk_set_pdl(int(bool(on))))


def timing_enable(on: bool):
    check(load().pk_timing_enable(int(bool(on))))


def timing_read():
    """-> {stage: (total_ms, launches)} for every stage recorded since the last read."""
    n = len(STAGES)
    ms = (ctypes.c_double * n)()
    cnt = (ctypes.c_int64 * n)()
    check(load().pk_timing_read(ms, cnt, n))
    return {STAGES[i]: (float(ms[i]), int(cnt[i])) for i in range(n) if cnt[i]}


def timing_read_graph():
    """-> {stage: (total_ms, launches)} of the last replay of the graphs captured while timing was enabled."""
    n = len(STAGES)
    ms = (ctypes.c_double * n)()
    cnt = (ctypes.c_int64 * n)()
    check(load().pk_timing_read_graph(ms, cnt, n))
    return {STAGES[i]: (float(ms[i]), int(cnt[i])) for i in range(n) if cnt[i]}


def timing_clear_graph():
    check(load().pk_timing_clear_graph())
