"""Value-weighted adaptive-k cache, per-head (varlen) form: KV head h attends exactly k_h rows, k_h clamped to
[min_k, max_k] (mirror of the class in cache_hub/polar_cache_adaptivek_varlen.py; constructor extras at
:192-204, environment overrides ADAPTIVE_TOPK_MIN_K / ADAPTIVE_TOPK_MAX_K at :255-256).  The reference packs
indices, gathers into a packed buffer and calls a varlen attention over bs*kv_heads virtual sequences; here the
attention kernel takes the per-head counts directly."""
import os

from ._adaptive import AdaptiveKCache


class polar_cache(AdaptiveKCache):

    def __init__(self, *args, collision_ratio=None, candidate_ratio=None, enable_recall: bool = False,
                 adaptive_topk_threshold: float = 0.85, adaptive_topk_min_k=None, adaptive_topk_max_k=None,
                 adaptive_topk_max_k_ratio: float = 0.1, **kwargs):
        # the reference's class is offload-only (cache_hub/polar_cache_adaptivek_varlen.py:228-231); here the same
        # kernels read the store from pinned host memory or from HBM, so enable_offload=False is allowed as well
        super().__init__(*args, **kwargs)
        max_k = int(adaptive_topk_max_k if adaptive_topk_max_k is not None else os.environ.get("ADAPTIVE_TOPK_MAX_K", "800"))
        min_k = int(adaptive_topk_min_k if adaptive_topk_min_k is not None else os.environ.get("ADAPTIVE_TOPK_MIN_K", "100"))
        self.adaptive_topk_max_k_ratio = adaptive_topk_max_k_ratio
        self._init_adaptive(adaptive_topk_threshold, min_k, max_k, per_head=True)
