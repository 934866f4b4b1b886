"""Value-weighted adaptive-k cache, dense form: every KV head attends the first max_h k_h rows of its own
benefit ranking (mirror of the class in cache_hub/polar_cache_atten_value_indices_adaptive_k.py; constructor
extras at :164-175).  The row count stays on the device: no `.item()` per layer."""
import torch

from ._adaptive import AdaptiveKCache


class polar_cache(AdaptiveKCache):

    def __init__(self, *args, collision_ratio=None, candidate_ratio=None, enable_recall: bool = False,
                 adaptive_topk_threshold: float = 0.9, adaptive_topk_max_k: int = 2048, **kwargs):
        super().__init__(*args, **kwargs)
        max_k = adaptive_topk_max_k if adaptive_topk_max_k is not None else self.final_topk
        self.adaptive_topk_max_k = max_k
        self._init_adaptive(adaptive_topk_threshold, 1, max_k, per_head=False)
