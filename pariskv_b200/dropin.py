"""Makes this package importable under the reference's module names, so a runtime written against the
reference (``from cache_hub.polar_cache import polar_cache``, ``from attn_hub import polar_decode_attn``)
picks up the B200 implementation without edits:

    import pariskv_b200.dropin as dropin
    dropin.install()
"""
import importlib
import sys

_SUBMODULES = [
    "cache_hub", "cache_hub.cache", "cache_hub.polar_cache", "cache_hub.polar_cache_adaptivek_varlen",
    "cache_hub.polar_cache_atten_value_indices_adaptive_k", "cache_hub.collision", "cache_hub.collision.collision",
    "cache_hub.collision_fused", "cache_hub.collision_fused.collison_interface", "cache_hub.topk", "cache_hub.rerank",
    "cache_hub.rerank.rerank", "cache_hub.adaptive_k_fused", "cache_hub.adaptive_k_fused.adaptive_topk",
    "cache_hub.gather", "cache_hub.gather.cpp_gather", "cache_hub.gather_trans", "cache_hub.gather_trans.trans_h2d",
    "attn_hub", "attn_hub.polar_attn",
]


def install(force: bool = False):
    """Register aliases in sys.modules.  Refuses to shadow an already imported reference module unless forced."""
    for name in _SUBMODULES:
        if name in sys.modules and not force:
            mod = sys.modules[name]
            if not getattr(mod, "__name__", "").startswith("pariskv_b200."):
                raise RuntimeError(f"{name} is already imported from elsewhere; pass force=True to replace it")
        sys.modules[name] = importlib.import_module("pariskv_b200." + name)
    return [n for n in _SUBMODULES]
