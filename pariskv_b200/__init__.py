"""B200-native (sm_100a) ParisKV retrieval engine: key coding, collision counting, top-k, 4-bit rerank,
UVA gather and sparse decode attention behind the reference's cache / operator surface.

``pariskv_b200.ops`` holds the op entry points (C ABI underneath, no fallback); ``pariskv_b200.cache_hub``
and ``pariskv_b200.attn_hub`` mirror the reference's modules of the same names; ``pariskv_b200.dropin``
installs them under the reference's import names.
"""
from . import _lib  # noqa: F401

__all__ = ["ops", "build", "_lib"]
__version__ = "0.1.0"
