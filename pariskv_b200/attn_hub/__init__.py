from .polar_attn import polar_decode_attn, polar_prefill_attn  # noqa: F401
