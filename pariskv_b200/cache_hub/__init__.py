from .polar_cache import polar_cache  # noqa: F401
