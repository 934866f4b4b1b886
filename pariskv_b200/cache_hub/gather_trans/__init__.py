from .trans_h2d import h2d_gather_kv, h2d_gather_kv_packed  # noqa: F401
