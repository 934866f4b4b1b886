from .cpp_gather import load_gather_ext  # noqa: F401
