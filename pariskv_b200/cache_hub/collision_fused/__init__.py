from .collison_interface import load_kernel_module, update_cache_cnt_cuda_interface  # noqa: F401
