"""Host-side K/V row gather with the reference's surface (cache_hub/gather/cpp_gather.py:10-41)."""
from types import SimpleNamespace

import torch

from ... import torch_ops  # noqa: F401  (registers torch.ops.pariskv.*)


def load_gather_ext(verbose: bool = False):
    return SimpleNamespace(gather_kv_out_cpu=lambda src, index, out: torch.ops.pariskv.gather(src, index, out))
