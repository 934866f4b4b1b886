import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def bf16_from_bits(a):
    """uint16 numpy bit patterns -> torch.bfloat16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(torch.bfloat16)


def bits_of(t):
    """torch.bfloat16 tensor -> int16 tensor of bit patterns (for exact comparison)."""
    return t.detach().cpu().contiguous().view(torch.int16)


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))
    return load


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


def synth_keys(gen, bs, H, N, outliers=(7, 37, 71, 101), device="cpu"):
    """Keys with the distribution of the headline benchmark: N(0,1), four fixed channels x8,
    per-token lognormal(0, 0.5) norm factor, bf16."""
    z = torch.randn(bs, H, N, 128, generator=gen)
    z[..., list(outliers)] *= 8.0
    g = torch.exp(0.5 * torch.randn(bs, H, N, 1, generator=gen))
    return (z * g).to(torch.bfloat16).to(device)


def synth_queries(gen, keys, group=4):
    """One query per query head: 0.3 * (a random cached key, unit norm) + N(0, 1/128), renormalised."""
    bs, H, N, D = keys.shape
    pick = torch.randint(0, N, (bs, H, group), generator=gen)
    k = torch.stack([torch.stack([keys[b, h, pick[b, h]].float().cpu() for h in range(H)]) for b in range(bs)])
    q = 0.3 * k / k.norm(dim=-1, keepdim=True).clamp(min=1e-6) + torch.randn(bs, H, group, D, generator=gen) / D ** 0.5
    q = q / q.norm(dim=-1, keepdim=True)
    return q.to(torch.bfloat16).view(bs, 1, H * group, D).contiguous()


def srht_signs(seed=42):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 2, (128,), generator=g).to(torch.bfloat16) * 2 - 1
