"""Seeded inputs shared by the tests: identical bits for the CPU oracle and the CUDA kernels."""
import numpy as np
import torch


def crandn(seed, *shape):
    """complex64 tensor with re, im ~ N(0,1) from a seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    re = torch.randn(*shape, generator=g, dtype=torch.float32)
    im = torch.randn(*shape, generator=g, dtype=torch.float32)
    return torch.complex(re, im)


def frandn(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def np_c(t):
    return np.ascontiguousarray(t.detach().cpu().numpy())


def rel_err(a, b):
    """max |a-b| / max(1, max|b|) over numpy arrays or torch tensors."""
    a = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    b = b.detach().cpu().numpy() if isinstance(b, torch.Tensor) else np.asarray(b)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / max(1.0, np.abs(b).max()))
