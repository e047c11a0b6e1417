"""``gelib.SO3weights`` / ``SO3linear``: per-l complex mixing matrices (python/src/gelib/SO3weights.py:22-85).

In the reference the mixing is ``torch.matmul`` per part (python/src/gelib/SO3vec.py:174-177), not GElib code; here
``SO3vec.__mul__`` takes the library's mixing kernels on a CUDA device (at most 64 channels a side) and ``torch.matmul``
otherwise.
"""
import torch

from .SO3vec import SO3vec, SO3vecArr


class SO3weights:

    def __init__(self, *args):
        self.parts = list(args)

    @classmethod
    def zeros(cls, tau_in, tau_out, device='cpu'):
        return SO3weights(*[torch.zeros([tau_in[l], tau_out[l]], dtype=torch.complex64, device=device)
                            for l in tau_in])

    @classmethod
    def randn(cls, tau_in, tau_out, device='cpu'):
        return SO3weights(*[torch.randn([tau_in[l], tau_out[l]], dtype=torch.complex64, device=device)
                            for l in tau_in])

    def __repr__(self):
        return "<SO3weights " + ",".join("(%d,%d)" % (w.size(0), w.size(1)) for w in self.parts) + ">"

    def __str__(self):
        return "\n".join(str(w) for w in self.parts)


class SO3linear(torch.nn.Module):

    def __init__(self, tau_in, tau_out, device='cpu'):
        super().__init__()
        W = SO3weights.randn(tau_in, tau_out, device)
        self.weights = torch.nn.ParameterList([torch.nn.Parameter(w) for w in W.parts])
        self.W = SO3weights(*self.weights)

    def forward(self, x):
        assert isinstance(x, (SO3vec, SO3vecArr))
        return x * self.W
