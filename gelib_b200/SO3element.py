"""``gelib.SO3element``: a 3x3 rotation matrix as a torch tensor (python/src/gelib/SO3element.py of GElib).

Host-side helper for the equivariance tests and for ``SO3part.apply``; nothing here is on the
Clebsch-Gordan hot path.
"""
import torch


class SO3element(torch.Tensor):

    @staticmethod
    def __new__(cls, t):
        return torch.Tensor._make_subclass(cls, t.detach() if isinstance(t, torch.Tensor) else torch.as_tensor(t))

    def __init__(self, t):
        pass

    @classmethod
    def identity(cls):
        return SO3element(torch.eye(3))

    @classmethod
    def random(cls, generator=None):
        """A Haar-random rotation: orthonormalise a Gaussian 3x3 matrix and fix det = +1
        (the construction of SO3element::random, SO3/SO3element.hpp:45-57)."""
        while True:
            A = torch.randn(3, 3, dtype=torch.float64, generator=generator)
            Q, R = torch.linalg.qr(A)
            if torch.abs(torch.diagonal(R)).min() > 1e-8:
                break
        Q = Q * torch.sign(torch.diagonal(R))  # unique factorisation, keeps the distribution uniform
        if torch.det(Q) < 0:
            Q = -Q
        return SO3element(Q.to(torch.float32))

    def __mul__(self, y):
        assert isinstance(y, SO3element)
        return SO3element(torch.matmul(self, y))

    def inv(self):
        return SO3element(self.t())
