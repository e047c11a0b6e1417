"""``gelib.SO3irrep``: Wigner D-matrices of SO(3) (SO3/SO3irrep.hpp:39-103 of GElib).

Host-side (numpy, float64) helper used by ``SO3part.apply`` and the equivariance tests; the
conventions are the reference's: z-y-z Euler angles read off the rotation matrix as in
SO3irrep::matrix (SO3/SO3irrep.hpp:45-66) and D[m1+l, m2+l] = d^l_{m2 m1}(beta) e^{i m1 alpha} e^{i m2 gamma}
(SO3/SO3irrep.hpp:69-77) with Wigner's little-d by the factorial sum (SO3/SO3irrep.hpp:80-103).
"""
import math

import numpy as np
import torch


def _littled(l, m1, m2, beta):
    x = 0.0
    c, s = math.cos(beta / 2), math.sin(beta / 2)
    pref = 0.5 * (math.lgamma(l + m1 + 1) + math.lgamma(l - m1 + 1) + math.lgamma(l + m2 + 1) + math.lgamma(l - m2 + 1))
    for k in range(max(0, m1 - m2), min(l + m1, l - m2) + 1):
        lg = pref - (math.lgamma(l + m1 - k + 1) + math.lgamma(k + 1) + math.lgamma(m2 - m1 + k + 1) +
                     math.lgamma(l - m2 - k + 1))
        sign = -1.0 if (m2 - m1 + k) % 2 else 1.0
        x += sign * math.exp(lg) * c ** (2 * l + m1 - m2 - 2 * k) * s ** (m2 - m1 + 2 * k)
    return x


def euler_zyz(R):
    """(alpha, beta, gamma) of a rotation matrix, with the reference's branch for beta near 0 or pi."""
    R = np.asarray(R, dtype=np.float64)
    r22 = min(1.0, max(-1.0, float(R[2, 2])))
    beta = math.acos(r22)
    if abs(r22) < 1 - 1e-6:
        alpha = math.atan2(R[0, 2], -R[1, 2])
        gamma = math.atan2(R[2, 0], R[2, 1])
    elif r22 >= 1 - 1e-6:
        alpha, gamma = math.atan2(R[1, 0], R[0, 0]), 0.0
    else:
        alpha, gamma = math.atan2(-R[1, 0], -R[0, 0]), 0.0
    return alpha, beta, gamma


class SO3irrep:

    def __init__(self, l):
        assert isinstance(l, int) and l >= 0
        self.l = l

    def matrix(self, R, beta=None, gamma=None):
        """D^l of a rotation given as an SO3element / 3x3 tensor, a list [alpha,beta,gamma] or three angles."""
        if beta is not None:
            alpha = R
        elif isinstance(R, (list, tuple)):
            alpha, beta, gamma = R
        else:
            alpha, beta, gamma = euler_zyz(R.detach().cpu().numpy())
        l = self.l
        M = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
        for m1 in range(-l, l + 1):
            for m2 in range(-l, l + 1):
                M[m1 + l, m2 + l] = _littled(l, m2, m1, beta) * np.exp(1j * m1 * alpha) * np.exp(1j * m2 * gamma)
        return torch.from_numpy(M.astype(np.complex64))

    def __repr__(self):
        return "<GElib::SO3irrep(l=%d)>" % self.l
