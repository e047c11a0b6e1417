"""Generates tests/golden/*.npz -- independent known answers that pin the CPU oracle.

Run in the development container (needs sympy and scipy, which the GPU box also has, but the
fixtures are committed so no test depends on them):

    python tests/golden/make_golden.py

* cg_sympy.npz    Clebsch-Gordan coefficients <l1 m1 l2 m2 | l m1+m2> from sympy (exact rationals/surds
                  evaluated to float64) for every band entry of a set of (l1,l2,l) triples up to l = 8.
* spharm_scipy.npz orthonormal complex spherical harmonics from scipy.special.sph_harm_y (float64) at
                  seeded random points, L = 0..8, the cross-check the reference does by hand in
                  python/tests/test_spharm.py:11-31.
* doc_cg122.npz   the (1,2,2) coefficient matrix printed to 4 decimals in python/docs/source/SO3CG.rst:49-53
                  (typed in from the documentation, not computed).
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def cg_sympy():
    from sympy import S
    from sympy.physics.quantum.cg import CG
    triples = [(0, 0, 0), (1, 1, 0), (1, 1, 1), (1, 1, 2), (1, 2, 2), (2, 2, 0), (2, 2, 2), (2, 2, 4), (3, 4, 1),
               (3, 4, 5), (3, 4, 7), (4, 2, 3), (5, 5, 5), (6, 6, 0), (6, 6, 6), (6, 5, 3), (8, 8, 8), (8, 7, 2),
               (6, 6, 12), (0, 6, 6), (6, 0, 6)]
    rows = []
    for l1, l2, l in triples:
        for m1 in range(-l1, l1 + 1):
            for m2 in range(-l2, l2 + 1):
                if abs(m1 + m2) <= l:
                    v = float(CG(S(l1), S(m1), S(l2), S(m2), S(l), S(m1 + m2)).doit().evalf(30))
                    rows.append((l1, l2, l, m1, m2, v))
    a = np.array(rows, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "cg_sympy.npz"), table=a)
    print("cg_sympy:", a.shape)


def spharm_scipy():
    from scipy.special import sph_harm_y
    rng = np.random.default_rng(20240829)
    pts = rng.standard_normal((64, 3)).astype(np.float32)
    pts *= rng.uniform(0.5, 2.0, size=(64, 1)).astype(np.float32)
    x, y, z = (pts[:, i].astype(np.float64) for i in range(3))
    theta = np.arccos(z / np.sqrt(x * x + y * y + z * z))
    phi = np.arctan2(y, x)
    out = {}
    for L in range(9):
        out["L%d" % L] = np.stack([sph_harm_y(L, m, theta, phi) for m in range(-L, L + 1)], axis=1)
    np.savez_compressed(os.path.join(HERE, "spharm_scipy.npz"), points=pts, **out)
    print("spharm_scipy: 64 points, L=0..8")


def doc_cg122():
    M = np.array([[0.0000, -0.5774, -0.7071, -0.7071, -0.5774],
                  [0.8165, 0.4082, 0.0000, -0.4082, -0.8165],
                  [0.5774, 0.7071, 0.7071, 0.5774, 0.0000]])
    np.savez_compressed(os.path.join(HERE, "doc_cg122.npz"), matrix=M)


if __name__ == "__main__":
    cg_sympy()
    spharm_scipy()
    doc_cg122()
