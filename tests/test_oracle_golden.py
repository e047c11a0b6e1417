"""Pins the CPU oracle (oracle/gelib_oracle.c) to independent known answers.

The reference ships no golden tensors (its tests are property tests on unseeded inputs), so the
pins are: sympy's Clebsch-Gordan coefficients, the coefficient matrix printed in the reference docs,
scipy's spherical harmonics, the Diag-is-the-diagonal-of-Full identity of the docs' listings, and the
reference's own property tests (equivariance, first-order gradient check) run on the oracle.
"""
import os

import numpy as np
import pytest
import torch

from util import crandn, np_c

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_cg_coefficients_match_sympy(oracle):
    tab = np.load(os.path.join(GOLD, "cg_sympy.npz"))["table"]
    err = 0.0
    for l1, l2, l, m1, m2, v in tab:
        err = max(err, abs(oracle.cg_coeff(int(l1), int(l2), int(l), int(m1), int(m2)) - v))
    assert err < 1e-12


def test_cg_matrix_doc_known_answer(oracle):
    # python/docs/source/SO3CG.rst:49-53 prints SO3CGmatrix(1,2,2) to four decimals
    M = np.load(os.path.join(GOLD, "doc_cg122.npz"))["matrix"]
    assert np.abs(oracle.cg_matrix(1, 2, 2) - M).max() < 5.1e-5


def test_cg_matrix_zero_off_band(oracle):
    C = oracle.cg_matrix(3, 2, 1)
    for m1 in range(-3, 4):
        for m2 in range(-2, 3):
            if abs(m1 + m2) > 1:
                assert C[m1 + 3, m2 + 2] == 0


def test_spharm_matches_scipy(oracle):
    z = np.load(os.path.join(GOLD, "spharm_scipy.npz"))
    pts = z["points"]
    X = np.ascontiguousarray(pts.T[None, :, :])  # (1, 3, 64): channels = points
    for L in range(9):
        R = np.zeros((1, 2 * L + 1, pts.shape[0]), np.complex64)
        oracle.add_spharm(R, X)
        ref = z["L%d" % L].T[None]
        assert np.abs(R - ref).max() < 5e-6, L  # float32 recursion vs float64 scipy


def test_spharm_z_axis_branch(oracle):
    # vx = vy = 0: only m = 0, value sqrt((2L+1)/4pi) whatever the sign of vz (SO3/SO3part.hpp:363-365)
    X = np.zeros((2, 3, 1), np.float32)
    X[0, 2, 0], X[1, 2, 0] = 1.5, -2.0
    for L in (0, 1, 3):
        R = np.zeros((2, 2 * L + 1, 1), np.complex64)
        oracle.add_spharm(R, X)
        want = np.zeros_like(R)
        want[:, L, 0] = np.float32(np.sqrt((2 * L + 1) / (4 * np.pi)))
        assert np.array_equal(R, want)


def test_spharm_accumulates_and_broadcasts(oracle):
    X = np.ascontiguousarray(np.random.default_rng(3).standard_normal((1, 3, 4)).astype(np.float32))
    R = np.ones((3, 5, 4), np.complex64)
    oracle.add_spharm(R, X)
    R1 = np.zeros((1, 5, 4), np.complex64)
    oracle.add_spharm(R1, X)
    assert np.allclose(R, 1 + np.broadcast_to(R1, R.shape))


@pytest.mark.parametrize("l1,l2,l,n1,n2", [(1, 2, 1, 2, 2), (2, 2, 2, 3, 3), (3, 1, 2, 4, 4)])
def test_diag_is_diagonal_of_full(oracle, l1, l2, l, n1, n2):
    # python/docs/source/SO3partB.rst:136-138 vs :177-179: Diag output = channels n*N2+n of the full product
    x, y = np_c(crandn(1, 3, 2 * l1 + 1, n1)), np_c(crandn(2, 3, 2 * l2 + 1, n2))
    full = np.zeros((3, 2 * l + 1, n1 * n2), np.complex64)
    oracle.add_CGproduct(full, x, y)
    diag = np.zeros((3, 2 * l + 1, n1), np.complex64)
    oracle.add_DiagCGproduct(diag, x, y)
    assert np.array_equal(diag, full[:, :, [n * n2 + n for n in range(n1)]])


def test_forward_matches_dense_einsum(oracle):
    # secondary check: r = einsum over the dense (L1,L2,L) coefficient tensor, in float64
    for (l1, l2, l) in [(2, 2, 2), (3, 4, 5), (1, 0, 1), (6, 6, 6)]:
        x, y = np_c(crandn(5, 2, 2 * l1 + 1, 3)), np_c(crandn(6, 2, 2 * l2 + 1, 2))
        r = np.zeros((2, 2 * l + 1, 6), np.complex64)
        oracle.add_CGproduct(r, x, y)
        C3 = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l + 1))
        for m1 in range(-l1, l1 + 1):
            for m2 in range(-l2, l2 + 1):
                if abs(m1 + m2) <= l:
                    C3[m1 + l1, m2 + l2, m1 + m2 + l] = oracle.cg_coeff(l1, l2, l, m1, m2)
        ref = np.einsum("abm,zai,zbj->zmij", C3, x.astype(np.complex128), y.astype(np.complex128)).reshape(2, 2 * l + 1, 6)
        assert np.abs(r - ref).max() < 2e-5


def test_offsets_and_accumulation(oracle):
    x, y = np_c(crandn(7, 2, 3, 2)), np_c(crandn(8, 2, 5, 3))
    r = np.ones((2, 5, 10), np.complex64)
    oracle.add_CGproduct(r, x, y, offs=3)
    r0 = np.zeros((2, 5, 6), np.complex64)
    oracle.add_CGproduct(r0, x, y)
    assert np.allclose(r[:, :, 3:9], 1 + r0) and np.all(r[:, :, :3] == 1) and np.all(r[:, :, 9:] == 1)


def test_rejects_what_the_reference_skips(oracle):
    x, y = np_c(crandn(1, 2, 3, 2)), np_c(crandn(2, 3, 3, 2))
    with pytest.raises(ValueError):  # batches 2 vs 3
        oracle.add_CGproduct(np.zeros((3, 3, 4), np.complex64), x, y)
    with pytest.raises(ValueError):  # l = 3 not in |1-1|..2
        oracle.add_CGproduct(np.zeros((2, 7, 4), np.complex64), x, x)
    with pytest.raises(ValueError):  # output row too short
        oracle.add_CGproduct(np.zeros((2, 3, 3), np.complex64), x, x)


def _odot(a, b):
    return float(np.sum(a.real.astype(np.float64) * b.real + a.imag.astype(np.float64) * b.imag))


@pytest.mark.parametrize("diag", [False, True])
@pytest.mark.parametrize("bx", [1, 3])
def test_gradients_first_order_exact(oracle, diag, bx):
    # the reference's gradient test (python/tests/ci_tests/test_SO3part.py:7-52): the op is bilinear, so
    # L(x+e) - L(x) = <e, grad_x> exactly; bx = 1 is the broadcast case (gradient summed over the batch)
    l1, l2, l, n = 2, 1, 2, 3
    B = 3
    x, y = np_c(crandn(11, bx, 2 * l1 + 1, n)), np_c(crandn(12, B, 2 * l2 + 1, n))
    nr = n if diag else n * n
    fwd = oracle.add_DiagCGproduct if diag else oracle.add_CGproduct
    b0 = oracle.add_DiagCGproduct_back0 if diag else oracle.add_CGproduct_back0
    b1 = oracle.add_DiagCGproduct_back1 if diag else oracle.add_CGproduct_back1
    g = np_c(crandn(13, B, 2 * l + 1, nr))

    def loss(xx, yy):
        r = np.zeros((B, 2 * l + 1, nr), np.complex64)
        fwd(r, xx, yy)
        return _odot(r, g)

    xg, yg = np.zeros_like(x), np.zeros_like(y)
    b0(xg, g, y)
    b1(yg, g, x)
    ex, ey = np_c(crandn(14, *x.shape)), np_c(crandn(15, *y.shape))
    assert abs(loss(x + ex, y) - loss(x, y) - _odot(ex, xg)) < 2e-3
    assert abs(loss(x, y + ey) - loss(x, y) - _odot(ey, yg)) < 2e-3


def test_vector_schedule_and_types(oracle):
    tau = {0: 2, 1: 2, 2: 1}
    t = oracle.cg_type(tau, tau, 2)
    # l=0: (0,0) (1,1) (2,2); l=1: (0,1) (1,0) (1,1) (1,2) (2,1) (2,2); l=2: (0,2) (1,1) (1,2) (2,0) (2,1) (2,2)
    assert t == {0: 4 + 4 + 1, 1: 4 + 4 + 4 + 2 + 2 + 1, 2: 2 + 4 + 2 + 2 + 2 + 1}
    tr = oracle.triples(tau, tau, set(t))
    # l1 ascending, then l2, then l; offsets run per output l
    assert tr[0] == (0, 0, 0, 0) and tr[1] == (0, 1, 1, 0) and tr[2] == (0, 2, 2, 0) and tr[3] == (1, 0, 1, 4)
    assert oracle.diag_type({0: 3, 1: 3}, {0: 3, 1: 3}, -1) == {0: 6, 1: 9, 2: 3}


def test_vector_product_equivariance(oracle):
    # python/tests/ci_tests/test_SO3vec.py:57-72 on the oracle, with the package's Wigner matrices
    import gelib_b200 as G
    torch.manual_seed(5)
    R = G.SO3element.random()
    tau = {0: 2, 1: 2, 2: 2}
    x = {l: np_c(crandn(20 + l, 2, 2 * l + 1, n)) for l, n in tau.items()}
    y = {l: np_c(crandn(30 + l, 2, 2 * l + 1, n)) for l, n in tau.items()}
    rt = oracle.cg_type(tau, tau, 2)

    def prod(a, b):
        r = {l: np.zeros((2, 2 * l + 1, n), np.complex64) for l, n in rt.items()}
        oracle.vec_cg(r, a, b)
        return r

    def rot(v):
        return {l: np.ascontiguousarray(np.einsum("ij,bjn->bin", G.SO3irrep(l).matrix(R).numpy(), p)) for l, p in v.items()}

    z, zr = rot(prod(x, y)), prod(rot(x), rot(y))
    for l in rt:
        assert np.allclose(z[l], zr[l], rtol=1e-3, atol=1e-4)


def test_threads_do_not_change_results(oracle):
    x, y = np_c(crandn(1, 16, 5, 4)), np_c(crandn(2, 16, 7, 4))
    r1, r2 = np.zeros((16, 7, 16), np.complex64), np.zeros((16, 7, 16), np.complex64)
    oracle.add_CGproduct(r1, x, y, nthreads=1)
    oracle.add_CGproduct(r2, x, y, nthreads=0)
    assert np.array_equal(r1, r2)
