"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on identical seeded inputs.

Tolerances (relative to max(1, max|reference|)): 1e-5 for single triples and vectors up to maxl 5,
1e-4 for accumulations over maxl >= 6 -- the tolerances the scope contract names.
"""
import numpy as np
import pytest
import torch

from util import crandn, frandn, np_c, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5
TOL_BIG = 1e-4


@pytest.fixture(scope="module")
def G():
    import gelib_b200
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    gelib_b200._lib.lib()  # fail loudly if the library was not built
    return gelib_b200


@pytest.fixture
def opt(G):
    """Pins kernel choices / test switches of the library for one test and restores the defaults afterwards."""
    touched = []

    def set_(name, value):
        touched.append(name)
        G._lib.set_option(name, value)

    yield set_
    for name in touched:
        G._lib.set_option(name, "0" if name == "inject_timeout" else "auto")  # "auto" = on for pair_tma, narrow1


def dev(t):
    return t.cuda()


def view(G, t):
    return G.backend.SO3part.view(t)


# ---- single triple, forward ------------------------------------------------------------------------

PART_CASES = [
    # (B, l1, l2, l, n1, n2)
    (3, 1, 1, 1, 1, 1), (2, 2, 2, 2, 2, 2), (4, 1, 2, 3, 3, 5), (1, 4, 4, 4, 8, 8), (5, 3, 4, 1, 7, 2),
    (3, 0, 3, 3, 4, 6), (3, 3, 0, 3, 6, 4), (2, 2, 2, 0, 32, 32), (9, 2, 2, 2, 32, 32), (3, 3, 4, 5, 64, 64),
    (2, 6, 6, 6, 32, 32), (17, 1, 3, 2, 1, 16), (5, 4, 2, 3, 16, 1), (2, 2, 1, 2, 33, 31), (2, 8, 8, 8, 4, 4),
    (1, 5, 5, 10, 3, 3), (2, 1, 1, 2, 40, 24),
]


@pytest.mark.parametrize("B,l1,l2,l,n1,n2", PART_CASES)
def test_part_forward(G, oracle, B, l1, l2, l, n1, n2):
    x, y = crandn(1, B, 2 * l1 + 1, n1), crandn(2, B, 2 * l2 + 1, n2)
    want = np.zeros((B, 2 * l + 1, n1 * n2), np.complex64)
    oracle.add_CGproduct(want, np_c(x), np_c(y))
    r = torch.zeros(B, 2 * l + 1, n1 * n2, dtype=torch.complex64, device="cuda")
    view(G, r).add_CGproduct(view(G, dev(x)), view(G, dev(y)))
    assert rel_err(r, want) < TOL
    # overwrite into garbage gives the same thing
    r2 = torch.full_like(r, 7 + 3j)
    view(G, r2).add_CGproduct(view(G, dev(x)), view(G, dev(y)), overwrite=True)
    assert rel_err(r2, want) < TOL


@pytest.mark.parametrize("B,l1,l2,l,n1,n2", PART_CASES)
def test_part_backward(G, oracle, B, l1, l2, l, n1, n2):
    x, y = crandn(1, B, 2 * l1 + 1, n1), crandn(2, B, 2 * l2 + 1, n2)
    g = crandn(3, B, 2 * l + 1, n1 * n2)
    xg_w, yg_w = np.zeros(x.shape, np.complex64), np.zeros(y.shape, np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(g), np_c(y))
    oracle.add_CGproduct_back1(yg_w, np_c(g), np_c(x))
    xd, yd, gd = dev(x), dev(y), dev(g)
    xg, yg = torch.zeros_like(xd), torch.zeros_like(yd)
    G.backend.SO3part.add_CGproduct_back01(view(G, xg), view(G, yg), view(G, gd), view(G, xd), view(G, yd))
    scale = 1e-5 * max(1.0, np.sqrt(n1 * n2))  # sums of up to (2l+1)*n terms of size O(1)
    assert rel_err(xg, xg_w) < max(TOL, scale) and rel_err(yg, yg_w) < max(TOL, scale)
    # the separate entry points agree with the fused one and accumulate into their output
    xg1, yg1 = torch.ones_like(xd), torch.ones_like(yd)
    view(G, xg1).add_CGproduct_back0(view(G, gd), view(G, yd))
    view(G, yg1).add_CGproduct_back1(view(G, gd), view(G, xd))
    assert rel_err(xg1 - 1, xg_w) < max(TOL, scale) and rel_err(yg1 - 1, yg_w) < max(TOL, scale)


def test_part_offsets_accumulation_and_untouched_channels(G, oracle):
    B, l1, l2, l, n1, n2 = 3, 2, 1, 2, 4, 6
    x, y = crandn(4, B, 5, n1), crandn(5, B, 3, n2)
    r0 = crandn(6, B, 5, 40)
    want = np_c(r0).copy()
    oracle.add_CGproduct(want, np_c(x), np_c(y), offs=10)
    r = dev(r0)
    view(G, r).add_CGproduct(view(G, dev(x)), view(G, dev(y)), 10)
    assert rel_err(r, want) < TOL
    assert torch.equal(r[:, :, :10].cpu(), r0[:, :, :10]) and torch.equal(r[:, :, 34:].cpu(), r0[:, :, 34:])
    # odd offset (no 16-byte alignment) and gradients through the same offset
    want = np_c(r0).copy()
    oracle.add_CGproduct(want, np_c(x), np_c(y), offs=7)
    r = dev(r0)
    view(G, r).add_CGproduct(view(G, dev(x)), view(G, dev(y)), 7)
    assert rel_err(r, want) < TOL
    xg_w = np.zeros(x.shape, np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(r0), np_c(y), offs=7)
    xg = torch.zeros(x.shape, dtype=torch.complex64, device="cuda")
    view(G, xg).add_CGproduct_back0(view(G, dev(r0)), view(G, dev(y)), 7)
    assert rel_err(xg, xg_w) < TOL


def test_broadcast_batch_forward_and_summed_gradient(G, oracle):
    # x has batch 1: used for every cell forward, gradient summed over the batch backward
    # (python/tests/ci_tests/test_SO3part.py:31-52; the reference's GPU kernels race here)
    B, l1, l2, l, n = 6, 2, 2, 2, 4
    x, y, g = crandn(1, 1, 5, n), crandn(2, B, 5, n), crandn(3, B, 5, n * n)
    want = np.zeros((B, 5, n * n), np.complex64)
    oracle.add_CGproduct(want, np_c(x), np_c(y))
    r = torch.zeros(B, 5, n * n, dtype=torch.complex64, device="cuda")
    view(G, r).add_CGproduct(view(G, dev(x)), view(G, dev(y)))
    assert rel_err(r, want) < TOL
    xg_w, yg_w = np.zeros(x.shape, np.complex64), np.zeros(y.shape, np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(g), np_c(y))
    oracle.add_CGproduct_back1(yg_w, np_c(g), np_c(x))
    xg, yg = torch.zeros(x.shape, dtype=torch.complex64, device="cuda"), torch.zeros(y.shape, dtype=torch.complex64, device="cuda")
    G.backend.SO3part.add_CGproduct_back01(view(G, xg), view(G, yg), view(G, dev(g)), view(G, dev(x)), view(G, dev(y)))
    assert rel_err(xg, xg_w) < 5e-5 and rel_err(yg, yg_w) < TOL


def test_strided_views(G, oracle):
    # rows and channels taken out of larger buffers: row stride != n, channel stride != 1
    B, l1, l2, l, n1, n2 = 3, 1, 2, 2, 3, 4
    xbuf, ybuf = crandn(1, B, 3, 2 * n1), crandn(2, B, 7, n2)
    x, y = xbuf[:, :, ::2], ybuf[:, 1:6, :]
    rbuf = torch.zeros(B, 5, n1 * n2 + 5, dtype=torch.complex64, device="cuda")
    want = np.zeros((B, 5, n1 * n2), np.complex64)
    oracle.add_CGproduct(want, np_c(x), np_c(y))
    xd, yd = dev(xbuf)[:, :, ::2], dev(ybuf)[:, 1:6, :]
    view(G, rbuf[:, :, 2:2 + n1 * n2]).add_CGproduct(view(G, xd), view(G, yd))
    assert rel_err(rbuf[:, :, 2:2 + n1 * n2], want) < TOL and rbuf[:, :, :2].abs().max() == 0
    g = crandn(3, B, 5, n1 * n2)
    xg_w = np.zeros((B, 3, n1), np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(g), np_c(y))
    xgbuf = torch.zeros(B, 3, 2 * n1, dtype=torch.complex64, device="cuda")
    view(G, xgbuf[:, :, ::2]).add_CGproduct_back0(view(G, dev(g)), view(G, yd))
    assert rel_err(xgbuf[:, :, ::2], xg_w) < TOL and xgbuf[:, :, 1::2].abs().max() == 0


def test_grid_cells_and_grid_broadcast(G, oracle):
    # SO3partArr layout (b, g0, g1, 2l+1, n); y has no grid and is broadcast over it (core/Gpart.hpp:366-432)
    B, g0, g1, n = 2, 3, 2, 4
    x, y = crandn(1, B, g0, g1, 3, n), crandn(2, B, 5, n)
    r = torch.zeros(B, g0, g1, 5, n * n, dtype=torch.complex64, device="cuda")
    view(G, r).add_CGproduct(view(G, dev(x)), view(G, dev(y)))
    want = np.zeros((B * g0 * g1, 5, n * n), np.complex64)
    yx = y[:, None, None].expand(B, g0, g1, 5, n).reshape(-1, 5, n)
    oracle.add_CGproduct(want, np_c(x.reshape(-1, 3, n)), np_c(yx))
    assert rel_err(r.reshape(-1, 5, n * n), want) < TOL
    # gradient wrt the grid-less y sums over the grid
    g = crandn(3, B, g0, g1, 5, n * n)
    yg = torch.zeros(B, 5, n, dtype=torch.complex64, device="cuda")
    view(G, yg).add_CGproduct_back1(view(G, dev(g)), view(G, dev(x)))
    yg_w = np.zeros((B * g0 * g1, 5, n), np.complex64)
    oracle.add_CGproduct_back1(yg_w, np_c(g.reshape(-1, 5, n * n)), np_c(x.reshape(-1, 3, n)))
    assert rel_err(yg, yg_w.reshape(B, g0 * g1, 5, n).sum(1)) < 5e-5


def test_skipped_calls_do_nothing(G, capfd):
    r = torch.zeros(2, 7, 4, dtype=torch.complex64, device="cuda")
    x = dev(crandn(1, 2, 3, 2))
    view(G, r).add_CGproduct(view(G, x), view(G, x))  # l = 3 is not in 1 x 1
    assert "skipped" in capfd.readouterr().err and r.abs().max() == 0
    with pytest.raises(RuntimeError, match="N1==N2"):
        view(G, r[:, :3]).add_DiagCGproduct(view(G, x), view(G, dev(crandn(1, 2, 3, 3))))


def test_empty_batch(G):
    r = torch.zeros(0, 5, 4, dtype=torch.complex64, device="cuda")
    x = torch.zeros(0, 5, 2, dtype=torch.complex64, device="cuda")
    view(G, r).add_CGproduct(view(G, x), view(G, x))
    assert r.numel() == 0


# ---- diagonal products -------------------------------------------------------------------------------

@pytest.mark.parametrize("B,l1,l2,l,n", [(3, 1, 1, 1, 1), (2, 2, 2, 2, 8), (4, 3, 4, 2, 5), (2, 4, 4, 8, 32),
                                         (3, 6, 6, 6, 40), (5, 0, 2, 2, 128), (2, 8, 8, 0, 3)])
def test_part_diag(G, oracle, B, l1, l2, l, n):
    x, y, g = crandn(1, B, 2 * l1 + 1, n), crandn(2, B, 2 * l2 + 1, n), crandn(3, B, 2 * l + 1, n)
    want = np.zeros((B, 2 * l + 1, n), np.complex64)
    oracle.add_DiagCGproduct(want, np_c(x), np_c(y))
    r = torch.zeros(B, 2 * l + 1, n, dtype=torch.complex64, device="cuda")
    view(G, r).add_DiagCGproduct(view(G, dev(x)), view(G, dev(y)))
    assert rel_err(r, want) < TOL
    xg_w, yg_w = np.zeros(x.shape, np.complex64), np.zeros(y.shape, np.complex64)
    oracle.add_DiagCGproduct_back0(xg_w, np_c(g), np_c(y))
    oracle.add_DiagCGproduct_back1(yg_w, np_c(g), np_c(x))
    xg, yg = torch.zeros(x.shape, dtype=torch.complex64, device="cuda"), torch.zeros(y.shape, dtype=torch.complex64, device="cuda")
    G.backend.SO3part.add_DiagCGproduct_back01(view(G, xg), view(G, yg), view(G, dev(g)), view(G, dev(x)), view(G, dev(y)))
    assert rel_err(xg, xg_w) < TOL and rel_err(yg, yg_w) < TOL
    xg1 = torch.zeros_like(xg)
    view(G, xg1).add_DiagCGproduct_back0(view(G, dev(g)), view(G, dev(y)))
    assert rel_err(xg1, xg_w) < TOL


# ---- vectors: all triples in one launch -----------------------------------------------------------------

def _vec_inputs(tau_x, tau_y, B, seed):
    x = {l: crandn(seed + l, B, 2 * l + 1, n) for l, n in tau_x.items()}
    y = {l: crandn(seed + 100 + l, B, 2 * l + 1, n) for l, n in tau_y.items()}
    return x, y


VEC_CASES = [
    # (B, tau_x, tau_y, maxl, tol)
    (3, {0: 1, 1: 1, 2: 1}, {0: 1, 1: 1, 2: 1}, 2, TOL),
    (2, {l: 4 for l in range(5)}, {l: 4 for l in range(5)}, 4, TOL),
    (5, {0: 3, 2: 2}, {1: 5, 3: 1}, -1, TOL),
    (2, {l: 32 for l in range(4)}, {l: 32 for l in range(4)}, 3, TOL),
    (2, {l: 8 for l in range(7)}, {l: 8 for l in range(7)}, 6, TOL_BIG),
    (9, {l: 1 for l in range(7)}, {l: 16 for l in range(7)}, 6, TOL_BIG),
    (2, {1: 64}, {2: 64}, -1, TOL),
    (2, {3: 64}, {4: 64}, -1, TOL_BIG),   # the SO3part benchmark configuration l1=3 x l2=4 -> l=1..7 as one vector call
]


@pytest.mark.parametrize("B,tau_x,tau_y,maxl,tol", VEC_CASES)
@pytest.mark.parametrize("diag", [False, True])
def test_vec_product_and_gradients(G, oracle, B, tau_x, tau_y, maxl, tol, diag):
    if diag and len(set(tau_x.values()) | set(tau_y.values())) != 1:
        pytest.skip("the diagonal product needs equal channel counts")
    x, y = _vec_inputs(tau_x, tau_y, B, 10)
    tau_r = oracle.cg_type(tau_x, tau_y, maxl, diag)
    want = {l: np.zeros((B, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, {l: np_c(t) for l, t in x.items()}, {l: np_c(t) for l, t in y.items()}, diag)

    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    assert (xv.get_tau().DiagCGproduct(yv.get_tau(), maxl) if diag else xv.get_tau().CGproduct(yv.get_tau(), maxl)).get_parts() == tau_r
    rparts = [torch.zeros(B, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    rv = G.backend.SO3vec.view(rparts)
    (rv.addDiagCGproduct if diag else rv.addCGproduct)(xv, yv)
    for p, (l, w) in zip(rparts, want.items()):
        assert rel_err(p, w) < tol, l

    g = {l: crandn(300 + l, B, 2 * l + 1, n) for l, n in tau_r.items()}
    gn = {l: np_c(t) for l, t in g.items()}
    xg_w = {l: np.zeros(t.shape, np.complex64) for l, t in x.items()}
    yg_w = {l: np.zeros(t.shape, np.complex64) for l, t in y.items()}
    oracle.vec_cg_back0(xg_w, gn, {l: np_c(t) for l, t in y.items()}, diag)
    oracle.vec_cg_back1(yg_w, gn, {l: np_c(t) for l, t in x.items()}, diag)
    gv = G.backend.SO3vec.view([dev(t) for t in g.values()])
    xg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
    yg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
    f = G.backend.SO3vec.addDiagCGproduct_back01 if diag else G.backend.SO3vec.addCGproduct_back01
    f(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
    gtol = max(tol, TOL_BIG)  # gradient entries are sums of thousands of O(1) terms
    for p, w in zip(xg, xg_w.values()):
        assert rel_err(p, w) < gtol
    for p, w in zip(yg, yg_w.values()):
        assert rel_err(p, w) < gtol
    # the two separate gradient entry points
    xg2 = [torch.zeros_like(t) for t in xg]
    yg2 = [torch.zeros_like(t) for t in yg]
    xg2v, yg2v = G.backend.SO3vec.view(xg2), G.backend.SO3vec.view(yg2)
    (xg2v.addDiagCGproduct_back0 if diag else xg2v.addCGproduct_back0)(gv, yv)
    (yg2v.addDiagCGproduct_back1 if diag else yg2v.addCGproduct_back1)(gv, xv)
    for p, w in zip(xg2, xg_w.values()):
        assert rel_err(p, w) < gtol
    for p, w in zip(yg2, yg_w.values()):
        assert rel_err(p, w) < gtol


def test_vec_backward_is_reproducible_to_rounding(G):
    B, tau = 4, {l: 8 for l in range(4)}
    x, y = _vec_inputs(tau, tau, B, 50)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    tau_r = xv.get_tau().CGproduct(yv.get_tau(), 3).get_parts()
    gv = G.backend.SO3vec.view([dev(crandn(70 + l, B, 2 * l + 1, n)) for l, n in tau_r.items()])
    outs = []
    for _ in range(2):
        xg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
        yg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
        G.backend.SO3vec.addCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
        outs.append(xg + yg)
    # warps add into the shared-memory gradient rows with atomics in no fixed order: equal up to rounding
    for a, b in zip(*outs):
        assert rel_err(a, b) < 2e-6


# ---- the tensor-core (tcgen05) backward kernel: opt-in, for channel counts that are multiples of 32 ----------

TC_CASES = [
    (3, {l: 32 for l in range(4)}, {l: 32 for l in range(4)}, 3, TOL_BIG),
    (2, {l: 32 for l in range(7)}, {l: 32 for l in range(7)}, 6, TOL_BIG),   # the headline channel layout
    (2, {1: 64}, {2: 64}, -1, TOL_BIG),                                     # four 32 x 32 tiles per slab
    (2, {0: 32, 1: 64}, {1: 32, 3: 96}, 4, TOL_BIG),                        # mixed channel counts
    (1, {0: 32}, {0: 32}, 0, TOL_BIG),                                      # a single slab, three idle warps
]


@pytest.mark.parametrize("B,tau_x,tau_y,maxl,tol", TC_CASES + [
    (3, {l: 32 for l in range(9)}, {l: 32 for l in range(9)}, 8, TOL_BIG),   # 17 accumulator rows, groups of 5..9 l split in two
    (2, {2: 32, 5: 64}, {0: 64, 4: 32, 6: 32}, 5, TOL_BIG),                 # gaps in l, truncated output
])
@pytest.mark.parametrize("bcast_y", [False, True])
@pytest.mark.parametrize("kernel", ["pair!", "tcgen05!", "simt"])
def test_vec_backward_named_kernel(G, oracle, opt, B, tau_x, tau_y, maxl, tol, bcast_y, kernel):
    if kernel == "tcgen05!" and max(list(tau_x) + list(tau_y)) > 7:
        pytest.skip("the tcgen05 backward covers l <= 7")
    opt("bwd", kernel)  # "!": fail instead of falling back to another kernel
    x, y = _vec_inputs(tau_x, tau_y, B, 90)
    if bcast_y:
        y = {l: t[:1].contiguous() for l, t in y.items()}
    tau_r = oracle.cg_type(tau_x, tau_y, maxl, False)
    g = {l: crandn(400 + l, B, 2 * l + 1, n) for l, n in tau_r.items()}
    gn = {l: np_c(t) for l, t in g.items()}
    xg_w = {l: np.zeros(t.shape, np.complex64) for l, t in x.items()}
    yg_w = {l: np.zeros(t.shape, np.complex64) for l, t in y.items()}
    oracle.vec_cg_back0(xg_w, gn, {l: np_c(t) for l, t in y.items()}, False)
    oracle.vec_cg_back1(yg_w, gn, {l: np_c(t) for l, t in x.items()}, False)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    gv = G.backend.SO3vec.view([dev(t) for t in g.values()])
    # accumulate on top of ones: the kernel adds to what is there
    xg = [torch.ones(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
    yg = [torch.ones(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
    for _ in range(2):  # twice: the second call reuses the cached plan and the tensor memory
        G.backend.SO3vec.addCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
    torch.cuda.synchronize()
    for p, w in zip(xg, xg_w.values()):
        assert rel_err(p - 1, 2 * w) < tol
    for p, w in zip(yg, yg_w.values()):
        assert rel_err(p - 1, 2 * w) < tol


@pytest.mark.parametrize("overwrite", [True, False])
@pytest.mark.parametrize("B,lx,tau_y,maxl,bcast", [
    (5, 3, {0: 16, 1: 16, 2: 16, 3: 16}, 3, False),     # two cells per warp
    (3, 2, {1: 5, 2: 5}, 4, False),                      # channel count that is not a power of two, gaps in l
    (4, 4, {0: 32, 2: 32}, 6, False),                    # one cell per warp, truncated output
    (6, 2, {0: 8, 1: 8, 2: 8}, 2, True),                 # y broadcast over the batch
])
def test_forward_for_single_channel_x(G, oracle, B, lx, tau_y, maxl, bcast, overwrite):
    """The forward with a one-channel x (the narrow kernel) against the oracle, overwriting an output full of garbage
    and accumulating on top of ones."""
    tau_x = {l: 1 for l in range(lx + 1)}
    x, y = _vec_inputs(tau_x, tau_y, B, 800)
    if bcast:
        y = {l: t[:1].contiguous() for l, t in y.items()}
    tau_r = oracle.cg_type(tau_x, tau_y, maxl, False)
    want = {l: np.zeros((B, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, {l: np_c(t) for l, t in x.items()}, {l: np_c(t) for l, t in y.items()}, False)
    V = G.backend.SO3vec.view
    fill = 7.0 + 3.0j if overwrite else 1.0
    rs = [torch.full((B, 2 * l + 1, n), fill, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    assert V(rs).addCGproduct(V([dev(t) for t in x.values()]), V([dev(t) for t in y.values()]), overwrite=overwrite)
    torch.cuda.synchronize()
    for p, w in zip(rs, want.values()):
        assert rel_err(p if overwrite else p - 1, w) < TOL


@pytest.mark.parametrize("kernel", ["single-channel", "general"])
@pytest.mark.parametrize("B,lx,tau_y,maxl,bcast", [
    (5, 3, {0: 16, 1: 16, 2: 16, 3: 16}, 3, False),     # two cells per warp
    (3, 2, {1: 5, 2: 5}, 4, False),                      # channel count that is not a power of two, gaps in l
    (4, 4, {0: 32, 2: 32}, 6, False),                    # one cell per warp, truncated output
    (6, 2, {0: 8, 1: 8, 2: 8}, 2, True),                 # y broadcast over the batch: its gradient is a sum over cells
])
def test_gradient_of_y_for_single_channel_x(G, oracle, opt, B, lx, tau_y, maxl, bcast, kernel):
    """back1 alone with a one-channel x (the first layer after spherical harmonics): the kernel that walks the band
    once per (l1,l2) pair and the general narrow kernel must both give the oracle's gradient, on top of what yg holds."""
    opt("narrow1", "1" if kernel == "single-channel" else "0")
    tau_x = {l: 1 for l in range(lx + 1)}
    x, y = _vec_inputs(tau_x, tau_y, B, 700)
    if bcast:
        y = {l: t[:1].contiguous() for l, t in y.items()}
    tau_r = oracle.cg_type(tau_x, tau_y, maxl, False)
    g = {l: crandn(730 + l, B, 2 * l + 1, n) for l, n in tau_r.items()}
    yg_w = {l: np.zeros(t.shape, np.complex64) for l, t in y.items()}
    oracle.vec_cg_back1(yg_w, {l: np_c(t) for l, t in g.items()}, {l: np_c(t) for l, t in x.items()}, False)
    V = G.backend.SO3vec.view
    yg = [torch.ones(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
    for _ in range(2):
        assert V(yg).addCGproduct_back1(V([dev(t) for t in g.values()]), V([dev(t) for t in x.values()]))
    torch.cuda.synchronize()
    for p, w in zip(yg, yg_w.values()):
        assert rel_err(p - 1, 2 * w) < TOL_BIG


@pytest.mark.parametrize("copies", ["tensor", "cp.async"])
@pytest.mark.parametrize("layout", ["dense", "sliced"])
def test_pair_backward_on_grids(G, oracle, opt, copies, layout):
    """The pair backward kernel on a (batch, g0, g1) grid of cells.  A dense grid merges into one dimension of the
    kernel's tensor maps; a grid cut out of a larger one has three independent cell dimensions, which a rank-5 map
    cannot hold, so there the kernel fills its ring with cp.async even when tensor copies are allowed.  Both ways of
    copying must give the oracle's gradients on the flattened cells."""
    opt("bwd", "pair!")
    opt("pair_tma", "1" if copies == "tensor" else "0")
    B, G0, G1 = 2, 2, 3
    tau_x, tau_y = {0: 32, 1: 32}, {1: 32, 2: 64}
    tau_r = oracle.cg_type(tau_x, tau_y, 3, False)
    pad = 1 if layout == "sliced" else 0

    def grid(seed, l, n):
        t = crandn(seed, B * G0 * (G1 + pad), 2 * l + 1, n).reshape(B, G0, G1 + pad, 2 * l + 1, n)
        return dev(t)[:, :, :G1]

    x = {l: grid(500 + l, l, n) for l, n in tau_x.items()}
    y = {l: grid(520 + l, l, n) for l, n in tau_y.items()}
    g = {l: grid(540 + l, l, n) for l, n in tau_r.items()}
    flat = lambda t: np_c(t.reshape(B * G0 * G1, t.shape[-2], t.shape[-1]).cpu())
    xg_w = {l: np.zeros((B * G0 * G1, 2 * l + 1, n), np.complex64) for l, n in tau_x.items()}
    yg_w = {l: np.zeros((B * G0 * G1, 2 * l + 1, n), np.complex64) for l, n in tau_y.items()}
    gn = {l: flat(t) for l, t in g.items()}
    oracle.vec_cg_back0(xg_w, gn, {l: flat(t) for l, t in y.items()}, False)
    oracle.vec_cg_back1(yg_w, gn, {l: flat(t) for l, t in x.items()}, False)
    xg = [torch.zeros(B, G0, G1, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_x.items()]
    yg = [torch.zeros(B, G0, G1, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_y.items()]
    V = G.backend.SO3vec.view
    # the tensor-core forward on the same grid: its output tiles leave through tensor stores when the views allow
    # (here y has two channel counts, so only a uniform sub-vector takes them) -- values against the oracle either way
    opt("fwd", "tcgen05!")
    for ty in (tau_y, {1: 32}):
        tr = oracle.cg_type(tau_x, ty, 3, False)
        want = {l: np.zeros((B * G0 * G1, 2 * l + 1, n), np.complex64) for l, n in tr.items()}
        oracle.vec_cg(want, {l: flat(t) for l, t in x.items()}, {l: flat(y[l]) for l in ty}, False)
        rfull = {l: grid(560 + l, l, n) for l, n in tr.items()}  # garbage to overwrite, same layout as the inputs
        assert V(list(rfull.values())).addCGproduct(V(list(x.values())), V([y[l] for l in ty]), overwrite=True)
        torch.cuda.synchronize()
        for l, w in want.items():
            assert rel_err(flat(rfull[l]), w) < TOL_BIG
    assert G.backend.SO3vec.addCGproduct_back01(V(xg), V(yg), V(list(g.values())), V(list(x.values())), V(list(y.values())))
    torch.cuda.synchronize()
    for p, w in zip(xg, xg_w.values()):
        assert rel_err(p.reshape(w.shape), w) < TOL_BIG
    for p, w in zip(yg, yg_w.values()):
        assert rel_err(p.reshape(w.shape), w) < TOL_BIG


@pytest.mark.parametrize("B,tau_x,tau_y,maxl,tol", TC_CASES)
@pytest.mark.parametrize("kernel", ["tcgen05!", "tcgen05! bulk stores", "simt", "auto"])
def test_vec_forward_named_kernel(G, oracle, opt, B, tau_x, tau_y, maxl, tol, kernel):
    if kernel.endswith("bulk stores"):  # the tensor-core forward without tensor stores (per-row bulk copies)
        opt("pair_tma", "0")
        kernel = "tcgen05!"
    opt("fwd", kernel)  # "tcgen05!": fail instead of falling back to the SIMT kernel
    x, y = _vec_inputs(tau_x, tau_y, B, 60)
    tau_r = oracle.cg_type(tau_x, tau_y, maxl, False)
    want = {l: np.zeros((B, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, {l: np_c(t) for l, t in x.items()}, {l: np_c(t) for l, t in y.items()}, False)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    # the output starts as garbage: the kernel overwrites every element
    rparts = [torch.full((B, 2 * l + 1, n), 7.0 + 3.0j, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    rv = G.backend.SO3vec.view(rparts)
    for _ in range(2):  # twice: the second call reuses the cached plan and the tensor memory
        rv.addCGproduct(xv, yv, overwrite=True)
    torch.cuda.synchronize()
    for p, (l, w) in zip(rparts, want.items()):
        assert rel_err(p, w) < TOL, l


def test_tcgen05_wait_that_runs_out_is_reported(G, oracle, opt):
    """The kernel's mbarrier waits are bounded: when the completion never arrives (injected on the host: the MMAs
    are issued but not committed) the kernel gives up within a fraction of a second, frees its tensor memory and
    returns; the next product call of any kind reports it, and the one after that works again."""
    opt("fwd", "tcgen05!")
    tau = {l: 32 for l in range(3)}
    x, y = _vec_inputs(tau, tau, 2, 77)
    tau_r = oracle.cg_type(tau, tau, 2, False)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    rparts = [torch.zeros(2, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    rv = G.backend.SO3vec.view(rparts)
    opt("inject_timeout", "1")
    rv.addCGproduct(xv, yv, overwrite=True)   # launches; its waits run out on the device
    torch.cuda.synchronize()                  # the context stays usable
    opt("inject_timeout", "0")
    small = torch.zeros(2, 3, 4, dtype=torch.complex64, device="cuda")
    sx = dev(crandn(1, 2, 3, 2))
    with pytest.raises(Exception, match="gave up waiting"):
        view(G, small).add_DiagCGproduct(view(G, sx), view(G, sx))   # a call that takes another kernel reports it
    assert small.abs().max() == 0
    rv.addCGproduct(xv, yv, overwrite=True)   # the status was cleared: this one computes
    torch.cuda.synchronize()
    G._lib.async_status()
    want = {l: np.zeros((2, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, {l: np_c(t) for l, t in x.items()}, {l: np_c(t) for l, t in y.items()}, False)
    for p, (l, w) in zip(rparts, want.items()):
        assert rel_err(p, w) < TOL, l


def test_pair_backward_wait_that_runs_out_is_reported(G, oracle, opt):
    """Same for the default backward kernel: the producer warp leaves out one group's copies (a host-side switch), the
    consumers' bounded waits run out, the kernel returns, gelib_async_status() names the kernel, the next call works."""
    opt("bwd", "pair!")
    tau = {l: 32 for l in range(3)}
    x, y = _vec_inputs(tau, tau, 2, 78)
    tau_r = oracle.cg_type(tau, tau, 2, False)
    g = {l: crandn(500 + l, 2, 2 * l + 1, n) for l, n in tau_r.items()}
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    gv = G.backend.SO3vec.view([dev(t) for t in g.values()])

    def run():
        xg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
        yg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
        G.backend.SO3vec.addCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
        torch.cuda.synchronize()
        return xg, yg

    opt("inject_timeout", "1")
    run()
    opt("inject_timeout", "0")
    with pytest.raises(Exception, match="cg_bwd_pair_kernel"):
        G._lib.async_status()
    xg, yg = run()
    G._lib.async_status()
    gn = {l: np_c(t) for l, t in g.items()}
    xg_w = {l: np.zeros(t.shape, np.complex64) for l, t in x.items()}
    oracle.vec_cg_back0(xg_w, gn, {l: np_c(t) for l, t in y.items()}, False)
    for p, w in zip(xg, xg_w.values()):
        assert rel_err(p, w) < TOL_BIG


def test_tcgen05_refuses_what_it_cannot_do(G, opt):
    opt("bwd", "tcgen05!")
    tau = {0: 8, 1: 8}
    x, y = _vec_inputs(tau, tau, 2, 5)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    tau_r = xv.get_tau().CGproduct(yv.get_tau(), 1).get_parts()
    gv = G.backend.SO3vec.view([dev(crandn(7 + l, 2, 2 * l + 1, n)) for l, n in tau_r.items()])
    xg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
    yg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
    with pytest.raises(Exception):
        G.backend.SO3vec.addCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
    opt("bwd", "pair!")
    with pytest.raises(Exception):
        G.backend.SO3vec.addCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)



# ---- the benchmark configurations' own layouts ----------------------------------------------------------------

def test_diag_vector_maxl8_128_channels(G, oracle):
    """DiagCGproduct of SO3vecs with parts l = 0..8, 128 channels each, truncated at 8 (369 triples): the layout of the
    diagonal benchmark configuration, which takes the one-cell-per-CTA kernels with multi-chunk staging."""
    B, tau = 2, {l: 128 for l in range(9)}
    x, y = _vec_inputs(tau, tau, B, 20)
    tau_r = oracle.cg_type(tau, tau, 8, True)
    assert list(tau_r.values()) == [1152, 3072, 4608, 5760, 6528, 6912, 6912, 6528, 5760]
    xn, yn = {l: np_c(t) for l, t in x.items()}, {l: np_c(t) for l, t in y.items()}
    want = {l: np.zeros((B, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, xn, yn, True)
    xv = G.backend.SO3vec.view([dev(t) for t in x.values()])
    yv = G.backend.SO3vec.view([dev(t) for t in y.values()])
    rparts = [torch.full((B, 2 * l + 1, n), 7.0 + 3.0j, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    G.backend.SO3vec.view(rparts).addDiagCGproduct(xv, yv, overwrite=True)
    for p, (l, w) in zip(rparts, want.items()):
        assert rel_err(p, w) < TOL_BIG, l
    racc = [torch.ones_like(p) for p in rparts]
    G.backend.SO3vec.view(racc).addDiagCGproduct(xv, yv)
    for p, (l, w) in zip(racc, want.items()):
        assert rel_err(p - 1, w) < TOL_BIG, l
    g = {l: crandn(300 + l, B, 2 * l + 1, n) for l, n in tau_r.items()}
    gn = {l: np_c(t) for l, t in g.items()}
    xg_w = {l: np.zeros(t.shape, np.complex64) for l, t in x.items()}
    yg_w = {l: np.zeros(t.shape, np.complex64) for l, t in y.items()}
    oracle.vec_cg_back0(xg_w, gn, yn, True)
    oracle.vec_cg_back1(yg_w, gn, xn, True)
    gv = G.backend.SO3vec.view([dev(t) for t in g.values()])
    xg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in x.values()]
    yg = [torch.zeros(t.shape, dtype=torch.complex64, device="cuda") for t in y.values()]
    G.backend.SO3vec.addDiagCGproduct_back01(G.backend.SO3vec.view(xg), G.backend.SO3vec.view(yg), gv, xv, yv)
    xg2, yg2 = [torch.zeros_like(t) for t in xg], [torch.zeros_like(t) for t in yg]
    G.backend.SO3vec.view(xg2).addDiagCGproduct_back0(gv, yv)
    G.backend.SO3vec.view(yg2).addDiagCGproduct_back1(gv, xv)
    for a, a2, w in zip(xg, xg2, xg_w.values()):
        assert rel_err(a, w) < TOL_BIG and rel_err(a2, w) < TOL_BIG
    for a, a2, w in zip(yg, yg2, yg_w.values()):
        assert rel_err(a, w) < TOL_BIG and rel_err(a2, w) < TOL_BIG


def test_vec_arr_product_values(G, oracle):
    """SO3vecArr products on a [3] grid are independent products per (batch, grid) cell: values of the full and of
    the diagonal product and the gradients through autograd, against the oracle on the flattened cells."""
    torch.manual_seed(9)
    tau = {0: 2, 1: 3, 2: 2}
    B, Gd = 2, 3
    u, v = G.SO3vecArr.randn(B, [Gd], tau, device="cuda"), G.SO3vecArr.randn(B, [Gd], tau, device="cuda")
    un = {l: np_c(p.reshape(B * Gd, 2 * l + 1, -1)) for l, p in u.parts.items()}
    vn = {l: np_c(p.reshape(B * Gd, 2 * l + 1, -1)) for l, p in v.parts.items()}
    for diag in (False, True):
        if diag:
            tau_d = {l: 2 for l in range(3)}
            ud, vd = G.SO3vecArr.randn(B, [Gd], tau_d, device="cuda"), G.SO3vecArr.randn(B, [Gd], tau_d, device="cuda")
            a, b = ud, vd
            an = {l: np_c(p.reshape(B * Gd, 2 * l + 1, -1)) for l, p in a.parts.items()}
            bn = {l: np_c(p.reshape(B * Gd, 2 * l + 1, -1)) for l, p in b.parts.items()}
            tx = tau_d
        else:
            a, b, an, bn, tx = u, v, un, vn, tau
        a.requires_grad_()
        b.requires_grad_()
        w = (G.DiagCGproduct if diag else G.CGproduct)(a, b, maxl=2)
        tau_r = oracle.cg_type(tx, tx, 2, diag)
        want = {l: np.zeros((B * Gd, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
        oracle.vec_cg(want, an, bn, diag)
        for l, wl in want.items():
            assert list(w.parts[l].shape) == [B, Gd, 2 * l + 1, tau_r[l]]
            assert rel_err(w.parts[l].reshape(B * Gd, 2 * l + 1, -1), wl) < TOL
        gvec = type(w).randn_like(w)
        w.odot(gvec).backward()
        gn = {l: np_c(p.reshape(B * Gd, 2 * l + 1, -1)) for l, p in gvec.parts.items()}
        ag_w = {l: np.zeros(t.shape, np.complex64) for l, t in an.items()}
        bg_w = {l: np.zeros(t.shape, np.complex64) for l, t in bn.items()}
        oracle.vec_cg_back0(ag_w, gn, bn, diag)
        oracle.vec_cg_back1(bg_w, gn, an, diag)
        for l in tx:
            assert rel_err(a.parts[l].grad.reshape(B * Gd, 2 * l + 1, -1), ag_w[l]) < TOL
            assert rel_err(b.parts[l].grad.reshape(B * Gd, 2 * l + 1, -1), bg_w[l]) < TOL


def test_part_beyond_2_to_31_floats(G, oracle, opt):
    """64-bit addressing: part l = 4 of the headline output at batch 4096 holds 4096 x 9 x 33792 complex numbers =
    2.49e9 floats (the reference's GPUtensor carries int32 strides, cuda/GPUtensor.hpp:19-20).  One triple
    (6,6)->4 is written into and read back from the last 1024 channels; the LAST batch rows, whose float offsets
    lie beyond 2^31, are compared with the oracle."""
    B, n, l1, l2, l, ntot = 4096, 32, 6, 6, 4, 33792
    if torch.cuda.mem_get_info()[0] < 14e9:
        pytest.skip("needs 10 GB of device memory")
    offs = ntot - n * n
    x, y = crandn(61, B, 2 * l1 + 1, n), crandn(62, B, 2 * l2 + 1, n)
    xd, yd = dev(x), dev(y)
    big = torch.zeros(B, 2 * l + 1, ntot, dtype=torch.complex64, device="cuda")
    assert big.numel() * 2 > 2 ** 31
    want = np.zeros((2, 2 * l + 1, n * n), np.complex64)
    oracle.add_CGproduct(want, np_c(x[-2:]), np_c(y[-2:]))
    view(G, big).add_CGproduct(view(G, xd), view(G, yd), offs)
    assert rel_err(big[-2:, :, offs:], want) < TOL
    assert float(big[-2:, :, offs - 8:offs].abs().max()) == 0.0
    # the same block as an upstream gradient: both backward kernels read rows past 2^31 floats
    gl = crandn(63, 2, 2 * l + 1, n * n)
    big[-2:, :, offs:] = dev(gl)
    xg_w, yg_w = np.zeros((2, 2 * l1 + 1, n), np.complex64), np.zeros((2, 2 * l2 + 1, n), np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(gl), np_c(y[-2:]), offs=0)
    oracle.add_CGproduct_back1(yg_w, np_c(gl), np_c(x[-2:]), offs=0)
    for kernel in ("pair!", "simt"):
        opt("bwd", kernel)
        xg, yg = torch.zeros_like(xd), torch.zeros_like(yd)
        G.backend.SO3part.add_CGproduct_back01(view(G, xg), view(G, yg), view(G, big), view(G, xd), view(G, yd), offs)
        assert rel_err(xg[-2:], xg_w) < TOL_BIG and rel_err(yg[-2:], yg_w) < TOL_BIG, kernel
    del big
    torch.cuda.empty_cache()


def test_views_that_are_only_8_byte_aligned(G, oracle):
    """x, y taken as channel slices [1:33] of wider tensors (base 8 bytes off a 16-byte boundary, row pitch 66 floats)
    under the default kernel choice: the kernels with 16-byte accesses must not be chosen for them, and the result is
    the oracle's, forward and backward."""
    B, tau, maxl = 3, {l: 32 for l in range(3)}, 2
    xw = {l: crandn(30 + l, B, 2 * l + 1, 34) for l in tau}
    yw = {l: crandn(40 + l, B, 2 * l + 1, 33) for l in tau}
    xd = [t.cuda()[:, :, 1:33] for t in xw.values()]
    yd = [t.cuda()[:, :, 1:33] for t in yw.values()]
    assert xd[0].data_ptr() % 16 == 8
    xn = {l: np_c(t[:, :, 1:33]) for l, t in xw.items()}
    yn = {l: np_c(t[:, :, 1:33]) for l, t in yw.items()}
    tau_r = oracle.cg_type(tau, tau, maxl, False)
    want = {l: np.zeros((B, 2 * l + 1, n), np.complex64) for l, n in tau_r.items()}
    oracle.vec_cg(want, xn, yn, False)
    gb = G.backend
    xv, yv = gb.SO3vec.view(xd), gb.SO3vec.view(yd)
    rs = [torch.empty(B, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    gb.SO3vec.view(rs).addCGproduct(xv, yv, overwrite=True)
    for p, (l, w) in zip(rs, want.items()):
        assert rel_err(p, w) < TOL, l
    g = {l: crandn(50 + l, B, 2 * l + 1, n) for l, n in tau_r.items()}
    xg_w, yg_w = {l: np.zeros_like(t) for l, t in xn.items()}, {l: np.zeros_like(t) for l, t in yn.items()}
    oracle.vec_cg_back0(xg_w, {l: np_c(t) for l, t in g.items()}, yn, False)
    oracle.vec_cg_back1(yg_w, {l: np_c(t) for l, t in g.items()}, xn, False)
    xgw = [torch.zeros(B, 2 * l + 1, 34, dtype=torch.complex64, device="cuda") for l in tau]
    ygw = [torch.zeros(B, 2 * l + 1, 33, dtype=torch.complex64, device="cuda") for l in tau]
    gb.SO3vec.addCGproduct_back01(gb.SO3vec.view([t[:, :, 1:33] for t in xgw]), gb.SO3vec.view([t[:, :, 1:33] for t in ygw]),
                                  gb.SO3vec.view([t.cuda() for t in g.values()]), xv, yv)
    for t, w in zip(xgw, xg_w.values()):
        assert rel_err(t[:, :, 1:33], w) < TOL_BIG and float(t[:, :, 0].abs().max()) == 0.0 and float(t[:, :, 33].abs().max()) == 0.0
    for t, w in zip(ygw, yg_w.values()):
        assert rel_err(t[:, :, 1:33], w) < TOL_BIG and float(t[:, :, 0].abs().max()) == 0.0


def test_skipped_product_returns_zeros_like_the_reference(G, capfd):
    """A product the reference GELIB_SKIPs (l outside |l1-l2|..l1+l2) leaves its zero-initialised output untouched
    (python/src/gelib/SO3part.py:183-185); the autograd layer allocates uninitialised memory, so it must zero it."""
    torch.manual_seed(2)
    x, y = G.SO3part.randn(3, 1, 4, device="cuda"), G.SO3part.randn(3, 1, 4, device="cuda")
    for _ in range(3):   # whatever the allocator hands back
        junk = torch.full((3, 7, 16), 5.0 + 1.0j, dtype=torch.complex64, device="cuda")
        del junk
        z = G.CGproduct(x, y, 3)
        assert list(z.shape) == [3, 7, 16] and float(z.abs().max()) == 0.0
    assert "skipped" in capfd.readouterr().err
    # an output broadcast over cells cannot be overwritten: refused, not silently accumulated into garbage
    r = torch.zeros(1, 5, 16, dtype=torch.complex64, device="cuda")
    with pytest.raises(RuntimeError, match="GELIB_OVERWRITE"):
        view(G, r).add_CGproduct(view(G, x), view(G, y), overwrite=True)
    # x with a size-1 array dimension against y with 3: the output takes the larger
    xa, ya = G.SO3partArr.randn(2, [1], 1, 2, device="cuda"), G.SO3partArr.randn(2, [3], 1, 2, device="cuda")
    assert list(G.CGproduct(xa, ya, 1).shape) == [2, 3, 3, 4]


# ---- spherical harmonics --------------------------------------------------------------------------------

@pytest.mark.parametrize("L", [0, 1, 2, 4, 6, 8, 11, 14])
@pytest.mark.parametrize("n", [1, 5])
def test_spharm_matches_oracle(G, oracle, L, n):
    X = frandn(40 + L, 33, 3, n) * (0.5 + 1.5 * torch.rand(33, 1, n, generator=torch.Generator().manual_seed(1)))
    X[0, :, 0] = torch.tensor([0.0, 0.0, 2.0])    # z axis: the degenerate branch
    X[1, :, 0] = torch.tensor([0.0, 0.0, -1.0])
    want = np.zeros((33, 2 * L + 1, n), np.complex64)
    oracle.add_spharm(want, np_c(X))
    got = G.SO3part.spharm(L, dev(X))
    assert rel_err(got, want) < 2e-6
    acc = torch.ones(33, 2 * L + 1, n, dtype=torch.complex64, device="cuda")
    view(G, acc).add_spharm(dev(X))
    assert rel_err(acc - 1, want) < 2e-6


def test_spharm_all_parts_in_one_pass(G, oracle):
    X = frandn(7, 100, 3, 1)
    v = G.SO3vec.spharms(6, dev(X))
    for L in range(7):
        want = np.zeros((100, 2 * L + 1, 1), np.complex64)
        oracle.add_spharm(want, np_c(X))
        assert rel_err(v.parts[L], want) < 2e-6


def test_spharm_matches_scipy_fixture(G):
    import os
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "spharm_scipy.npz"))
    X = torch.from_numpy(np.ascontiguousarray(z["points"].T[None]))
    for L in range(9):
        got = G.SO3part.spharm(L, dev(X))
        assert np.abs(got.cpu().numpy() - z["L%d" % L].T[None]).max() < 5e-6


# ---- the Python API: the reference's own property tests on device ---------------------------------------

@pytest.mark.parametrize("b", [1, 2])
@pytest.mark.parametrize("l", [1, 2, 4])
@pytest.mark.parametrize("n", [1, 2, 4, 8])
@pytest.mark.parametrize("diag", [False, True])
def test_api_equivariance(G, b, l, n, diag):
    # python/tests/ci_tests/test_SO3part.py:55-86
    torch.manual_seed(b * 100 + l * 10 + n)
    x, y = G.SO3part.randn(b, l, n, device="cuda"), G.SO3part.randn(b, l, n, device="cuda")
    fn = G.DiagCGproduct if diag else G.CGproduct
    R = G.SO3element.random()
    z, zr = fn(x, y, l), fn(x.apply(R), y.apply(R), l)
    assert torch.allclose(z.apply(R), zr, rtol=1e-3, atol=1e-4)


def _backprop_check(G, x, y, fn, arg):
    x.requires_grad_()
    y.requires_grad_()
    z = fn(x, y, arg)
    test_vec = type(z).randn_like(z)
    loss = z.odot(test_vec)
    loss.backward(torch.tensor(1.0, device="cuda"))
    xeps, yeps = type(x).randn_like(x), type(y).randn_like(y)
    xloss = fn(x + xeps, y, arg).odot(test_vec)
    assert torch.allclose(xloss - loss, xeps.odot(x.grad), rtol=1e-3, atol=1e-3)
    yloss = fn(x, y + yeps, arg).odot(test_vec)
    assert torch.allclose(yloss - loss, yeps.odot(y.grad), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("b", [1, 2])
@pytest.mark.parametrize("l", [1, 2, 4])
@pytest.mark.parametrize("n", [1, 4, 8])
@pytest.mark.parametrize("diag", [False, True])
def test_api_backprop(G, b, l, n, diag):
    # python/tests/ci_tests/test_SO3part.py:7-28,89-100
    torch.manual_seed(7 + b + l + n)
    x, y = G.SO3part.randn(b, l, n, device="cuda"), G.SO3part.randn(b, l, n, device="cuda")
    _backprop_check(G, x, y, G.DiagCGproduct if diag else G.CGproduct, l)


@pytest.mark.parametrize("b", [1, 2])
@pytest.mark.parametrize("l", [2, 4])
def test_api_backprop_bcast(G, b, l):
    # python/tests/ci_tests/test_SO3part.py:31-52,103-107: x has batch 1
    torch.manual_seed(11)
    x, y = G.SO3part.randn(1, l, 4, device="cuda"), G.SO3part.randn(b, l, 4, device="cuda")
    _backprop_check(G, x, y, G.CGproduct, l)


@pytest.mark.parametrize("maxl", [2, 4])
@pytest.mark.parametrize("b", [1, 3])
@pytest.mark.parametrize("nc", [1, 4])
@pytest.mark.parametrize("diag", [False, True])
def test_api_vec_equivariance_and_backprop(G, maxl, b, nc, diag):
    # python/tests/ci_tests/test_SO3vec.py:57-105
    torch.manual_seed(maxl + b + nc)
    tau = {l: nc for l in range(maxl + 1)}
    x, y = G.SO3vec.randn(b, tau, device="cuda"), G.SO3vec.randn(b, tau, device="cuda")
    fn = (lambda a, c: G.DiagCGproduct(a, c, maxl=maxl)) if diag else (lambda a, c: G.CGproduct(a, c, maxl=maxl))
    R = G.SO3element.random()
    z, zr = fn(x, y), fn(x.apply(R), y.apply(R))
    rz = z.apply(R)
    for l in range(maxl + 1):
        assert torch.allclose(rz.parts[l], zr.parts[l], rtol=1e-3, atol=1e-4)
    x.requires_grad_()
    y.requires_grad_()
    z = fn(x, y)
    test_vec = G.SO3vec.randn_like(z)
    loss = z.odot(test_vec)
    loss.backward(torch.tensor(1.0, device="cuda"))
    xeps = G.SO3vec.randn_like(x)
    xloss = fn(x + xeps, y).odot(test_vec)
    assert torch.allclose(xloss - loss, xeps.odot(x.get_grad()), rtol=1e-3, atol=1e-2)
    yeps = G.SO3vec.randn_like(y)
    yloss = fn(x, y + yeps).odot(test_vec)
    assert torch.allclose(yloss - loss, yeps.odot(y.get_grad()), rtol=1e-3, atol=1e-2)


def test_api_arr_products(G, oracle):
    # SO3partArr / SO3vecArr: cells of a [2,2] grid are independent products
    torch.manual_seed(3)
    x, y = G.SO3partArr.randn(2, [2, 2], 1, 3, device="cuda"), G.SO3partArr.randn(2, [2, 2], 2, 3, device="cuda")
    z = G.CGproduct(x, y, 2)
    assert isinstance(z, G.SO3partArr) and list(z.shape) == [2, 2, 2, 5, 9]
    want = np.zeros((8, 5, 9), np.complex64)
    oracle.add_CGproduct(want, np_c(x.reshape(-1, 3, 3)), np_c(y.reshape(-1, 5, 3)))
    assert rel_err(z.reshape(-1, 5, 9), want) < TOL
    tau = {0: 2, 1: 2}
    u, v = G.SO3vecArr.randn(2, [3], tau, device="cuda"), G.SO3vecArr.randn(2, [3], tau, device="cuda")
    w = G.CGproduct(u, v, maxl=1)
    assert list(w.parts[1].shape) == [2, 3, 3, 12]
    d = G.DiagCGproduct(u, v, maxl=1)
    assert list(d.parts[0].shape) == [2, 3, 1, 4]


def test_diag_is_diagonal_of_full_on_device(G):
    torch.manual_seed(5)
    x, y = G.SO3part.randn(3, 1, 4, device="cuda"), G.SO3part.randn(3, 2, 4, device="cuda")
    full, diag = G.CGproduct(x, y, 1), G.DiagCGproduct(x, y, 1)
    assert torch.allclose(diag, full[:, :, [n * 4 + n for n in range(4)]], atol=1e-6)


def test_weights_mix_channels(G):
    tau = G.SO3type({0: 3, 1: 3})
    v = G.SO3vec.randn(2, tau, device="cuda")
    W = G.SO3weights.randn(tau, G.SO3type({0: 5, 1: 2}), device="cuda")
    out = v * W
    assert list(out.parts[0].shape) == [2, 1, 5] and list(out.parts[1].shape) == [2, 3, 2]


# ---- size-independent properties at the benchmark's full channel counts -----------------------------------

def test_large_forward_linearity_and_backward_adjointness(G):
    """At the headline shape (maxl 6, 32 channels) on a slice of the batch: the product is bilinear, and the
    gradients are the adjoints of the forward maps: <g, CG(x,y)> = <xg, x> = <yg, y> (real inner product)."""
    B, tau = 24, {l: 32 for l in range(7)}
    x, y = _vec_inputs(tau, tau, B, 900)
    x2, _ = _vec_inputs(tau, tau, B, 950)
    xs, ys, x2s = [dev(t) for t in x.values()], [dev(t) for t in y.values()], [dev(t) for t in x2.values()]
    gb = G.backend
    tau_r = gb.SO3vec.view(xs).get_tau().CGproduct(gb.SO3vec.view(ys).get_tau(), 6).get_parts()
    assert list(tau_r.values()) == [7168, 18432, 26624, 31744, 33792, 32768, 28672]

    def prod(a):
        r = [torch.empty(B, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
        gb.SO3vec.view(r).addCGproduct(gb.SO3vec.view(a), gb.SO3vec.view(ys), overwrite=True)
        return r

    r1, r2, r12 = prod(xs), prod(x2s), prod([a + 2 * b for a, b in zip(xs, x2s)])
    for a, b, c in zip(r1, r2, r12):
        assert rel_err(c, a + 2 * b) < TOL_BIG
    g = [torch.randn_like(t) for t in r1]
    xg, yg = [torch.zeros_like(t) for t in xs], [torch.zeros_like(t) for t in ys]
    gb.SO3vec.addCGproduct_back01(gb.SO3vec.view(xg), gb.SO3vec.view(yg), gb.SO3vec.view(g), gb.SO3vec.view(xs), gb.SO3vec.view(ys))
    dot = lambda a, b: sum(float((torch.view_as_real(u).double() * torch.view_as_real(v).double()).sum()) for u, v in zip(a, b))
    lhs = dot(g, r1)
    assert abs(dot(xg, xs) - lhs) < 1e-4 * abs(lhs) + 1.0
    assert abs(dot(yg, ys) - lhs) < 1e-4 * abs(lhs) + 1.0
