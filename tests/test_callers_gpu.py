"""Callers of the Clebsch-Gordan path on device: gather over an array dimension, the Wigner-D apply, O(3) parts and
vectors (parity bookkeeping over the SO(3) kernels)."""
import numpy as np
import pytest
import torch

from util import crandn, np_c, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gelib_b200
    assert torch.cuda.is_available()
    gelib_b200._lib.lib()
    return gelib_b200


def test_gather_sums_sources_into_targets_and_backpropagates(G):
    # core/Gpart.hpp:537-561: r = x.gather(map, d); the gradient runs through the transposed map
    torch.manual_seed(1)
    B, A0, A1, l, n = 2, 5, 3, 2, 4
    x = G.SO3partArr.randn(B, [A0, A1], l, n, device="cuda")
    sources, targets = [0, 1, 1, 4, 2, 2, 3], [3, 0, 3, 3, 1, 5, 5]
    gm = G.gather_map.sources_targets(sources, targets, n_in=A0, n_out=7)
    x.requires_grad_()
    r = G.gather(x, gm, 0)
    assert isinstance(r, G.SO3partArr) and list(r.shape) == [B, 7, A1, 5, n]
    want = torch.zeros_like(r.detach().as_subclass(torch.Tensor))
    want.index_add_(1, torch.tensor(targets, device="cuda"), x.detach().as_subclass(torch.Tensor)[:, sources])
    assert rel_err(r, want) < 1e-6
    rd = r.detach()
    assert float(rd[:, 2].abs().max()) == 0.0 and float(rd[:, 4].abs().max()) == 0.0 and float(rd[:, 6].abs().max()) == 0.0
    g = torch.randn_like(want)
    r.backward(g)
    gw = torch.zeros_like(x.detach().as_subclass(torch.Tensor))
    gw.index_add_(1, torch.tensor(sources, device="cuda"), g[:, targets])
    assert rel_err(x.grad, gw) < 1e-6
    # along the second array dimension, and a map given as a matrix
    M = (torch.rand(4, A1, generator=torch.Generator().manual_seed(2)) < 0.6)
    gm2 = G.gather_map.from_matrix(M, A1, 4)
    r2 = x.detach().gather(gm2, 1)
    want2 = torch.einsum("ts,bastn->batn".replace("stn", "sxn").replace("batn", "batxn").replace("bastn", "basxn"),
                         M.to(torch.complex64).cuda(), x.detach().as_subclass(torch.Tensor))
    assert rel_err(r2, want2) < 1e-6
    v = G.SO3vecArr.randn(B, [A0], {0: 2, 1: 3}, device="cuda")
    w = v.gather(gm, 0)
    assert list(w.parts[1].shape) == [B, 7, 3, 3]


@pytest.mark.parametrize("l", [0, 1, 3, 6])
def test_wigner_matrix_and_device_apply(G, l):
    # D from the C ABI equals the Python restatement of SO3/SO3irrep.hpp:69-103; apply = D x cell by cell; D is unitary
    R = G.SO3element.random(torch.Generator().manual_seed(l))
    from gelib_b200.SO3irrep import euler_zyz
    a, b, c = euler_zyz(R.numpy())
    D1 = G.backend.SO3irrep_matrix(l, a, b, c)
    D2 = G.SO3irrep(l).matrix(R)
    assert rel_err(D1, D2) < 1e-6
    assert rel_err(D1 @ D1.conj().t(), torch.eye(2 * l + 1, dtype=torch.complex64)) < 1e-5
    x = G.SO3part.randn(3, l, 5, device="cuda")
    x.requires_grad_()
    y = x.apply(R)
    assert rel_err(y, torch.matmul(D2.cuda(), x.detach().as_subclass(torch.Tensor))) < 1e-6
    g = torch.randn_like(y.detach().as_subclass(torch.Tensor))
    y.backward(g)
    assert rel_err(x.grad, torch.matmul(D2.cuda().conj().t(), g)) < 1e-6
    arr = G.SO3partArr.randn(2, [3], l, 4, device="cuda")
    assert rel_err(arr.apply(R), torch.matmul(D2.cuda(), arr.as_subclass(torch.Tensor))) < 1e-6


def test_o3_vector_product_matches_the_reference_loop(G, oracle):
    """O3vec.CGproduct against a direct restatement of the reference's loop (core/Gvec.hpp:311-321 with O(3) indices):
    parts in index order 2l + [p = -1], (l1,p1) x (l2,p2) feeds (l, p1 p2), offsets advance by n1 n2 per triple."""
    torch.manual_seed(4)
    B, maxl = 3, 3
    tx = {(0, 1): 2, (1, -1): 3, (1, 1): 1, (2, 1): 2}
    ty = {(0, -1): 2, (1, 1): 2, (2, -1): 1, (2, 1): 3}
    x, y = G.O3vec.randn(B, tx, device="cuda"), G.O3vec.randn(B, ty, device="cuda")
    assert list(x.parts) == [(0, 1), (1, 1), (1, -1), (2, 1)]
    x.requires_grad_()
    y.requires_grad_()
    z = x.CGproduct(y, maxl)
    rtype = G.O3type(tx).CGproduct(G.O3type(ty), maxl).get_parts()
    assert z.tau() == rtype
    want = {mu: np.zeros((B, 2 * mu[0] + 1, n), np.complex64) for mu, n in rtype.items()}
    offs = {mu: 0 for mu in rtype}
    for (l1, p1), xp in x.parts.items():
        for (l2, p2), yp in y.parts.items():
            for l in range(abs(l1 - l2), min(l1 + l2, maxl) + 1):
                mu = (l, p1 * p2)
                oracle.add_CGproduct(want[mu], np_c(xp.as_subclass(torch.Tensor)), np_c(yp.as_subclass(torch.Tensor)), offs=offs[mu])
                offs[mu] += xp.size(-1) * yp.size(-1)
    for mu, w in want.items():
        assert rel_err(z.parts[mu], w) < 1e-5, mu
    # gradients: first-order check as in python/tests/ci_tests/test_SO3vec.py:83-105
    tv = G.O3vec.randn_like(z)
    loss = z.odot(tv)
    loss.backward()
    xeps = G.O3vec.randn_like(x)
    xloss = (x + xeps).CGproduct(y, maxl).odot(tv)
    assert torch.allclose(xloss - loss, xeps.odot(x.get_grad()), rtol=1e-3, atol=1e-2)
    yeps = G.O3vec.randn_like(y)
    yloss = x.CGproduct(y + yeps, maxl).odot(tv)
    assert torch.allclose(yloss - loss, yeps.odot(y.get_grad()), rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("diag", [False, True])
def test_o3_products_are_equivariant_under_improper_rotations(G, diag):
    torch.manual_seed(6)
    gen = torch.Generator().manual_seed(8)
    R = G.O3element(-G.SO3element.random(gen).as_subclass(torch.Tensor))   # determinant -1
    assert R.parity() == -1
    tau = {(0, 1): 2, (1, -1): 2, (1, 1): 2, (2, -1): 2}
    x, y = G.O3vec.randn(2, tau, device="cuda"), G.O3vec.randn(2, tau, device="cuda")
    f = (lambda a, c: a.DiagCGproduct(c, 2)) if diag else (lambda a, c: a.CGproduct(c, 2))
    z, zr = f(x, y).apply(R), f(x.apply(R), y.apply(R))
    for mu in z.parts:
        assert torch.allclose(z.parts[mu].as_subclass(torch.Tensor), zr.parts[mu].as_subclass(torch.Tensor), rtol=1e-3, atol=1e-4), mu
    # parts: the parity rule is enforced, spherical harmonics carry (-1)^l
    a, c = G.O3part.randn(2, (1, -1), 3, device="cuda"), G.O3part.randn(2, (2, -1), 3, device="cuda")
    w = a.CGproduct(c, (2, 1))
    assert w.mu == (2, 1) and list(w.shape) == [2, 5, 9]
    with pytest.raises(AssertionError):
        a.CGproduct(c, (2, -1))
    X = torch.randn(4, 3, 2, device="cuda")
    s = G.O3part.spharm(3, X)
    assert s.mu == (3, -1) and rel_err(G.O3part.spharm(3, -X), -s) < 1e-5


def test_fused_spharm_cg_first_layer(G, oracle):
    """CGproduct(spharms(6, X), y) with the harmonics generated inside the kernel equals the two-step pipeline and the
    oracle (harmonics by the oracle, then the vector product), forward and the gradient with respect to y."""
    from util import frandn
    B, lx, maxl, n = 37, 6, 6, 16
    X = frandn(5, B, 3, 1) * (0.5 + 1.5 * torch.rand(B, 1, 1, generator=torch.Generator().manual_seed(3)))
    X[0, :, 0] = torch.tensor([0.0, 0.0, 1.5])   # z axis: the degenerate branch
    y = {l: crandn(70 + l, B, 2 * l + 1, n) for l in range(lx + 1)}
    Xd = X.cuda()
    yv = G.SO3vec(*[G.SO3part(t.cuda()) for t in y.values()])
    yv.requires_grad_()
    z = G.SO3vec.spharm_CGproduct(lx, Xd, yv, maxl)
    z2 = G.CGproduct(G.SO3vec.spharms(lx, Xd), yv, maxl=maxl)
    un = {}
    for l in range(lx + 1):
        un[l] = np.zeros((B, 2 * l + 1, 1), np.complex64)
        oracle.add_spharm(un[l], np_c(X))
    tau_r = oracle.cg_type({l: 1 for l in range(lx + 1)}, {l: n for l in range(lx + 1)}, maxl, False)
    want = {l: np.zeros((B, 2 * l + 1, k), np.complex64) for l, k in tau_r.items()}
    oracle.vec_cg(want, un, {l: np_c(t) for l, t in y.items()}, False)
    for l, w in want.items():
        assert rel_err(z.parts[l], w) < 1e-5 and rel_err(z.parts[l], z2.parts[l].detach()) < 1e-5, l
    g = {l: crandn(170 + l, B, 2 * l + 1, k) for l, k in tau_r.items()}
    torch.autograd.backward(list(z.parts.values()), grad_tensors=[t.cuda() for t in g.values()])
    yg_w = {l: np.zeros(t.shape, np.complex64) for l, t in y.items()}
    oracle.vec_cg_back1(yg_w, {l: np_c(t) for l, t in g.items()}, un, False)
    for l, w in yg_w.items():
        assert rel_err(yv.parts[l].grad, w) < 1e-4, l
    # a y the narrow kernels do not take is refused, not silently routed elsewhere
    wide = G.SO3vec(G.SO3part(crandn(1, B, 3, 64).cuda()))
    with pytest.raises(RuntimeError, match="fused spherical-harmonics"):
        G.SO3vec.spharm_CGproduct(2, Xd, wide, 2)


def test_fp64_option_keeps_double_coefficients_and_sums(G):
    """GELIB_FP64: against a complex128 evaluation with double coefficients the result is exact to float rounding of the
    output, for the forward product and both gradients at l = 8 with 48 channels (sums of up to 17 x 48 terms)."""
    import ctypes
    B, l1, l2, l, n = 2, 8, 8, 8, 48
    x, y, g = crandn(1, B, 2 * l1 + 1, n), crandn(2, B, 2 * l2 + 1, n), crandn(3, B, 2 * l + 1, n * n)
    L = G._lib.lib()
    C = np.zeros((2 * l1 + 1, 2 * l2 + 1))
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            if abs(m1 + m2) <= l:
                C[m1 + l1, m2 + l2] = L.gelib_CGcoefficient(l1, l2, l, m1, m2)
    C3 = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l + 1))
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            if abs(m1 + m2) <= l:
                C3[m1 + l1, m2 + l2, m1 + m2 + l] = C[m1 + l1, m2 + l2]
    xn, yn, gn = np_c(x).astype(np.complex128), np_c(y).astype(np.complex128), np_c(g).astype(np.complex128)
    want = np.einsum("abm,zai,zbj->zmij", C3, xn, yn).reshape(B, 2 * l + 1, n * n)
    g4 = gn.reshape(B, 2 * l + 1, n, n)
    xg_w = np.einsum("abm,zmij,zbj->zai", C3, g4, yn.conj())
    yg_w = np.einsum("abm,zmij,zai->zbj", C3, g4, xn.conj())
    view = G.backend.SO3part.view
    xd, yd, gd = x.cuda(), y.cuda(), g.cuda()

    def run(fp64):
        r = torch.zeros(B, 2 * l + 1, n * n, dtype=torch.complex64, device="cuda")
        view(r).add_CGproduct(view(xd), view(yd), fp64=fp64)
        xg, yg = torch.zeros_like(xd), torch.zeros_like(yd)
        view(xg).add_CGproduct_back0(view(gd), view(yd), fp64=fp64)
        view(yg).add_CGproduct_back1(view(gd), view(xd), fp64=fp64)
        return [float(np.abs(a.cpu().numpy() - w).max() / np.abs(w).max()) for a, w in ((r, want), (xg, xg_w), (yg, yg_w))]

    e64, e32 = run(True), run(False)
    assert max(e64) < 1.5e-7, e64            # float rounding of the stored result only
    assert max(e32) < 1e-5 and e64[1] < e32[1] and e64[2] < e32[2], (e64, e32)


@pytest.mark.gpu
@pytest.mark.parametrize("rows_shape,n_in,n_out", [((1000, 5), 16, 16), ((7, 3), 5, 9), ((300, 2, 13), 32, 64), ((1,), 1, 1)])
def test_weight_mixing_kernels_match_matmul(G, rows_shape, n_in, n_out):
    """part * W and both of its gradients through the mixing kernels against torch.matmul and its autograd."""
    torch.manual_seed(11)
    x = torch.randn(*rows_shape, n_in, dtype=torch.complex64, device="cuda")
    w = torch.randn(n_in, n_out, dtype=torch.complex64, device="cuda") / n_in ** 0.5
    g = torch.randn(*rows_shape, n_out, dtype=torch.complex64, device="cuda")
    want = torch.matmul(x, w)
    got = G.backend.mix(x, w)
    assert (got - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))
    gx_w = torch.matmul(g, w.conj().T)
    gx = G.backend.mix(g, w, adjoint=True)
    assert (gx - gx_w).abs().max() < 1e-5 * max(1.0, float(gx_w.abs().max()))
    gw_w = torch.matmul(x.reshape(-1, n_in).conj().T, g.reshape(-1, n_out))
    gw = G.backend.mix_back_w(x, g, n_in, n_out)
    assert (gw - gw_w).abs().max() < 2e-5 * max(1.0, float(gw_w.abs().max()))


@pytest.mark.gpu
def test_vec_times_weights_autograd(G):
    """SO3vec * SO3weights on the device: values and gradients equal those of torch.matmul per part."""
    torch.manual_seed(12)
    tau = {0: 16, 1: 16, 2: 16}
    v = G.SO3vec.randn(9, tau, device="cuda")
    ws = [torch.randn(16, 8, dtype=torch.complex64, device="cuda").requires_grad_() for _ in tau]
    ps = [p.detach().clone().requires_grad_() for p in v.parts.values()]
    out = G.SO3vec(*[G.SO3part(p) for p in ps]) * G.SO3weights(*ws)
    gs = [torch.randn_like(p) for p in out.parts.values()]
    torch.autograd.backward(list(out.parts.values()), grad_tensors=gs)
    for p, w_, g_, o in zip(ps, ws, gs, out.parts.values()):
        p2, w2 = p.detach().clone().requires_grad_(), w_.detach().clone().requires_grad_()
        ref = torch.matmul(p2.as_subclass(torch.Tensor), w2)
        ref.backward(g_.as_subclass(torch.Tensor))
        assert (o.as_subclass(torch.Tensor) - ref).abs().max() < 1e-5
        assert (p.grad - p2.grad).abs().max() < 1e-5
        assert (w_.grad - w2.grad).abs().max() < 1e-4
