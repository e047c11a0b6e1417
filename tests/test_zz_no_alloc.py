"""The allocation-free forward entry point, gelib_SO3vec_addCGproduct_static.

Collected last on purpose (the file name sorts after the others), so that a run that stops at the first failure has
already run everything else.  The entry point serves callers that cannot call cudaMalloc (a plug-in confined to its
host framework's memory pool, a process whose device memory is fully handed out, a loop that cannot afford
cudaMalloc's implicit synchronisation): its tables live in a fixed device array instead of plan memory.  It is checked
through the C ABI against the ordinary entry point on the same inputs, on two calls in a row with different product
signatures, because every call reuses the one array and finds the previous call's tables in it.
"""
import pytest
import torch

from util import crandn, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _product(G, tau_x, tau_y, maxl, B, seed, static):
    gb = G.backend
    xs = [crandn(seed + l, B, 2 * l + 1, n).cuda() for l, n in tau_x.items()]
    ys = [crandn(seed + 50 + l, B, 2 * l + 1, n).cuda() for l, n in tau_y.items()]
    xv, yv = gb.SO3vec.view(xs), gb.SO3vec.view(ys)
    tau_r = xv.get_tau().CGproduct(yv.get_tau(), maxl).get_parts()
    # start from ones: both entry points add to what is there
    rs = [torch.ones(B, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    rv = gb.SO3vec.view(rs)
    assert (rv.addCGproduct_static if static else rv.addCGproduct)(xv, yv)
    torch.cuda.synchronize()
    return rs


def test_static_entry_point_matches_the_ordinary_one_twice_in_a_row():
    import gelib_b200 as G
    assert torch.cuda.is_available()
    G._lib.lib()
    cases = [({0: 3, 1: 2, 2: 4}, {0: 2, 1: 5, 3: 1}, 3, 5, 11),      # first call: also looks up the array's address
             ({l: 8 for l in range(5)}, {l: 8 for l in range(5)}, 4, 3, 23)]  # second: other tables over the first's
    for tau_x, tau_y, maxl, B, seed in cases:
        n0 = G.backend.kernel_launch_count()
        got = _product(G, tau_x, tau_y, maxl, B, seed, static=True)
        assert G.backend.kernel_launch_count() == n0 + 1
        want = _product(G, tau_x, tau_y, maxl, B, seed, static=False)
        for a, b in zip(got, want):
            assert rel_err(a, b) < TOL


def test_static_entry_point_rejects_tables_beyond_its_array():
    import gelib_b200 as G
    gb = G.backend
    tau = {l: 1 for l in range(8)}    # 344 triples and 26216 coefficients: 112 KB of tables, 15 output parts
    xs = [torch.zeros(1, 2 * l + 1, 1, dtype=torch.complex64, device="cuda") for l in tau]
    xv = gb.SO3vec.view(xs)
    tau_r = xv.get_tau().CGproduct(xv.get_tau(), -1).get_parts()
    rs = [torch.zeros(1, 2 * l + 1, n, dtype=torch.complex64, device="cuda") for l, n in tau_r.items()]
    with pytest.raises(RuntimeError, match="static array holds 65536"):
        gb.SO3vec.view(rs).addCGproduct_static(xv, xv)
