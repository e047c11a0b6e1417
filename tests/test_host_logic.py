"""CPU-side checks of the shipped library: symbol table of the C ABI, host helpers (coefficients, type
calculus, triple schedule), descriptor canonicalisation and argument validation.  No kernel is launched."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(cabi):
    from gelib_b200 import _lib
    header = open(os.path.join(ROOT, "include", "gelib_b200.h")).read()
    declared = set(re.findall(r"\b(gelib_[A-Za-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(cabi, name), name
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    assert b"sm_100a" in cabi.gelib_version()


def test_coefficients_match_oracle(cabi, oracle):
    for (l1, l2, l) in [(1, 2, 2), (2, 2, 2), (3, 4, 5), (6, 6, 6), (8, 8, 8), (6, 6, 0), (0, 5, 5), (12, 12, 10)]:
        C = np.zeros((2 * l1 + 1, 2 * l2 + 1), np.float32)
        assert cabi.gelib_CGmatrix(l1, l2, l, C.ctypes.data) == 0
        assert np.abs(C - oracle.cg_matrix(l1, l2, l)).max() <= 1.2e-7
        for m1 in (-l1, 0, l1):
            for m2 in (-l2, 0, l2):
                if abs(m1 + m2) <= l:
                    assert abs(cabi.gelib_CGcoefficient(l1, l2, l, m1, m2) - oracle.cg_coeff(l1, l2, l, m1, m2)) < 1e-12
    assert cabi.gelib_CGmatrix(1, 1, 3, C.ctypes.data) == 1  # triangle violated -> skipped


def test_type_product_and_schedule_match_oracle(oracle):
    from gelib_b200 import backend as gb
    from gelib_b200._lib import lib
    for tau_x, tau_y, maxl in [({0: 2, 1: 3, 2: 1}, {0: 1, 1: 2}, -1), ({l: 4 for l in range(5)}, {l: 4 for l in range(5)}, 4),
                               ({1: 2, 3: 1}, {2: 5}, 3)]:
        for diag in (False, True):
            if diag and set(tau_x.values()) | set(tau_y.values()) != {next(iter(tau_x.values()))}:
                continue
            tx, ty = gb.SO3type(tau_x), gb.SO3type(tau_y)
            got = (tx.DiagCGproduct(ty, maxl) if diag else tx.CGproduct(ty, maxl)).get_parts()
            want = oracle.cg_type(tau_x, tau_y, maxl, diag)
            assert got == want
            rl = sorted(want)
            cap = 4096
            out = (ctypes.c_int * (4 * cap))()
            arr = lambda v: (ctypes.c_int * len(v))(*v)
            k = lib().gelib_SO3vec_CGproduct_schedule(len(tau_x), arr(list(tau_x)), arr(list(tau_x.values())), len(tau_y),
                                                      arr(list(tau_y)), arr(list(tau_y.values())), len(rl), arr(rl),
                                                      1 if diag else 0, cap, out)
            got_tr = [tuple(out[4 * i:4 * i + 4]) for i in range(k)]
            assert got_tr == oracle.triples(tau_x, tau_y, set(rl), diag)


def test_maxl6_schedule_has_175_triples():
    from gelib_b200._lib import lib
    ls = list(range(7))
    ns = [32] * 7
    arr = lambda v: (ctypes.c_int * len(v))(*v)
    out = (ctypes.c_int * (4 * 400))()
    assert lib().gelib_SO3vec_CGproduct_schedule(7, arr(ls), arr(ns), 7, arr(ls), arr(ns), 7, arr(ls), 0, 400, out) == 175


def _fake(shape, strides, ptr=0x10000):
    from gelib_b200._lib import Tensor5
    t = Tensor5()
    t.base = ptr
    for i in range(5):
        t.dims[i] = shape[i]
        t.strides[i] = strides[i]
    return t


def test_validation_happens_before_any_cuda_call(cabi):
    """Arguments the reference would GELIB_SKIP come back as GELIB_SKIPPED with its message
    (cuda/SO3part_addCGproduct.cu:189-214, core/CGproduct.hpp:48-49); nothing is launched."""
    from gelib_b200._lib import GELIB_INVALID, GELIB_SKIPPED
    dense = lambda b, L, n: _fake((b, 1, 1, L, n), (L * n * 2, 0, 0, n * 2, 2))
    by = ctypes.byref
    r, x, y = dense(4, 5, 4), dense(4, 5, 2), dense(3, 5, 2)
    assert cabi.gelib_SO3part_addCGproduct(by(r), by(x), by(y), 0, 0, None) == GELIB_SKIPPED
    assert b"batch dimensions cannot be reconciled" in cabi.gelib_last_error()
    r, x, y = dense(4, 7, 4), dense(4, 3, 2), dense(4, 3, 2)   # l=3 from 1 x 1
    assert cabi.gelib_SO3part_addCGproduct(by(r), by(x), by(y), 0, 0, None) == GELIB_SKIPPED
    assert b"|l1-l_2| <= l <= l1+l2 not satisfied" in cabi.gelib_last_error()
    r, x, y = dense(4, 3, 4), dense(4, 3, 2), dense(4, 3, 2)
    assert cabi.gelib_SO3part_addCGproduct(by(r), by(x), by(y), 1, 0, None) == GELIB_SKIPPED
    assert b"fragment dimension of r not large enough" in cabi.gelib_last_error()
    r, x, y = dense(4, 3, 4), dense(4, 3, 2), dense(4, 3, 3)
    assert cabi.gelib_SO3part_addDiagCGproduct(by(r), by(x), by(y), 0, 0, None) == GELIB_INVALID
    assert b"N1==N2" in cabi.gelib_last_error()
    assert cabi.gelib_SO3part_addCGproduct(None, by(x), by(y), 0, 0, None) == GELIB_INVALID
    g = _fake((4, 2, 3, 3, 4), (72 * 2, 36 * 2, 12 * 2, 8, 2))
    xg = _fake((4, 2, 2, 3, 2), (48, 24, 12, 4, 2))
    assert cabi.gelib_SO3part_addCGproduct_back0(by(xg), by(g), by(dense(4, 3, 2)), 0, 0, None) == GELIB_SKIPPED
    assert b"grid dimensions cannot be reconciled" in cabi.gelib_last_error()
    assert cabi.gelib_status_string(GELIB_SKIPPED).startswith(b"skipped")


def test_cpu_tensors_are_refused_not_computed():
    """There is no CPU path in the product: a CPU tensor raises instead of silently falling back."""
    import gelib_b200 as G
    x, y = G.SO3part.randn(2, 1, 2), G.SO3part.randn(2, 1, 2)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        G.CGproduct(x, y, 1)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        G.SO3part.spharm(2, torch.randn(2, 3, 4))


def test_descriptor_canonical_form():
    """core/Gpart.hpp:450-469: 3-D -> (b,1,1,L,n), 4-D -> (b,g,1,L,n), >5-D grids fused; float strides."""
    from gelib_b200 import _lib

    class FakeCuda(torch.Tensor):
        is_cuda = True

    def desc(t, **kw):
        return _lib.descriptor(t.as_subclass(FakeCuda), **kw)

    d = desc(torch.zeros(4, 5, 6, dtype=torch.complex64))
    assert list(d.dims) == [4, 1, 1, 5, 6] and list(d.strides) == [60, 0, 0, 12, 2]
    d = desc(torch.zeros(4, 3, 5, 6, dtype=torch.complex64))
    assert list(d.dims) == [4, 3, 1, 5, 6] and list(d.strides) == [180, 60, 0, 12, 2]
    d = desc(torch.zeros(4, 2, 3, 5, 6, dtype=torch.complex64))
    assert list(d.dims) == [4, 2, 3, 5, 6] and list(d.strides) == [360, 180, 60, 12, 2]
    d = desc(torch.zeros(4, 2, 3, 2, 5, 6, dtype=torch.complex64))
    assert list(d.dims) == [4, 12, 1, 5, 6] and list(d.strides) == [720, 60, 0, 12, 2]
    d = desc(torch.zeros(1, 5, 6, dtype=torch.complex64).expand(4, 5, 6))
    assert list(d.strides)[0] == 0
    d = desc(torch.zeros(4, 3, 6), real=True)
    assert list(d.dims) == [4, 1, 1, 3, 6] and list(d.strides) == [18, 0, 0, 6, 1]
    with pytest.raises(RuntimeError):
        desc(torch.zeros(4, 2, 3, 2, 5, 6, dtype=torch.complex64).transpose(1, 2))
    with pytest.raises(RuntimeError):
        desc(torch.zeros(4, 5, 6))


def test_python_surface_matches_reference_names():
    import gelib_b200 as G
    for name in ["SO3part", "SO3vec", "SO3partArr", "SO3vecArr", "SO3type", "SO3weights", "SO3linear", "SO3element",
                 "SO3irrep", "CGproduct", "DiagCGproduct", "SO3part_CGproductFn", "SO3part_DiagCGproductFn",
                 "SO3vec_CGproductFn", "SO3vec_DiagCGproductFn", "common_batch"]:
        assert hasattr(G, name), name
    for name in ["add_CGproduct", "add_CGproduct_back0", "add_CGproduct_back1", "add_DiagCGproduct",
                 "add_DiagCGproduct_back0", "add_DiagCGproduct_back1", "add_spharm", "view"]:
        assert hasattr(G.backend.SO3part, name), name
    for name in ["addCGproduct", "addCGproduct_back0", "addCGproduct_back1", "addDiagCGproduct",
                 "addDiagCGproduct_back0", "addDiagCGproduct_back1", "get_tau", "view"]:
        assert hasattr(G.backend.SO3vec, name), name
    R = G.SO3element.random()
    assert torch.allclose(R @ R.t(), torch.eye(3), atol=1e-5) and abs(float(torch.det(R)) - 1) < 1e-5
    D = G.SO3irrep(3).matrix(R)
    assert torch.allclose(D @ D.conj().t(), torch.eye(7, dtype=torch.complex64), atol=1e-5)


def test_gather_map_csr_and_transpose():
    """gather_map keeps targets -> sources as CSR and the transpose for the gradient; three constructors agree."""
    import torch
    from gelib_b200.backend import gather_map
    m = gather_map.sources_targets([0, 1, 1, 4, 2], [3, 0, 3, 3, 1], n_in=5, n_out=4)
    ptr, col = m._fwd
    assert ptr.tolist() == [0, 1, 2, 2, 5] and col.tolist() == [1, 2, 0, 1, 4]
    bptr, bcol = m._bwd
    assert bptr.tolist() == [0, 1, 3, 4, 4, 5] and bcol.tolist() == [3, 0, 3, 1, 3]
    M = torch.zeros(4, 5)
    for s, t in zip([0, 1, 1, 4, 2], [3, 0, 3, 3, 1]):
        M[t, s] = 1
    m2 = gather_map.from_matrix(M, 5, 4)
    assert m2._fwd[0].tolist() == ptr.tolist() and m2._fwd[1].tolist() == col.tolist()
    assert m.d_in() == 5 and m.d_out() == 4
    r = gather_map.random(6, 3, 0.5, generator=torch.Generator().manual_seed(1))
    assert r.d_in() == 6 and r.d_out() == 3 and int(r._fwd[0][-1]) == int(r._bwd[0][-1])


def test_o3_type_calculus_and_call_plan():
    """O(3) bookkeeping on the host: index order 2l + [p = -1] (O3/O3index.hpp:51-53), p = p1 p2
    (O3/O3group.hpp:38-44), and the slices of the per-(x part, y parity sector) calls tile every output part exactly."""
    from gelib_b200.O3 import O3type, _sector_calls
    tx = O3type({(1, -1): 3, (0, 1): 2, (1, 1): 1})
    assert list(tx.parts) == [(0, 1), (1, 1), (1, -1)]
    ty = O3type({(0, -1): 2, (1, 1): 2, (2, -1): 1})
    tr = tx.CGproduct(ty, 2)
    want = {}
    for (l1, p1), n1 in tx.parts.items():
        for (l2, p2), n2 in ty.parts.items():
            for l in range(abs(l1 - l2), min(l1 + l2, 2) + 1):
                want[(l, p1 * p2)] = want.get((l, p1 * p2), 0) + n1 * n2
    assert tr.parts == dict(sorted(want.items(), key=lambda kv: 2 * kv[0][0] + (kv[0][1] == -1)))
    xmus, ymus = list(tx.parts), list(ty.parts)
    calls = _sector_calls(xmus, list(tx.parts.values()), ymus, list(ty.parts.values()), tr.parts, 2, False)
    covered = {mu: [] for mu in tr.parts}
    for i, js, p, slices in calls:
        assert all(ymus[j][1] * xmus[i][1] == p for j in js)
        for l, (o, w) in slices.items():
            covered[(l, p)].append((o, w))
    for mu, segs in covered.items():
        segs.sort()
        pos = 0
        for o, w in segs:
            assert o == pos
            pos += w
        assert pos == tr.parts[mu]


def test_reference_python_package_imports_on_gelib_base():
    """With this repository's gelib_base on the path, GElib's own Python package imports unchanged and its host-side
    pieces work through the C ABI: type calculus, random group elements, Wigner matrices.  Skipped where the reference
    tree is not present (nothing here needs it at run time on a GPU box)."""
    import os
    import subprocess
    import sys
    import pytest
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # the GElib checkout: GELIB_REFERENCE_SRC, or a directory "reference" beside this repository
    ref = os.environ.get("GELIB_REFERENCE_SRC", os.path.join(os.path.dirname(root), "reference", "python", "src"))
    if not os.path.isdir(os.path.join(ref, "gelib")):
        pytest.skip("the GElib source tree is not present")
    code = (
        "import torch, gelib, gelib_base\n"
        "assert gelib_base.SO3part.view.__module__ == 'gelib_b200.backend'\n"
        "v = gelib.SO3vec.randn(2, {0: 2, 1: 3, 2: 1})\n"
        "tau = v.backend().get_tau().CGproduct(v.backend().get_tau(), 2).get_parts()\n"
        "want = {}\n"
        "t = {0: 2, 1: 3, 2: 1}\n"
        "for l1, n1 in t.items():\n"
        "    for l2, n2 in t.items():\n"
        "        for l in range(abs(l1 - l2), min(l1 + l2, 2) + 1):\n"
        "            want[l] = want.get(l, 0) + n1 * n2\n"
        "assert tau == want, (tau, want)\n"
        "R = gelib.SO3element.random()\n"
        "assert torch.allclose(R @ R.t(), torch.eye(3), atol=1e-5)\n"
        "D = gelib.SO3irrep(2).matrix(R)\n"
        "assert torch.allclose(D @ D.conj().t(), torch.eye(5, dtype=torch.complex64), atol=1e-5)\n"
        "x = gelib.SO3part.randn(2, 1, 3)\n"
        "try:\n"
        "    gelib.CGproduct(x, x, 1)\n"
        "    raise SystemExit('a CPU product must raise: there is no CPU path')\n"
        "except RuntimeError as e:\n"
        "    assert 'CUDA' in str(e)\n"
        "print('ok')\n")
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + ref)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
