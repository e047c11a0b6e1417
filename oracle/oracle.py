"""ctypes front end of the CPU oracle (``oracle/gelib_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``; never by the shipped package.

Besides binding the C routines it restates the vector-level bookkeeping of the reference
(file:line relative to the GElib tree):

* ``cg_type`` / ``diag_type``  -- ``Gtype::CGproduct`` / ``DiagCGproduct``, core/Gtype.hpp:115-138,
  with ``SO3group::for_each_CGcomponent`` (SO3/SO3group.hpp:43-47) and the ``z<=limit`` truncation;
* ``vec_cg`` / ``vec_cg_back0`` / ``vec_cg_back1`` (+ diag) -- ``Gvec::add_CGproduct*`` and
  ``add_DiagCGproduct*``, core/Gvec.hpp:311-389: parts visited in ascending l1, then ascending
  l2, then l = |l1-l2|..l1+l2, skipping l absent from the result, with a running channel
  offset per output l advanced by n1*n2 (full) or n1 (diag).

All tensors are numpy complex64 arrays of shape (batch, 2l+1, n); a batch of 1 broadcasts.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "gelib_oracle.c")
_SO = os.path.join(_HERE, "libgelib_oracle.so")
_lib = None


def build(force=False):
    """Compile the oracle with gcc (no FMA contraction, OpenMP for the all-cores baseline)."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", _SO, _SRC, "-lm"]
    subprocess.check_call(cmd)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.oracle_cg_coeff.restype = ctypes.c_double
        L.oracle_cg_coeff.argtypes = [ctypes.c_int] * 5
        L.oracle_cg_matrix.restype = None
        L.oracle_cg_matrix.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p]
        L.oracle_cg.restype = ctypes.c_int
        L.oracle_cg.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 12
        L.oracle_spharm.restype = ctypes.c_int
        L.oracle_spharm.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5
        L.oracle_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def max_threads():
    return int(lib().oracle_max_threads())


# ---- coefficients ------------------------------------------------------------------------


def cg_coeff(l1, l2, l, m1, m2):
    return float(lib().oracle_cg_coeff(l1, l2, l, m1, m2))


def cg_matrix(l1, l2, l):
    C = np.zeros((2 * l1 + 1, 2 * l2 + 1), dtype=np.float32)
    lib().oracle_cg_matrix(l1, l2, l, C.ctypes.data)
    return C


# ---- single-triple routines -----------------------------------------------------------------


def _chk(a):
    assert isinstance(a, np.ndarray) and a.dtype == np.complex64 and a.ndim == 3 and a.flags.c_contiguous, (
        "oracle tensors are C-contiguous complex64 (batch, 2l+1, n)")
    return a


def _cg(mode, diag, r, x, y, offs, nthreads):
    _chk(r), _chk(x), _chk(y)
    B = max(r.shape[0], x.shape[0], y.shape[0])
    l1, l2, l = (x.shape[1] - 1) // 2, (y.shape[1] - 1) // 2, (r.shape[1] - 1) // 2
    st = lib().oracle_cg(mode, diag, r.ctypes.data, x.ctypes.data, y.ctypes.data, B, r.shape[0], x.shape[0],
                         y.shape[0], l1, l2, l, x.shape[2], y.shape[2], r.shape[2], offs, nthreads)
    if st != 0:
        raise ValueError("oracle: arguments the reference would skip (status %d)" % st)


def add_CGproduct(r, x, y, offs=0, nthreads=1):
    """r += CG(x,y); SO3/SO3part.hpp:205-221."""
    _cg(0, 0, r, x, y, offs, nthreads)


def add_CGproduct_back0(xg, g, y, offs=0, nthreads=1):
    """xg += C g conj(y); SO3/SO3part.hpp:223-239."""
    _cg(1, 0, g, xg, y, offs, nthreads)


def add_CGproduct_back1(yg, g, x, offs=0, nthreads=1):
    """yg += C g conj(x); SO3/SO3part.hpp:241-257."""
    _cg(2, 0, g, x, yg, offs, nthreads)


def add_DiagCGproduct(r, x, y, offs=0, nthreads=1):
    """SO3/SO3part.hpp:276-290."""
    _cg(0, 1, r, x, y, offs, nthreads)


def add_DiagCGproduct_back0(xg, g, y, offs=0, nthreads=1):
    """SO3/SO3part.hpp:292-306."""
    _cg(1, 1, g, xg, y, offs, nthreads)


def add_DiagCGproduct_back1(yg, g, x, offs=0, nthreads=1):
    """SO3/SO3part.hpp:308-322."""
    _cg(2, 1, g, x, yg, offs, nthreads)


def add_spharm(R, X, nthreads=1):
    """R += Y_L(X), X float32 (b,3,n); SO3/SO3part.hpp:340-397."""
    _chk(R)
    assert X.dtype == np.float32 and X.ndim == 3 and X.shape[1] == 3 and X.flags.c_contiguous
    assert X.shape[2] == R.shape[2]
    L = (R.shape[1] - 1) // 2
    st = lib().oracle_spharm(R.ctypes.data, X.ctypes.data, R.shape[0], X.shape[0], L, R.shape[2], nthreads)
    if st != 0:
        raise ValueError("oracle: batch dimensions cannot be reconciled")


# ---- type calculus and vector-level loops ------------------------------------------------------


def cg_type(xtau, ytau, maxl=-1, diag=False):
    """Gtype::CGproduct / DiagCGproduct, core/Gtype.hpp:115-138 (limit -1 = no truncation)."""
    R = {}
    for l1 in sorted(xtau):
        for l2 in sorted(ytau):
            for l in range(abs(l1 - l2), l1 + l2 + 1):
                if maxl == -1 or l <= maxl:
                    R[l] = R.get(l, 0) + (xtau[l1] if diag else xtau[l1] * ytau[l2])
    return dict(sorted(R.items()))


def diag_type(xtau, ytau, maxl=-1):
    return cg_type(xtau, ytau, maxl, diag=True)


def triples(xtau, ytau, rls, diag=False):
    """The (l1,l2,l,offs) schedule of Gvec::add_CGproduct, core/Gvec.hpp:311-321 (diag: :358-367)."""
    offset = {}
    out = []
    for l1 in sorted(xtau):
        for l2 in sorted(ytau):
            for l in range(abs(l1 - l2), l1 + l2 + 1):
                if l not in rls:
                    continue
                out.append((l1, l2, l, offset.get(l, 0)))
                offset[l] = offset.get(l, 0) + (xtau[l1] if diag else xtau[l1] * ytau[l2])
    return out


def _tau(parts):
    return {l: p.shape[2] for l, p in parts.items()}


def vec_cg(r, x, y, diag=False, nthreads=1):
    """r, x, y: dict l -> array.  Gvec::add_CGproduct / add_DiagCGproduct."""
    f = add_DiagCGproduct if diag else add_CGproduct
    for l1, l2, l, offs in triples(_tau(x), _tau(y), set(r), diag):
        f(r[l], x[l1], y[l2], offs, nthreads)


def vec_cg_back0(xg, g, y, diag=False, nthreads=1):
    """Gvec::add_CGproduct_back0, core/Gvec.hpp:323-333 (diag :369-378)."""
    f = add_DiagCGproduct_back0 if diag else add_CGproduct_back0
    for l1, l2, l, offs in triples(_tau(xg), _tau(y), set(g), diag):
        f(xg[l1], g[l], y[l2], offs, nthreads)


def vec_cg_back1(yg, g, x, diag=False, nthreads=1):
    """Gvec::add_CGproduct_back1, core/Gvec.hpp:335-345 (diag :380-389)."""
    f = add_DiagCGproduct_back1 if diag else add_CGproduct_back1
    for l1, l2, l, offs in triples(_tau(x), _tau(yg), set(g), diag):
        f(yg[l2], g[l], x[l1], offs, nthreads)


if __name__ == "__main__":
    print(build(force=True))
