"""Stand-in for GElib's pybind11 module ``gelib_base`` on the Clebsch-Gordan path.

Same class and method names, argument order and defaults as the reference bindings
(python/bindings/SO3part_py.cpp:15-58, python/bindings/SO3vec_py.cpp:15-59,
python/bindings/SO3type_py.cpp:16-43 of GElib); the objects are zero-copy views of torch tensors and
every method forwards to one C-ABI call of ``libgelib_b200.so``.  Additions over the reference are
keyword-only or new names: ``overwrite=`` on the forward products, the fused ``*_back01`` gradients and
``SO3vec.add_spharm``.
"""
import ctypes

import torch

from . import _lib
from ._lib import GELIB_FP64, GELIB_OVERWRITE, check, descriptor, descriptor_array, device_guard, lib, stream_of


def _ints(v):
    return (ctypes.c_int * max(1, len(v)))(*v)


def _flags(overwrite, fp64):
    return (GELIB_OVERWRITE if overwrite else 0) | (GELIB_FP64 if fp64 else 0)


def _one_device(*tensors):
    """The reference asserts that the operands of a product live on one device (SO3/SO3part.hpp:351,
    core/CGproduct.hpp:47-49); here a tensor on another GPU would be dereferenced as a raw pointer."""
    dev = tensors[0].device
    for t in tensors:
        if t.device != dev:
            raise RuntimeError("GElib error: operands on different devices (%s and %s)." % (dev, t.device))


class SO3type:
    """The type of an SO3vec: l -> number of channels.  python/bindings/SO3type_py.cpp:16-43."""

    def __init__(self, arg=None):
        self.parts = {}
        if isinstance(arg, dict):
            self.parts = {int(l): int(n) for l, n in sorted(arg.items())}
        elif arg is not None:
            self.parts = {l: int(n) for l, n in enumerate(arg)}

    def __len__(self):
        return len(self.parts)

    def maxl(self):
        return max(self.parts) if self.parts else -1

    def __getitem__(self, l):
        return self.parts.get(l, 0)

    def __setitem__(self, l, n):
        self.parts[l] = n
        self.parts = dict(sorted(self.parts.items()))

    def get_parts(self):
        return dict(self.parts)

    def _product(self, y, maxl, diag):
        xl, xn = list(self.parts.keys()), list(self.parts.values())
        yl, yn = list(y.parts.keys()), list(y.parts.values())
        cap = (max(xl) + max(yl) + 1) if xl and yl else 1
        ol, on = (ctypes.c_int * cap)(), (ctypes.c_int * cap)()
        k = lib().gelib_SO3type_CGproduct(len(xl), _ints(xl), _ints(xn), len(yl), _ints(yl), _ints(yn), maxl,
                                          1 if diag else 0, cap, ol, on)
        if k < 0:
            raise RuntimeError("GElib error: product type does not fit")
        return SO3type({ol[i]: on[i] for i in range(k)})

    def CGproduct(self, y, maxl=-1):
        return self._product(y, maxl, False)

    def DiagCGproduct(self, y, maxl=-1):
        return self._product(y, maxl, True)

    def __eq__(self, other):
        return isinstance(other, SO3type) and self.parts == other.parts

    def str(self, indent=""):
        return indent + "(" + ",".join("%d:%d" % (l, n) for l, n in self.parts.items()) + ")"

    __str__ = str

    def __repr__(self):
        return "<GElib::SO3type" + self.str() + ">"


def CGproduct(x, y, maxl=-1):
    """``gelib_base.CGproduct`` on two SO3types (python/bindings/SO3type_py.cpp:39-43)."""
    return x.CGproduct(y, maxl)


class gather_map:
    """``gelib_base.gather_map`` (python/bindings/gather_map_py.cpp:15-29): which cells of an array dimension are summed
    into which.  cnine's GatherMapB is not part of the reference tree, so the three constructors are restated from
    their published signatures: ``sources_targets`` pairs up two index lists (source i feeds target i),
    ``from_matrix`` reads an (n_out, n_in) matrix whose non-zero entries mark (target, source) pairs, ``random`` draws
    every (target, source) pair with probability p.  Held as CSR (targets -> sources) and its transpose, as int32
    tensors that follow the operand's device."""

    def __init__(self, n_in, n_out, targets, sources):
        self.n_in, self.n_out = int(n_in), int(n_out)
        t = torch.as_tensor(targets, dtype=torch.int64).reshape(-1)
        s = torch.as_tensor(sources, dtype=torch.int64).reshape(-1)
        assert t.numel() == s.numel()
        if t.numel():
            assert int(t.min()) >= 0 and int(t.max()) < self.n_out and int(s.min()) >= 0 and int(s.max()) < self.n_in
        self._fwd = self._csr(t, s, self.n_out)
        self._bwd = self._csr(s, t, self.n_in)
        self._dev = {}

    @staticmethod
    def _csr(rows, cols, nrows):
        order = torch.argsort(rows, stable=True)
        counts = torch.bincount(rows, minlength=nrows)
        ptr = torch.zeros(nrows + 1, dtype=torch.int64)
        ptr[1:] = torch.cumsum(counts, 0)
        return ptr.to(torch.int32), cols[order].to(torch.int32)

    @classmethod
    def sources_targets(cls, sources, targets, n_in=None, n_out=None):
        n_in = (max(sources) + 1 if len(sources) else 0) if n_in is None else n_in
        n_out = (max(targets) + 1 if len(targets) else 0) if n_out is None else n_out
        return cls(n_in, n_out, targets, sources)

    @classmethod
    def from_matrix(cls, M, n_in, n_out):
        M = torch.as_tensor(M)
        assert list(M.shape) == [n_out, n_in]
        idx = torch.nonzero(M.cpu())
        return cls(n_in, n_out, idx[:, 0], idx[:, 1])

    @classmethod
    def random(cls, n, m, p=0.5, generator=None):
        return cls.from_matrix(torch.rand(m, n, generator=generator) < p, n, m)

    def d_in(self):
        return self.n_in

    def d_out(self):
        return self.n_out

    def csr(self, device, transposed=False):
        key = (str(device), transposed)
        if key not in self._dev:
            ptr, col = self._bwd if transposed else self._fwd
            if col.numel() == 0:
                col = torch.zeros(1, dtype=torch.int32)
            self._dev[key] = (ptr.to(device), col.to(device))
        return self._dev[key]

    def __repr__(self):
        return "<GElib::gather_map(n_in=%d,n_out=%d,pairs=%d)>" % (self.n_in, self.n_out, int(self._fwd[0][-1]))

    def str(self, indent=""):
        ptr, col = self._fwd
        return "\n".join("%s%d<-(%s)" % (indent, t, ",".join(str(int(c)) for c in col[ptr[t]:ptr[t + 1]]))
                         for t in range(self.n_out) if ptr[t + 1] > ptr[t])

    __str__ = str


def _gather(r, x, gmap, d, transposed):
    """r[.., t, ..] += sum of x[.., s, ..] along array dimension d (tensor dimension d + 1)."""
    _one_device(r, x)
    if not r.is_cuda:
        raise RuntimeError("gelib_b200: tensors must live on a CUDA device (there is no CPU path).")
    if not (r.is_contiguous() and x.is_contiguous()):
        raise RuntimeError("GElib error: add_gather needs contiguous tensors.")
    n_out, n_in = (gmap.n_in, gmap.n_out) if transposed else (gmap.n_out, gmap.n_in)
    if r.size(d + 1) != n_out or x.size(d + 1) != n_in:
        raise RuntimeError("GElib error: gather map does not match the array dimension.")
    outer = 1
    for k in range(d + 1):
        outer *= r.size(k)
    inner = 1
    for k in range(d + 2, r.dim()):
        inner *= r.size(k)
    ptr, col = gmap.csr(r.device, transposed)
    with device_guard(r):
        return check(lib().gelib_add_gather(r.data_ptr(), x.data_ptr(), outer, n_out, n_in, inner, ptr.data_ptr(),
                                            col.data_ptr(), stream_of(r)))


MIX_MAX_CHANNELS = 64


def mix_supported(x, w):
    """True when (x, w) can take the mixing kernels: CUDA complex64, w a matrix with at most 64 channels a side."""
    return (x.is_cuda and w.is_cuda and x.dtype == torch.complex64 and w.dtype == torch.complex64 and w.dim() == 2
            and x.dim() >= 2 and x.size(-1) == w.size(0) and 1 <= w.size(0) <= MIX_MAX_CHANNELS
            and 1 <= w.size(1) <= MIX_MAX_CHANNELS and x.numel() > 0)


def mix(x, w, adjoint=False):
    """x (.., n_in) times w (n_in, n_out), or with adjoint=True x (.., n_out) times w^H: a new dense tensor."""
    _one_device(x, w)
    x, w = x.contiguous(), w.contiguous()
    n_in, n_out = w.size(0), w.size(1)
    rows = x.numel() // x.size(-1)
    r = torch.empty(list(x.shape[:-1]) + [n_in if adjoint else n_out], dtype=torch.complex64, device=x.device)
    with device_guard(x):
        check(lib().gelib_SO3part_mix(r.data_ptr(), x.data_ptr(), w.data_ptr(), rows, n_in, n_out, 1 if adjoint else 0,
                                      stream_of(x)))
    return r


def mix_back_w(x, g, n_in, n_out):
    """x^H g summed over all rows: the gradient of the weight matrix, (n_in, n_out)."""
    _one_device(x, g)
    x, g = x.contiguous(), g.contiguous()
    rows = x.numel() // x.size(-1)
    wg = torch.zeros(n_in, n_out, dtype=torch.complex64, device=x.device)
    with device_guard(x):
        check(lib().gelib_SO3part_mix_back_w(wg.data_ptr(), x.data_ptr(), g.data_ptr(), rows, n_in, n_out, stream_of(x)))
    return wg


def SO3irrep_matrix(l, alpha, beta, gamma):
    """D^l(alpha, beta, gamma) as a (2l+1, 2l+1) complex64 CPU tensor (SO3irrep::matrix, SO3/SO3irrep.hpp:69-103)."""
    out = torch.zeros(2 * l + 1, 2 * l + 1, dtype=torch.complex64)
    check(lib().gelib_SO3irrep_matrix(l, float(alpha), float(beta), float(gamma), out.data_ptr()))
    return out


class SO3part:
    """Zero-copy view of a complex64 tensor (batch, [grid...], 2l+1, channels)."""

    def __init__(self, t):
        self.t = t

    @staticmethod
    def view(t):
        return SO3part(t)

    def getl(self):
        return (self.t.size(-2) - 1) // 2

    def getn(self):
        return self.t.size(-1)

    def _call3(self, name, a, b, c, offs, flags=0):
        _one_device(a, b, c)
        with device_guard(a):
            da, db, dc = descriptor(a), descriptor(b), descriptor(c)
            return check(getattr(lib(), name)(ctypes.byref(da), ctypes.byref(db), ctypes.byref(dc), offs, flags,
                                              stream_of(a)))

    # fp64=True: coefficients and sums in double (GELIB_FP64), through the general strided kernels
    def add_CGproduct(self, x, y, offs=0, *, overwrite=False, fp64=False):
        return self._call3("gelib_SO3part_addCGproduct", self.t, x.t, y.t, offs, _flags(overwrite, fp64))

    def add_CGproduct_back0(self, g, y, offs=0, *, fp64=False):
        return self._call3("gelib_SO3part_addCGproduct_back0", self.t, g.t, y.t, offs, _flags(False, fp64))

    def add_CGproduct_back1(self, g, x, offs=0, *, fp64=False):
        return self._call3("gelib_SO3part_addCGproduct_back1", self.t, g.t, x.t, offs, _flags(False, fp64))

    def add_DiagCGproduct(self, x, y, offs=0, *, overwrite=False, fp64=False):
        return self._call3("gelib_SO3part_addDiagCGproduct", self.t, x.t, y.t, offs, _flags(overwrite, fp64))

    def add_DiagCGproduct_back0(self, g, y, offs=0, *, fp64=False):
        return self._call3("gelib_SO3part_addDiagCGproduct_back0", self.t, g.t, y.t, offs, _flags(False, fp64))

    def add_DiagCGproduct_back1(self, g, x, offs=0, *, fp64=False):
        return self._call3("gelib_SO3part_addDiagCGproduct_back1", self.t, g.t, x.t, offs, _flags(False, fp64))

    @staticmethod
    def _back01(name, xg, yg, g, x, y, offs):
        _one_device(xg.t, yg.t, g.t, x.t, y.t)
        with device_guard(g.t):
            d = [descriptor(v.t) for v in (xg, yg, g, x, y)]
            return check(getattr(lib(), name)(*[ctypes.byref(v) for v in d], offs, 0, stream_of(g.t)))

    @staticmethod
    def add_CGproduct_back01(xg, yg, g, x, y, offs=0):
        """Both gradients from one pass over g (fused back0 + back1)."""
        return SO3part._back01("gelib_SO3part_addCGproduct_back01", xg, yg, g, x, y, offs)

    @staticmethod
    def add_DiagCGproduct_back01(xg, yg, g, x, y, offs=0):
        return SO3part._back01("gelib_SO3part_addDiagCGproduct_back01", xg, yg, g, x, y, offs)

    def add_gather(self, x, gmap, d=0):
        """python/bindings/SO3part_py.cpp:21-22."""
        return _gather(self.t, x.t if isinstance(x, SO3part) else x, gmap, d, False)

    def add_gather_back(self, rg, gmap, d=0):
        """python/bindings/SO3part_py.cpp:23-24: the gradient of add_gather (the transposed map)."""
        return _gather(self.t, rg.t if isinstance(rg, SO3part) else rg, gmap, d, True)

    def add_apply(self, x, D, *, overwrite=False):
        """self (+)= D x cell by cell; D a (2l+1, 2l+1) complex64 tensor on the same device."""
        _one_device(self.t, x.t, D)
        with device_guard(self.t):
            dr, dx = descriptor(self.t), descriptor(x.t)
            Dc = D.contiguous()
            return check(lib().gelib_SO3part_apply(ctypes.byref(dr), ctypes.byref(dx), Dc.data_ptr(),
                                                   GELIB_OVERWRITE if overwrite else 0, stream_of(self.t)))

    def add_spharm(self, X, *, overwrite=False):
        """self += Y_l(X) for X (batch, [grid...], 3, channels) float32, or (3, channels) broadcast over the batch."""
        if X.dim() == 2:
            X = X.unsqueeze(0)
        _one_device(self.t, X)
        with device_guard(self.t):
            dr, dx = descriptor(self.t), descriptor(X, real=True)
            check(lib().gelib_SO3part_addSPharm(ctypes.byref(dr), ctypes.byref(dx), GELIB_OVERWRITE if overwrite else 0,
                                                stream_of(self.t)))

    def __repr__(self):
        return "<GElib::SO3part(l=%d,n=%d)>" % (self.getl(), self.getn())

    def str(self, indent=""):
        return indent + str(self.t)

    __str__ = str


class SO3vec:
    """Zero-copy view of a list (l read from the shapes) or dict l -> tensor of SO3parts."""

    def __init__(self, parts):
        self.parts = parts  # dict l -> tensor, ascending l

    @staticmethod
    def view(parts):
        if isinstance(parts, dict):
            return SO3vec(dict(sorted((int(l), t) for l, t in parts.items())))
        return SO3vec(dict(sorted(((t.size(-2) - 1) // 2, t) for t in parts)))

    def get_tau(self):
        return SO3type({l: t.size(-1) for l, t in self.parts.items()})

    def _tensors(self):
        return list(self.parts.values())

    def _call3(self, name, a, b, c, flags=0):
        ta, tb, tc = a._tensors(), b._tensors(), c._tensors()
        if not ta or not tb or not tc:
            return True
        _one_device(*(ta + tb + tc))
        with device_guard(ta[0]):
            return check(getattr(lib(), name)(len(ta), descriptor_array(ta), len(tb), descriptor_array(tb), len(tc),
                                              descriptor_array(tc), flags, stream_of(ta[0])))

    def addCGproduct(self, x, y, *, overwrite=False, fp64=False):
        return self._call3("gelib_SO3vec_addCGproduct", self, x, y, _flags(overwrite, fp64))

    def addCGproduct_static(self, x, y, *, overwrite=False):
        """addCGproduct through the entry point that allocates no device memory (tables in a fixed 64 KB device
        array shared by all calls: do not let two such calls overlap on the GPU)."""
        return self._call3("gelib_SO3vec_addCGproduct_static", self, x, y, GELIB_OVERWRITE if overwrite else 0)

    def addCGproduct_spharm(self, X, lmax_x, y, *, overwrite=False):
        """self (+)= CGproduct(spharms(lmax_x, X), y) with the harmonics generated inside the kernel; X (batch, 3, 1)."""
        tr, ty = self._tensors(), y._tensors()
        _one_device(*(tr + ty + [X]))
        with device_guard(tr[0]):
            dx = descriptor(X, real=True)
            return check(lib().gelib_SO3vec_addCGproduct_spharm(len(tr), descriptor_array(tr), ctypes.byref(dx), lmax_x,
                                                                len(ty), descriptor_array(ty),
                                                                GELIB_OVERWRITE if overwrite else 0, stream_of(tr[0])))

    def addCGproduct_spharm_back1(self, g, X, lmax_x):
        """self (the gradient of y) += C g conj(spharms(lmax_x, X))."""
        tyg, tg = self._tensors(), g._tensors()
        _one_device(*(tyg + tg + [X]))
        with device_guard(tg[0]):
            dx = descriptor(X, real=True)
            return check(lib().gelib_SO3vec_addCGproduct_spharm_back1(len(tyg), descriptor_array(tyg), len(tg),
                                                                      descriptor_array(tg), ctypes.byref(dx), lmax_x, 0,
                                                                      stream_of(tg[0])))

    def addCGproduct_back0(self, g, y, *, fp64=False):
        return self._call3("gelib_SO3vec_addCGproduct_back0", self, g, y, _flags(False, fp64))

    def addCGproduct_back1(self, g, x, *, fp64=False):
        return self._call3("gelib_SO3vec_addCGproduct_back1", self, g, x, _flags(False, fp64))

    def addDiagCGproduct(self, x, y, *, overwrite=False):
        return self._call3("gelib_SO3vec_addDiagCGproduct", self, x, y, GELIB_OVERWRITE if overwrite else 0)

    def addDiagCGproduct_back0(self, g, y):
        return self._call3("gelib_SO3vec_addDiagCGproduct_back0", self, g, y)

    def addDiagCGproduct_back1(self, g, x):
        return self._call3("gelib_SO3vec_addDiagCGproduct_back1", self, g, x)

    @staticmethod
    def _back01(name, xg, yg, g, x, y):
        txg, tyg, tg, tx, ty = (v._tensors() for v in (xg, yg, g, x, y))
        if not tg or not tx or not ty:
            return True
        if len(txg) != len(tx) or len(tyg) != len(ty):
            raise RuntimeError("GElib error: gradient vectors must have the parts of x and y.")
        _one_device(*(txg + tyg + tg + tx + ty))
        with device_guard(tg[0]):
            return check(getattr(lib(), name)(len(txg), descriptor_array(txg), len(tyg), descriptor_array(tyg),
                                              len(tg), descriptor_array(tg), descriptor_array(tx),
                                              descriptor_array(ty), 0, stream_of(tg[0])))

    @staticmethod
    def addCGproduct_back01(xg, yg, g, x, y):
        """Both gradients of the full product from one pass over g."""
        return SO3vec._back01("gelib_SO3vec_addCGproduct_back01", xg, yg, g, x, y)

    @staticmethod
    def addDiagCGproduct_back01(xg, yg, g, x, y):
        return SO3vec._back01("gelib_SO3vec_addDiagCGproduct_back01", xg, yg, g, x, y)

    def add_spharm(self, X, *, overwrite=False):
        """Every part += its spherical harmonics of X, from one Legendre recursion per point."""
        tr = self._tensors()
        if X.dim() == 2:
            X = X.unsqueeze(0)
        _one_device(*(tr + [X]))
        with device_guard(tr[0]):
            dx = descriptor(X, real=True)
            check(lib().gelib_SO3vec_addSPharm(len(tr), descriptor_array(tr), ctypes.byref(dx),
                                               GELIB_OVERWRITE if overwrite else 0, stream_of(tr[0])))

    def __repr__(self):
        return "<GElib::SO3vec of type " + self.get_tau().str() + ">"

    def str(self, indent=""):
        return "\n".join("%sPart l=%d:\n%s\n" % (indent, l, t) for l, t in self.parts.items())

    __str__ = str


def SO3CGmatrix(l1, l2, l):
    """Dense (2l1+1) x (2l2+1) coefficient matrix (``gelib.SO3CGmatrix`` of the docs, python/docs/source/SO3CG.rst:49-53)."""
    out = torch.zeros(2 * l1 + 1, 2 * l2 + 1, dtype=torch.float32)
    if lib().gelib_CGmatrix(l1, l2, l, out.data_ptr()) != _lib.GELIB_OK:
        raise RuntimeError(_lib.last_error())
    return out


def kernel_launch_count():
    return int(lib().gelib_kernel_launch_count())


# ---- the remaining names GElib's Python package takes from gelib_base ----------------------------------------------
# (python/src/gelib/SO3element.py:31, SO3irrep.py:22-34, O3element.py, O3irrep.py, O3part.py:118, O3vec.py:101-102)


class _Element:
    """What ``gelib_base.SO3element`` / ``O3element`` hand to Python: a 3x3 matrix with ``.torch()``."""

    def __init__(self, t):
        self.t = t

    def torch(self):
        return self.t

    @classmethod
    def view(cls, t):
        return cls(t)


class SO3element(_Element):

    @classmethod
    def random(cls):
        from .SO3element import SO3element as E
        return cls(E.random().as_subclass(torch.Tensor))


class O3element(_Element):

    @classmethod
    def random(cls):
        from .O3 import O3element as E
        return cls(E.random().as_subclass(torch.Tensor))


class SO3irrep:
    """``gelib_base.SO3irrep``: matrix(element view) or matrix(alpha, beta, gamma) -> (2l+1, 2l+1) complex64."""

    def __init__(self, l):
        self.l = l

    def matrix(self, *args):
        from .SO3irrep import euler_zyz
        if len(args) == 3:
            a, b, c = args
        else:
            R = args[0].t if isinstance(args[0], _Element) else args[0]
            a, b, c = euler_zyz(R.detach().cpu().numpy())
        return SO3irrep_matrix(self.l, a, b, c)

    def __repr__(self):
        return "<GElib::SO3irrep(l=%d)>" % self.l


class O3irrep:

    def __init__(self, l, p):
        self.l, self.p = l, p

    def matrix(self, *args):
        from .O3 import O3irrep as I
        if len(args) >= 3:
            return I(self.l, self.p).matrix(list(args[:3]), p=args[3] if len(args) > 3 else 1)
        R = args[0].t if isinstance(args[0], _Element) else args[0]
        return I(self.l, self.p).matrix(R)

    def __repr__(self):
        return "<GElib::O3irrep(l=%d,p=%d)>" % (self.l, self.p)


class O3type:

    def __init__(self, x=None):
        from .O3 import O3type as T
        self.obj = T(x)

    def get_parts(self):
        return self.obj.get_parts()

    def CGproduct(self, y, maxl=-1):
        r = O3type()
        r.obj = self.obj.CGproduct(y.obj, maxl)
        return r

    def DiagCGproduct(self, y, maxl=-1):
        r = O3type()
        r.obj = self.obj.DiagCGproduct(y.obj, maxl)
        return r

    def __repr__(self):
        return repr(self.obj)

    __str__ = __repr__


class O3part(SO3part):
    """``gelib_base.O3part.view(t, mu)``: the SO(3) view plus the parity (O3/O3part.hpp:222-269 forwards every product)."""

    def __init__(self, t, mu=None):
        super().__init__(t)
        self.mu = mu

    @staticmethod
    def view(t, mu=None):
        return O3part(t, mu)

    def __repr__(self):
        return "<GElib::O3part(l=%d,n=%d)>" % (self.getl(), self.getn())
