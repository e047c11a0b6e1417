"""O(3) parts and vectors on the SO(3) kernels (O3/O3part.hpp:214-278, O3/O3group.hpp:38-52 of GElib).

An irrep of O(3) is mu = (l, p) with parity p = +1 or -1.  The reference's O3part forwards every product to the
SO3part kernels (O3/O3part.hpp:222-269); what O(3) adds is bookkeeping: a product (l1,p1) x (l2,p2) -> (l,p) exists
only for p = p1 p2 (O3group::CGmultiplicity, O3/O3group.hpp:38-44), parts are ordered by 2l + [p = -1]
(O3/O3index.hpp:51-53), and a group element with determinant -1 acts on a part of parity -1 with an extra sign
(O3/O3irrep.hpp:36-41).  The classes mirror python/src/gelib/O3element.py, O3irrep.py, O3type.py, O3part.py and O3vec.py.

A vector-level product runs as one C-ABI vector call per (part of x, parity sector of y): inside such a call the output
blocks appear in the order the reference's loop writes them, so every output part is handed over as a channel slice at
the running offset of that loop (core/Gvec.hpp:311-321 with O(3) indices).
"""
import torch

from . import backend as gb
from .gelib_common import common_batch
from .SO3element import SO3element
from .SO3irrep import SO3irrep


def _key(mu):
    return 2 * mu[0] + (1 if mu[1] == -1 else 0)


def _check_mu(mu):
    assert isinstance(mu, tuple) and len(mu) == 2 and isinstance(mu[0], int) and mu[1] in (1, -1)


class O3element(torch.Tensor):
    """A 3x3 orthogonal matrix (python/src/gelib/O3element.py)."""

    @staticmethod
    def __new__(cls, t):
        return torch.Tensor._make_subclass(cls, t.detach() if isinstance(t, torch.Tensor) else torch.as_tensor(t))

    def __init__(self, t):
        pass

    @classmethod
    def identity(cls):
        return O3element(torch.eye(3))

    @classmethod
    def random(cls, generator=None):
        """A random rotation, reflected through the origin with probability one half."""
        R = SO3element.random(generator).as_subclass(torch.Tensor)
        if torch.rand(1, generator=generator).item() < 0.5:
            R = -R
        return O3element(R)

    def parity(self):
        return 1 if torch.det(self.as_subclass(torch.Tensor).double()) > 0 else -1

    def __mul__(self, y):
        assert isinstance(y, O3element)
        return O3element(torch.matmul(self, y))

    def inv(self):
        return O3element(self.t())


class O3irrep:
    """python/src/gelib/O3irrep.py, O3/O3irrep.hpp:36-48."""

    def __init__(self, l, p):
        assert isinstance(l, int) and p in (1, -1)
        self.l, self.p = l, p

    def matrix(self, R, beta=None, gamma=None, p=1):
        if isinstance(R, torch.Tensor):
            det = O3element(R).parity()
            D = SO3irrep(self.l).matrix(SO3element(R.as_subclass(torch.Tensor) * det))
            return -D if (self.p == -1 and det == -1) else D
        if isinstance(R, (list, tuple)):
            R, beta, gamma = R
        D = SO3irrep(self.l).matrix(R, beta, gamma)
        return -D if (self.p == -1 and p == -1) else D

    def __repr__(self):
        return "<GElib::O3irrep(l=%d,p=%d)>" % (self.l, self.p)


class O3type:
    """The type of an O3vec: (l, p) -> number of channels, ordered by 2l + [p = -1]."""

    def __init__(self, x=None):
        self.parts = {}
        if isinstance(x, dict):
            for mu, n in x.items():
                _check_mu(mu)
                self.parts[mu] = int(n)
        self.parts = dict(sorted(self.parts.items(), key=lambda kv: _key(kv[0])))

    def get_parts(self):
        return dict(self.parts)

    def _product(self, y, maxl, diag):
        out = {}
        for (l1, p1), n1 in self.parts.items():
            for (l2, p2), n2 in y.parts.items():
                for l in range(abs(l1 - l2), l1 + l2 + 1):
                    if maxl == -1 or l <= maxl:
                        out[(l, p1 * p2)] = out.get((l, p1 * p2), 0) + (n1 if diag else n1 * n2)
        return O3type(out)

    def CGproduct(self, y, maxl=-1):
        return self._product(y, maxl, False)

    def DiagCGproduct(self, y, maxl=-1):
        return self._product(y, maxl, True)

    def __eq__(self, other):
        return isinstance(other, O3type) and self.parts == other.parts

    def __repr__(self):
        return "<GElib::O3type(" + ",".join("(%d,%d):%d" % (l, p, n) for (l, p), n in self.parts.items()) + ")>"

    __str__ = __repr__


class O3part(torch.Tensor):
    """n vectors per batch element transforming under the irrep mu = (l, p) of O(3): a complex64 tensor
    (batch, 2l+1, n) that carries mu (python/src/gelib/O3part.py:21-40)."""

    @staticmethod
    def __new__(cls, t, mu):
        _check_mu(mu)
        r = t.as_subclass(cls)
        r.mu = mu
        return r

    def __init__(self, t, mu):
        pass

    @classmethod
    def zeros(cls, b, mu, n, device='cpu'):
        return O3part(torch.zeros([b, 2 * mu[0] + 1, n], dtype=torch.complex64, device=device), mu)

    @classmethod
    def randn(cls, b, mu, n, device='cpu'):
        return O3part(torch.randn([b, 2 * mu[0] + 1, n], dtype=torch.complex64, device=device), mu)

    @classmethod
    def spharm(cls, l, X):
        """Spherical harmonics have parity (-1)^l (O3/O3part.hpp:274-277)."""
        assert X.dim() == 3
        R = torch.empty([X.size(0), 2 * l + 1, X.size(2)], dtype=torch.complex64, device=X.device)
        gb.SO3part.view(R).add_spharm(X, overwrite=True)
        return O3part(R, (l, 1 - 2 * (l % 2)))

    @classmethod
    def randn_like(cls, x):
        return O3part(torch.randn_like(x.as_subclass(torch.Tensor)), x.mu)

    def zeros_like(self):
        return O3part(torch.zeros_like(self.as_subclass(torch.Tensor)), self.mu)

    def backend(self):
        return gb.SO3part.view(self.as_subclass(torch.Tensor))

    def getb(self):
        return self.size(0)

    def get_mu(self):
        return self.mu

    def getl(self):
        return self.mu[0]

    def getp(self):
        return self.mu[1]

    def getn(self):
        return self.size(2)

    def apply(self, R):
        assert isinstance(R, O3element)
        D = O3irrep(self.getl(), self.getp()).matrix(R).to(self.device)
        t = self.as_subclass(torch.Tensor)
        if not t.is_cuda:
            return O3part(torch.matmul(D, t), self.mu)
        from .SO3part import _ApplyFn
        return O3part(_ApplyFn.apply(t, D), self.mu)

    def odot(self, y):
        return torch.sum(torch.view_as_real(self.as_subclass(torch.Tensor)) * torch.view_as_real(y.as_subclass(torch.Tensor)))

    def CGproduct(self, y, mu):
        assert isinstance(y, O3part)
        return O3part_CGproductFn.apply(self, y, mu)

    def DiagCGproduct(self, y, mu):
        assert isinstance(y, O3part)
        return O3part_DiagCGproductFn.apply(self, y, mu)

    def __repr__(self):
        return "<GElib::O3part(b=%d,l=%d,p=%d,n=%d)>" % (self.getb(), self.getl(), self.getp(), self.getn())

    def __str__(self):
        return str(self.as_subclass(torch.Tensor))


def _plain(t):
    return t.detach().as_subclass(torch.Tensor)


def _part_forward(ctx, x, y, mu, diag):
    _check_mu(mu)
    assert x.getp() * y.getp() == mu[1], "parity of the product is the product of the parities"
    ctx.mu, ctx.diag = mu, diag
    ctx.save_for_backward(x, y)
    b = common_batch(x, y)
    n = x.size(-1) if diag else x.size(-1) * y.size(-1)
    r = torch.empty([b, 2 * mu[0] + 1, n], dtype=torch.complex64, device=x.device)
    rb, xb, yb = gb.SO3part.view(r), gb.SO3part.view(_plain(x)), gb.SO3part.view(_plain(y))
    done = (rb.add_DiagCGproduct if diag else rb.add_CGproduct)(xb, yb, overwrite=True)
    if not done:
        r.zero_()
    return O3part(r, mu)


def _part_backward(ctx, g):
    x, y = ctx.saved_tensors
    xg, yg = torch.zeros_like(_plain(x)), torch.zeros_like(_plain(y))
    f = gb.SO3part.add_DiagCGproduct_back01 if ctx.diag else gb.SO3part.add_CGproduct_back01
    f(gb.SO3part.view(xg), gb.SO3part.view(yg), gb.SO3part.view(_plain(g).contiguous()), gb.SO3part.view(_plain(x)),
      gb.SO3part.view(_plain(y)))
    return xg, yg, None


class O3part_CGproductFn(torch.autograd.Function):
    """python/src/gelib/O3part.py:175-202."""

    @staticmethod
    def forward(ctx, x, y, mu):
        return _part_forward(ctx, x, y, mu, False)

    @staticmethod
    def backward(ctx, g):
        return _part_backward(ctx, g)


class O3part_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/O3part.py:205-232."""

    @staticmethod
    def forward(ctx, x, y, mu):
        return _part_forward(ctx, x, y, mu, True)

    @staticmethod
    def backward(ctx, g):
        return _part_backward(ctx, g)


# ---- vectors ------------------------------------------------------------------------------------------------


def _sector_calls(xmus, xn, ymus, yn, rtype, maxl, diag):
    """The calls a vector product is made of: for every part of x (in index order) and either parity sector of y, the
    parts of y in the sector and, per output l, (first channel, width) of the slice of part (l, p) the call writes."""
    offs = {mu: 0 for mu in rtype}
    calls = []
    for i, (l1, p1) in enumerate(xmus):
        slices = {1: {}, -1: {}}
        # the reference's loop order: y parts in index order, both parities interleaved
        for j, (l2, p2) in enumerate(ymus):
            for l in range(abs(l1 - l2), l1 + l2 + 1):
                if maxl != -1 and l > maxl:
                    continue
                w = xn[i] if diag else xn[i] * yn[j]
                mu = (l, p1 * p2)
                s = slices[p2].setdefault(l, [offs[mu], 0])
                assert s[0] + s[1] == offs[mu]  # a sector's blocks of one output part are contiguous
                s[1] += w
                offs[mu] += w
        for p2 in (1, -1):
            js = [j for j, mu in enumerate(ymus) if mu[1] == p2]
            if js and slices[p2]:
                calls.append((i, js, p1 * p2, slices[p2]))
    return calls


def _vec_forward(ctx, k1, k2, maxl, xmus, ymus, args, diag):
    xs, ys = [_plain(a) for a in args[:k1]], [_plain(a) for a in args[k1:k1 + k2]]
    xn, yn = [t.size(-1) for t in xs], [t.size(-1) for t in ys]
    rtype = (O3type(dict(zip(xmus, xn))).DiagCGproduct if diag else O3type(dict(zip(xmus, xn))).CGproduct)(
        O3type(dict(zip(ymus, yn))), maxl).get_parts()
    b = common_batch(xs[0], ys[0])
    rparts = {mu: torch.empty([b, 2 * mu[0] + 1, n], dtype=torch.complex64, device=xs[0].device) for mu, n in rtype.items()}
    calls = _sector_calls(xmus, xn, ymus, yn, rtype, maxl, diag)
    ctx.calls, ctx.k1, ctx.k2, ctx.diag, ctx.rmus = calls, k1, k2, diag, list(rtype)
    ctx.save_for_backward(*args)
    for i, js, p, slices in calls:
        rv = gb.SO3vec.view([rparts[(l, p)][..., o:o + w] for l, (o, w) in slices.items()])
        xv, yv = gb.SO3vec.view([xs[i]]), gb.SO3vec.view([ys[j] for j in js])
        (rv.addDiagCGproduct if diag else rv.addCGproduct)(xv, yv, overwrite=True)
    return tuple(O3part(t, mu) for mu, t in rparts.items())


def _vec_backward(ctx, gargs):
    saved = [_plain(t) for t in ctx.saved_tensors]
    xs, ys = saved[:ctx.k1], saved[ctx.k1:ctx.k1 + ctx.k2]
    g = {mu: _plain(t).contiguous() for mu, t in zip(ctx.rmus, gargs)}
    xg, yg = [torch.zeros_like(t) for t in xs], [torch.zeros_like(t) for t in ys]
    f = gb.SO3vec.addDiagCGproduct_back01 if ctx.diag else gb.SO3vec.addCGproduct_back01
    for i, js, p, slices in ctx.calls:
        gv = gb.SO3vec.view([g[(l, p)][..., o:o + w] for l, (o, w) in slices.items()])
        f(gb.SO3vec.view([xg[i]]), gb.SO3vec.view([yg[j] for j in js]), gv, gb.SO3vec.view([xs[i]]),
          gb.SO3vec.view([ys[j] for j in js]))
    return tuple([None] * 5 + xg + yg)


class O3vec_CGproductFn(torch.autograd.Function):
    """python/src/gelib/O3vec.py:188-224."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, xmus, ymus, *args):
        return _vec_forward(ctx, k1, k2, maxl, xmus, ymus, args, False)

    @staticmethod
    def backward(ctx, *gargs):
        return _vec_backward(ctx, gargs)


class O3vec_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/O3vec.py:228-264."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, xmus, ymus, *args):
        return _vec_forward(ctx, k1, k2, maxl, xmus, ymus, args, True)

    @staticmethod
    def backward(ctx, *gargs):
        return _vec_backward(ctx, gargs)


class O3vec:
    """An O(3)-covariant vector: O3parts keyed by (l, p), in index order (python/src/gelib/O3vec.py:22-40)."""

    def __init__(self, *args):
        self.parts = {}
        for x in args:
            assert isinstance(x, O3part)
            self.parts[x.mu] = x
        self.parts = dict(sorted(self.parts.items(), key=lambda kv: _key(kv[0])))

    @classmethod
    def zeros(cls, b, tau, device='cpu'):
        return O3vec(*[O3part.zeros(b, mu, n, device) for mu, n in tau.items()])

    @classmethod
    def randn(cls, b, tau, device='cpu'):
        return O3vec(*[O3part.randn(b, mu, n, device) for mu, n in tau.items()])

    @classmethod
    def spharm(cls, l, X):
        return O3vec(O3part.spharm(l, X))

    @classmethod
    def zeros_like(cls, x):
        return O3vec(*[p.zeros_like() for p in x.parts.values()])

    @classmethod
    def randn_like(cls, x):
        return O3vec(*[O3part.randn_like(p) for p in x.parts.values()])

    def getb(self):
        return next(iter(self.parts.values())).size(0)

    def tau(self):
        return {mu: p.size(-1) for mu, p in self.parts.items()}

    get_type = tau

    def requires_grad_(self):
        for p in self.parts.values():
            p.requires_grad_()

    def get_grad(self):
        return O3vec(*[O3part(p.grad, mu) for mu, p in self.parts.items()])

    def apply(self, R):
        return O3vec(*[p.apply(R) for p in self.parts.values()])

    def odot(self, y):
        assert list(self.parts) == list(y.parts)
        return sum(self.parts[mu].odot(y.parts[mu]) for mu in self.parts)

    def __add__(self, y):
        assert list(self.parts) == list(y.parts)
        return O3vec(*[O3part(self.parts[mu].as_subclass(torch.Tensor) + y.parts[mu].as_subclass(torch.Tensor), mu)
                       for mu in self.parts])

    def _product(self, y, maxl, fn):
        xp, yp = list(self.parts.values()), list(y.parts.values())
        diag = fn is O3vec_DiagCGproductFn
        tx, ty = O3type(self.tau()), O3type(y.tau())
        rmus = list((tx.DiagCGproduct(ty, maxl) if diag else tx.CGproduct(ty, maxl)).get_parts())
        out = fn.apply(len(xp), len(yp), maxl, list(self.parts), list(y.parts), *(xp + yp))
        return O3vec(*[O3part(t, mu) for t, mu in zip(out, rmus)])

    def CGproduct(self, y, maxl=-1):
        """All (l1,p1) x (l2,p2) -> (l, p1 p2) with l <= maxl, blocks in the reference's order."""
        return self._product(y, maxl, O3vec_CGproductFn)

    def DiagCGproduct(self, y, maxl=-1):
        return self._product(y, maxl, O3vec_DiagCGproductFn)

    def __repr__(self):
        return "<GElib::O3vec of type %s [b=%d]>" % (self.tau(), self.getb())
