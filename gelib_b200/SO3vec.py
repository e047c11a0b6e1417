"""``gelib.SO3vec`` / ``gelib.SO3vecArr`` and their autograd functions on the B200 kernels.

Mirrors python/src/gelib/SO3vec.py and python/src/gelib/SO3vecArr.py of GElib (constructors, accessors,
``CGproduct`` / ``DiagCGproduct`` with ``maxl`` truncation, ``odot``, ``apply``, ``*`` with SO3weights,
same autograd Function names).  The whole product -- every (l1,l2)->l triple -- is one kernel launch
forward and one backward instead of one launch per triple (core/Gvec.hpp:311-389).
"""
import torch

from . import backend as gb
from .gelib_common import common_batch
from .SO3part import SO3part, SO3partArr


def _vec_forward(ctx, k1, k2, maxl, args, diag, part_cls):
    ctx.k1, ctx.k2, ctx.diag = k1, k2, diag
    ctx.save_for_backward(*args)
    xs, ys = [a.detach() for a in args[0:k1]], [a.detach() for a in args[k1:k1 + k2]]
    x, y = gb.SO3vec.view(xs), gb.SO3vec.view(ys)
    b = common_batch(xs[0], ys[0])
    tau = x.get_tau().DiagCGproduct(y.get_tau(), maxl) if diag else x.get_tau().CGproduct(y.get_tau(), maxl)
    gx, gy = list(xs[0].shape[1:-2]), list(ys[0].shape[1:-2])
    if len(gx) == len(gy):  # size-1 grid dimensions of one operand are broadcast against the other's
        grid = [max(a, c) for a, c in zip(gx, gy)]
    else:
        grid = gx if len(gx) > len(gy) else gy
    rparts = [torch.empty([b] + grid + [2 * l + 1, n], dtype=torch.complex64, device=xs[0].device)
              for l, n in tau.get_parts().items()]
    r = gb.SO3vec.view(rparts)
    done = (r.addDiagCGproduct if diag else r.addCGproduct)(x, y, overwrite=True)
    if not done:  # a skipped call computes nothing: the reference's outputs are its zero-initialised tensors
        for p in rparts:
            p.zero_()
    return tuple(p.as_subclass(part_cls) for p in rparts)


def _vec_backward(ctx, gargs):
    k1, k2 = ctx.k1, ctx.k2
    saved = ctx.saved_tensors
    need = ctx.needs_input_grad[3:]
    need_x, need_y = any(need[0:k1]), any(need[k1:k1 + k2])
    # a side that needs no gradient (spherical harmonics of fixed points, say) is not computed at all
    grads = [torch.zeros_like(t) if (need_x if i < k1 else need_y) else None for i, t in enumerate(saved)]
    x, y = gb.SO3vec.view(list(saved[0:k1])), gb.SO3vec.view(list(saved[k1:k1 + k2]))
    g = gb.SO3vec.view([a.as_subclass(torch.Tensor) for a in gargs])
    if need_x and need_y:
        xg, yg = gb.SO3vec.view(grads[0:k1]), gb.SO3vec.view(grads[k1:k1 + k2])
        (gb.SO3vec.addDiagCGproduct_back01 if ctx.diag else gb.SO3vec.addCGproduct_back01)(xg, yg, g, x, y)
    elif need_x:
        xg = gb.SO3vec.view(grads[0:k1])
        (xg.addDiagCGproduct_back0 if ctx.diag else xg.addCGproduct_back0)(g, y)
    elif need_y:
        yg = gb.SO3vec.view(grads[k1:k1 + k2])
        (yg.addDiagCGproduct_back1 if ctx.diag else yg.addCGproduct_back1)(g, x)
    return tuple([None, None, None] + grads)


class _MixFn(torch.autograd.Function):
    """part @ W through gelib_SO3part_mix; gradients g @ W^H and part^H @ g (summed over all rows)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gb.mix(x, w)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        gx = gb.mix(g, w, adjoint=True) if ctx.needs_input_grad[0] else None
        gw = gb.mix_back_w(x, g, w.size(0), w.size(1)) if ctx.needs_input_grad[1] else None
        return gx, gw


def _mix(p, m):
    t = p.as_subclass(torch.Tensor) if type(p) is not torch.Tensor else p
    if gb.mix_supported(t, m):
        return _MixFn.apply(t, m)
    return torch.matmul(p, m)


class SO3vec_CGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3vec.py:233-270."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, *args):
        return _vec_forward(ctx, k1, k2, maxl, args, False, SO3part)

    @staticmethod
    def backward(ctx, *args):
        return _vec_backward(ctx, args)


class SO3vec_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3vec.py:273-309."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, *args):
        return _vec_forward(ctx, k1, k2, maxl, args, True, SO3part)

    @staticmethod
    def backward(ctx, *args):
        return _vec_backward(ctx, args)


class SO3vecArr_CGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3vecArr.py:324-361."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, *args):
        return _vec_forward(ctx, k1, k2, maxl, args, False, SO3partArr)

    @staticmethod
    def backward(ctx, *args):
        return _vec_backward(ctx, args)


class SO3vecArr_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3vecArr.py:364-401 (which drops maxl; here maxl is honoured as for SO3vec)."""

    @staticmethod
    def forward(ctx, k1, k2, maxl, *args):
        return _vec_forward(ctx, k1, k2, maxl, args, True, SO3partArr)

    @staticmethod
    def backward(ctx, *args):
        return _vec_backward(ctx, args)


class SO3vec_SpharmCGproductFn(torch.autograd.Function):
    """CGproduct(spharms(lmax_x, X), y, maxl) as one fused call per direction: the harmonics are generated inside the
    kernels and never reach memory (the first layer of a network on point clouds: SO3/SO3part.hpp:150-156, 340-397
    followed by core/Gvec.hpp:311-321).  X carries no gradient."""

    @staticmethod
    def forward(ctx, X, lmax_x, maxl, *yparts):
        ys = [a.detach() for a in yparts]
        ctx.lmax_x = lmax_x
        ctx.save_for_backward(X, *yparts)
        tx = gb.SO3type({l: 1 for l in range(lmax_x + 1)})
        y = gb.SO3vec.view(ys)
        tau = tx.CGproduct(y.get_tau(), maxl)
        rparts = [torch.empty([X.size(0), 2 * l + 1, n], dtype=torch.complex64, device=X.device)
                  for l, n in tau.get_parts().items()]
        if not gb.SO3vec.view(rparts).addCGproduct_spharm(X, lmax_x, y, overwrite=True):
            for p in rparts:
                p.zero_()
        return tuple(p.as_subclass(SO3part) for p in rparts)

    @staticmethod
    def backward(ctx, *gargs):
        X = ctx.saved_tensors[0]
        grads = [torch.zeros_like(t) for t in ctx.saved_tensors[1:]]
        g = gb.SO3vec.view([a.as_subclass(torch.Tensor).contiguous() for a in gargs])
        gb.SO3vec.view(grads).addCGproduct_spharm_back1(g, X, ctx.lmax_x)
        return tuple([None, None, None] + grads)


class _VecBase:
    """What SO3vec and SO3vecArr share: a dict l -> part tensor."""
    _part = SO3part
    _cg_fn = SO3vec_CGproductFn
    _diag_fn = SO3vec_DiagCGproductFn

    def __init__(self, *args):
        self.parts = {}
        for x in args:
            assert isinstance(x, torch.Tensor)
            self.parts[(x.size(-2) - 1) // 2] = x

    @classmethod
    def zeros_like(cls, x):
        R = cls()
        for l, p in x.parts.items():
            R.parts[l] = cls._part(torch.zeros_like(p))
        return R

    @classmethod
    def randn_like(cls, x):
        R = cls()
        for l, p in x.parts.items():
            R.parts[l] = cls._part(torch.randn_like(p))
        return R

    def backend(self):
        return gb.SO3vec.view(self.parts)

    def getb(self):
        return self.parts[min(self.parts)].size(0)

    def tau(self):
        return {l: p.size(-1) for l, p in self.parts.items()}

    get_type = tau

    def l_max(self):
        return max(self.parts)

    def requires_grad_(self):
        for p in self.parts.values():
            p.requires_grad_()

    def get_grad(self):
        return type(self)(*[p.grad for p in self.parts.values()])

    def apply(self, R):
        r = type(self)()
        for l, p in self.parts.items():
            r.parts[l] = self._part(p).apply(R)
        return r

    def odot(self, y):
        assert list(self.parts.keys()) == list(y.parts.keys())
        return sum(self._part(self.parts[l]).odot(y.parts[l]) for l in self.parts)

    def __add__(self, y):
        assert list(self.parts.keys()) == list(y.parts.keys())
        return type(self)(*[self.parts[l] + y.parts[l] for l in self.parts])

    def __mul__(self, w):
        """Channel mixing with SO3weights: part l times the l-th weight matrix (python/src/gelib/SO3vec.py:174-177).
        On a CUDA device with at most 64 channels the memory-bound mixing kernels do it, otherwise torch.matmul."""
        return type(self)(*[_mix(p, m) for p, m in zip(self.parts.values(), w.parts)])

    def to(self, device):
        return type(self)(*[p.to(device) for p in self.parts.values()])

    def CGproduct(self, y, maxl=-1):
        """Full Clebsch-Gordan product: all (l1,l2)->l with l <= maxl, blocks ordered by (l1, l2)."""
        xp, yp = list(self.parts.values()), list(y.parts.values())
        return type(self)(*self._cg_fn.apply(len(xp), len(yp), maxl, *(xp + yp)))

    def DiagCGproduct(self, y, maxl=-1):
        xp, yp = list(self.parts.values()), list(y.parts.values())
        return type(self)(*self._diag_fn.apply(len(xp), len(yp), maxl, *(xp + yp)))

    def __repr__(self):
        return "<GElib::%s of type %s [b=%d]>" % (type(self).__name__, self.tau(), self.getb())

    def __str__(self):
        return "\n".join("Part l=%d:\n%s\n" % (l, p.as_subclass(torch.Tensor)) for l, p in self.parts.items())


class SO3vec(_VecBase):
    """An SO(3)-covariant vector: a sequence of SO3parts keyed by l."""

    @classmethod
    def zeros(cls, b, tau, device='cpu'):
        R = SO3vec()
        for l, n in tau.items():
            R.parts[l] = SO3part.zeros(b, l, n, device=device)
        return R

    @classmethod
    def randn(cls, b, tau, device='cpu'):
        R = SO3vec()
        for l, n in tau.items():
            R.parts[l] = SO3part.randn(b, l, n, device=device)
        return R

    @classmethod
    def Fzeros(cls, b, maxl, device='cpu'):
        return SO3vec(*[SO3part.Fzeros(b, l, device) for l in range(maxl + 1)])

    @classmethod
    def Frandn(cls, b, maxl, device='cpu'):
        return SO3vec(*[SO3part.Frandn(b, l, device) for l in range(maxl + 1)])

    @classmethod
    def spharm(cls, l, X):
        """The SO3vec whose only part is Y_l(X), X (b, 3, n) float32."""
        assert X.dim() == 3
        return SO3vec(SO3part.spharm(l, X))

    @classmethod
    def spharm_CGproduct(cls, lmax_x, X, y, maxl=-1):
        """CGproduct(SO3vec.spharms(lmax_x, X), y, maxl) without materialising the harmonics; X (b, 3, 1) float32."""
        assert X.dim() == 3 and X.size(1) == 3 and X.size(2) == 1
        return SO3vec(*SO3vec_SpharmCGproductFn.apply(X, lmax_x, maxl, *list(y.parts.values())))

    @classmethod
    def spharms(cls, maxl, X):
        """Parts l = 0..maxl of the spherical harmonics of X from one pass over the points."""
        assert X.dim() == 3
        parts = [torch.empty([X.size(0), 2 * l + 1, X.size(2)], dtype=torch.complex64, device=X.device)
                 for l in range(maxl + 1)]
        gb.SO3vec.view(parts).add_spharm(X, overwrite=True)
        return SO3vec(*[SO3part(p) for p in parts])


class SO3vecArr(_VecBase):
    """An array of SO3vecs: parts are (b, a1..ak, 2l+1, n)."""
    _part = SO3partArr
    _cg_fn = SO3vecArr_CGproductFn
    _diag_fn = SO3vecArr_DiagCGproductFn

    @classmethod
    def zeros(cls, b, adims, tau, device='cpu'):
        return SO3vecArr(*[SO3partArr.zeros(b, adims, l, n, device) for l, n in tau.items()])

    @classmethod
    def ones(cls, b, adims, tau, device='cpu'):
        return SO3vecArr(*[SO3partArr.ones(b, adims, l, n, device) for l, n in tau.items()])

    @classmethod
    def randn(cls, b, adims, tau, device='cpu'):
        return SO3vecArr(*[SO3partArr.randn(b, adims, l, n, device) for l, n in tau.items()])

    @classmethod
    def spharm(cls, l, X):
        return SO3vecArr(SO3partArr.spharm(l, X))

    def get_adims(self):
        p = self.parts[min(self.parts)]
        return list(p.size()[1:p.dim() - 2])

    def gather(self, gmap, dim=0):
        """python/src/gelib/SO3vecArr.py:230-234: every part is gathered with the same map."""
        return SO3vecArr(*[SO3partArr(p).gather(gmap, dim) for p in self.parts.values()])


def MakeZeroSO3parts(b, tau, device):
    """python/src/gelib/SO3vec.py:531-536."""
    return [SO3part.zeros(b, l, n, device) for l, n in tau.items()]


def MakeZeroSO3partArrs(b, adims, tau, device):
    """python/src/gelib/SO3vecArr.py:584-588."""
    return [SO3partArr.zeros(b, adims, l, n, device) for l, n in tau.items()]
