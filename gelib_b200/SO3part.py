"""``gelib.SO3part`` / ``gelib.SO3partArr`` and their autograd functions on the B200 kernels.

Mirrors python/src/gelib/SO3part.py and python/src/gelib/SO3partArr.py of GElib: same constructors,
accessors, ``CGproduct`` / ``DiagCGproduct`` / ``spharm`` / ``apply`` / ``odot`` and the same
``torch.autograd.Function`` names.  Differences in how the work is done, not in what is returned:
the forward output is allocated uninitialised and written once (no zero fill, no read-modify-write),
and the backward pass reads the upstream gradient once for both input gradients.
"""
import torch

from . import backend as gb
from .gelib_common import common_batch
from .SO3element import SO3element
from .SO3irrep import SO3irrep


class _ApplyFn(torch.autograd.Function):
    """x -> D x on the device (gelib_SO3part_apply); the gradient is D^H g."""

    @staticmethod
    def forward(ctx, x, D):
        ctx.save_for_backward(D)
        xd = x.detach().as_subclass(torch.Tensor)
        r = torch.empty_like(xd)
        gb.SO3part.view(r).add_apply(gb.SO3part.view(xd), D, overwrite=True)
        return r

    @staticmethod
    def backward(ctx, g):
        (D,) = ctx.saved_tensors
        gd = g.as_subclass(torch.Tensor).contiguous()
        xg = torch.empty_like(gd)
        gb.SO3part.view(xg).add_apply(gb.SO3part.view(gd), D.conj().t().contiguous(), overwrite=True)
        return xg, None


def _apply_rotation(t, R, cls):
    assert isinstance(R, SO3element)
    l = (t.size(-2) - 1) // 2
    D = SO3irrep(l).matrix(R).to(t.device)
    if not t.is_cuda:  # host helper for tests on CPU tensors, as in the reference (python/src/gelib/SO3part.py:132-135)
        return cls(torch.matmul(D, t))
    return cls(_ApplyFn.apply(t, D))


class SO3partArr_GatherFn(torch.autograd.Function):
    """python/src/gelib/SO3partArr.py:240-256."""

    @staticmethod
    def forward(ctx, x, gmap, d):
        ctx.gmap, ctx.d = gmap, d
        ctx.xshape = list(x.shape)
        shape = list(x.shape)
        shape[d + 1] = gmap.d_out()
        r = torch.zeros(shape, dtype=torch.complex64, device=x.device)
        gb.SO3part.view(r).add_gather(x.detach().as_subclass(torch.Tensor).contiguous(), gmap, d)
        return r.as_subclass(SO3partArr)

    @staticmethod
    def backward(ctx, rg):
        xg = torch.zeros(ctx.xshape, dtype=torch.complex64, device=rg.device)
        gb.SO3part.view(xg).add_gather_back(rg.as_subclass(torch.Tensor).contiguous(), ctx.gmap, ctx.d)
        return xg, None, None


def _odot(x, y):
    return torch.sum(torch.mul(torch.view_as_real(x), torch.view_as_real(y))).as_subclass(torch.Tensor)


def _product_forward(ctx, x, y, l, diag):
    ctx.l = l
    ctx.diag = diag
    ctx.save_for_backward(x, y)
    b = common_batch(x, y)
    if diag:
        assert x.size(-1) == y.size(-1)
    n = x.size(-1) if diag else x.size(-1) * y.size(-1)
    gx, gy = list(x.shape[1:-2]), list(y.shape[1:-2])
    if len(gx) == len(gy):  # size-1 grid dimensions of one operand are broadcast against the other's
        grid = [max(a, c) for a, c in zip(gx, gy)]
    else:
        grid = gx if len(gx) > len(gy) else gy
    r = torch.empty([b] + grid + [2 * l + 1, n], dtype=torch.complex64, device=x.device)
    xb, yb, rb = gb.SO3part.view(x.detach()), gb.SO3part.view(y.detach()), gb.SO3part.view(r)
    done = (rb.add_DiagCGproduct if diag else rb.add_CGproduct)(xb, yb, overwrite=True)
    if not done:  # a skipped call computes nothing: the reference's output is its zero-initialised tensor
        r.zero_()
    return r


def _product_backward(ctx, g):
    x, y = ctx.saved_tensors
    need_x, need_y = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    xg = torch.zeros_like(x) if need_x else None
    yg = torch.zeros_like(y) if need_y else None
    gv, xv, yv = gb.SO3part.view(g), gb.SO3part.view(x), gb.SO3part.view(y)
    if need_x and need_y:
        f = gb.SO3part.add_DiagCGproduct_back01 if ctx.diag else gb.SO3part.add_CGproduct_back01
        f(gb.SO3part.view(xg), gb.SO3part.view(yg), gv, xv, yv)
    elif need_x:
        v = gb.SO3part.view(xg)
        (v.add_DiagCGproduct_back0 if ctx.diag else v.add_CGproduct_back0)(gv, yv)
    elif need_y:
        v = gb.SO3part.view(yg)
        (v.add_DiagCGproduct_back1 if ctx.diag else v.add_CGproduct_back1)(gv, xv)
    return xg, yg, None


class SO3part_CGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3part.py:175-196."""

    @staticmethod
    def forward(ctx, x, y, l):
        return _product_forward(ctx, x, y, l, False).as_subclass(SO3part)

    @staticmethod
    def backward(ctx, g):
        return _product_backward(ctx, g)


class SO3part_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3part.py:199-220."""

    @staticmethod
    def forward(ctx, x, y, l):
        return _product_forward(ctx, x, y, l, True).as_subclass(SO3part)

    @staticmethod
    def backward(ctx, g):
        return _product_backward(ctx, g)


class SO3partArr_CGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3partArr.py:187-209."""

    @staticmethod
    def forward(ctx, x, y, l):
        return _product_forward(ctx, x, y, l, False).as_subclass(SO3partArr)

    @staticmethod
    def backward(ctx, g):
        return _product_backward(ctx, g)


class SO3partArr_DiagCGproductFn(torch.autograd.Function):
    """python/src/gelib/SO3partArr.py:212-234."""

    @staticmethod
    def forward(ctx, x, y, l):
        return _product_forward(ctx, x, y, l, True).as_subclass(SO3partArr)

    @staticmethod
    def backward(ctx, g):
        return _product_backward(ctx, g)


class SO3part(torch.Tensor):
    """n vectors per batch element transforming under the l-th irrep of SO(3): a complex64 tensor
    (batch, 2l+1, n); index 1 is m = -l..l."""

    @staticmethod
    def __new__(cls, t):
        return t.as_subclass(cls)

    def __init__(self, t):
        pass

    # ---- constructors ------------------------------------------------------------------------------

    @classmethod
    def zeros(cls, b, l, n, device='cpu'):
        return SO3part(torch.zeros([b, 2 * l + 1, n], dtype=torch.complex64, device=device))

    @classmethod
    def randn(cls, b, l, n, device='cpu'):
        return SO3part(torch.randn([b, 2 * l + 1, n], dtype=torch.complex64, device=device))

    @classmethod
    def spharm(cls, l, X):
        """Spherical harmonics Y_l of the vectors X (b, 3, n) float32 -> (b, 2l+1, n)."""
        assert X.dim() == 3
        R = torch.empty([X.size(0), 2 * l + 1, X.size(2)], dtype=torch.complex64, device=X.device)
        gb.SO3part.view(R).add_spharm(X, overwrite=True)
        return SO3part(R)

    @classmethod
    def Fzeros(cls, b, l, device='cpu'):
        return SO3part(torch.zeros([b, 2 * l + 1, 2 * l + 1], dtype=torch.complex64, device=device))

    @classmethod
    def Frandn(cls, b, l, device='cpu'):
        return SO3part(torch.randn([b, 2 * l + 1, 2 * l + 1], dtype=torch.complex64, device=device))

    def zeros_like(self, *args):
        if not args:
            return SO3part(torch.zeros_like(self))
        dims = list(self.size())
        if len(args) == 2:
            dims[-2], dims[-1] = 2 * args[0] + 1, args[1]
        else:
            dims[0], dims[-2], dims[-1] = args[0], 2 * args[1] + 1, args[2]
        return SO3part(torch.zeros(dims, dtype=torch.complex64, device=self.device))

    @classmethod
    def randn_like(cls, x):
        return SO3part(torch.randn_like(x))

    def backend(self):
        return gb.SO3part.view(self)

    # ---- access ------------------------------------------------------------------------------------

    def getb(self):
        return self.size(0)

    def getl(self):
        return (self.size(-2) - 1) // 2

    def getn(self):
        return self.size(-1)

    # ---- operations ----------------------------------------------------------------------------------

    def apply(self, R):
        return _apply_rotation(self, R, SO3part)

    def odot(self, y):
        return _odot(self, y)

    def CGproduct(self, y, l):
        """The l component of the Clebsch-Gordan product with y: channels n1*N2+n2."""
        assert isinstance(y, SO3part)
        assert isinstance(l, int)
        return SO3part_CGproductFn.apply(self, y, l)

    def DiagCGproduct(self, y, l):
        """The l component of the diagonal Clebsch-Gordan product: channel n pairs with channel n."""
        assert isinstance(y, SO3part)
        assert isinstance(l, int)
        return SO3part_DiagCGproductFn.apply(self, y, l)

    def __repr__(self):
        return "<GElib::SO3part(b=%d,l=%d,n=%d)>" % (self.getb(), self.getl(), self.getn())

    def __str__(self):
        return str(self.as_subclass(torch.Tensor))


class SO3partArr(torch.Tensor):
    """An array of SO3parts: complex64 (batch, a1, ..., ak, 2l+1, n)."""

    @staticmethod
    def __new__(cls, t):
        return t.as_subclass(cls)

    def __init__(self, t):
        pass

    @staticmethod
    def zeros(b, adims, l, n, device='cpu'):
        return SO3partArr(torch.zeros([b] + list(adims) + [2 * l + 1, n], dtype=torch.complex64, device=device))

    @staticmethod
    def ones(b, adims, l, n, device='cpu'):
        return SO3partArr(torch.ones([b] + list(adims) + [2 * l + 1, n], dtype=torch.complex64, device=device))

    @staticmethod
    def randn(b, adims, l, n, device='cpu'):
        return SO3partArr(torch.randn([b] + list(adims) + [2 * l + 1, n], dtype=torch.complex64, device=device))

    @classmethod
    def spharm(cls, l, X):
        """X: (b, a1..ak, 3, n) float32."""
        assert X.dim() >= 3
        R = torch.empty(list(X.shape[:-2]) + [2 * l + 1, X.size(-1)], dtype=torch.complex64, device=X.device)
        gb.SO3part.view(R).add_spharm(X, overwrite=True)
        return SO3partArr(R)

    @staticmethod
    def Fzeros(b, adims, l, device='cpu'):
        return SO3partArr.zeros(b, adims, l, 2 * l + 1, device)

    @staticmethod
    def Frandn(b, adims, l, device='cpu'):
        return SO3partArr.randn(b, adims, l, 2 * l + 1, device)

    def zeros_like(self, *args):
        if not args:
            return SO3partArr(torch.zeros_like(self))
        dims = list(self.size())
        dims[-2], dims[-1] = 2 * args[0] + 1, args[1]
        return SO3partArr(torch.zeros(dims, dtype=torch.complex64, device=self.device))

    @classmethod
    def randn_like(cls, x):
        return SO3partArr(torch.randn_like(x))

    def backend(self):
        return gb.SO3part.view(self)

    def getb(self):
        return self.size(0)

    def get_adims(self):
        return list(self.size()[1:self.dim() - 2])

    def get_nadims(self):
        return self.dim() - 3

    def getl(self):
        return (self.size(-2) - 1) // 2

    def getn(self):
        return self.size(-1)

    def odot(self, y):
        return _odot(self, y)

    def apply(self, R):
        return _apply_rotation(self, R, SO3partArr)

    def gather(self, gmap, dim=0):
        """Sums the cells of array dimension `dim` into new cells as the gather_map says
        (python/src/gelib/SO3partArr.py:142-146)."""
        return SO3partArr_GatherFn.apply(self, gmap, dim)

    def CGproduct(self, y, l):
        assert isinstance(y, SO3partArr)
        return SO3partArr_CGproductFn.apply(self, y, l)

    def DiagCGproduct(self, y, l):
        assert isinstance(y, SO3partArr)
        return SO3partArr_DiagCGproductFn.apply(self, y, l)

    def __repr__(self):
        return "<GElib::SO3partArr(b=%d,adims=%s,l=%d,n=%d)>" % (self.getb(), self.get_adims(), self.getl(), self.getn())

    def __str__(self):
        return str(self.as_subclass(torch.Tensor))
