"""gelib_b200: GElib's Clebsch-Gordan hot path on B200 (sm_100a).

Drop-in for the ``gelib`` Python package on that path: ``SO3part`` / ``SO3vec`` (and the ``Arr``
variants) with ``CGproduct``, ``DiagCGproduct``, ``spharm`` and autograd; ``gelib_b200.backend`` stands
in for the pybind11 module ``gelib_base``.  All products run in hand-written CUDA kernels behind the
C ABI of ``include/gelib_b200.h``; tensors must live on a CUDA device.
"""
from . import backend
from .backend import SO3CGmatrix, gather_map
from .gelib_common import common_batch
from .SO3element import SO3element
from .SO3irrep import SO3irrep
from .SO3type import SO3type
from .SO3part import (SO3part, SO3partArr, SO3part_CGproductFn, SO3part_DiagCGproductFn, SO3partArr_CGproductFn,
                      SO3partArr_DiagCGproductFn)
from .SO3vec import (SO3vec, SO3vecArr, SO3vec_SpharmCGproductFn, SO3vec_CGproductFn, SO3vec_DiagCGproductFn, SO3vecArr_CGproductFn,
                     SO3vecArr_DiagCGproductFn, MakeZeroSO3parts, MakeZeroSO3partArrs)
from .SO3weights import SO3weights, SO3linear
from .O3 import (O3element, O3irrep, O3type, O3part, O3vec, O3part_CGproductFn, O3part_DiagCGproductFn, O3vec_CGproductFn,
                 O3vec_DiagCGproductFn)


def CGproduct(x, y, maxl=-1):
    """``gelib.CGproduct`` (python/src/gelib/__init__.py:56-57): for parts the third argument is l."""
    return x.CGproduct(y, maxl)


def gather(x, gmap, dim=0):
    """``gelib.gather`` (python/src/gelib/__init__.py:65-66)."""
    return x.gather(gmap, dim)


def DiagCGproduct(x, y, maxl=-1):
    """``gelib.DiagCGproduct`` (python/src/gelib/__init__.py:59-60)."""
    return x.DiagCGproduct(y, maxl)
