"""``gelib_base`` for GElib's own Python package, on the B200 kernels.

GElib's Python sources (python/src/gelib/*.py) reach the compiled library through one module, ``gelib_base`` (built from
python/bindings/GElib_py.cpp:16-40).  This module offers the names those sources use, backed by ``gelib_b200.backend``
(ctypes over libgelib_b200.so), so that with this directory and GElib's ``python/src`` on ``sys.path`` the unmodified
``import gelib`` runs its Clebsch-Gordan products, spherical harmonics and gathers on the kernels of this repository.
Tensors must live on a CUDA device: there is no CPU path behind these calls.
"""
from gelib_b200.backend import (CGproduct, O3element, O3irrep, O3part, O3type, SO3CGmatrix, SO3element, SO3irrep, SO3part,  # noqa: F401
                                SO3type, SO3vec, gather_map)

O3vec = SO3vec  # O3vec.view(parts): the same zero-copy view (the parity lives in the Python layer)
