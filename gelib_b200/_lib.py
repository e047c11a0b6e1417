"""ctypes binding of ``libgelib_b200.so`` (declared in ``include/gelib_b200.h``).

Torch is used only to own device memory and to supply the current stream; what crosses into
the library are raw pointers, sizes and strides.  There is no CPU or pure-PyTorch fallback: if
the shared library is missing, importing a product fails with instructions to build it, and a
product on CPU tensors raises.
"""
import ctypes
import os
import sys

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgelib_b200.so")

GELIB_OK, GELIB_SKIPPED, GELIB_INVALID, GELIB_CUDA_ERROR = 0, 1, 2, 3
GELIB_OVERWRITE = 1
GELIB_FP64 = 2
GELIB_MAX_PARTS = 16


class Tensor5(ctypes.Structure):
    """``gelib_tensor5``: 5-D canonical view (batch, grid0, grid1, 2l+1, channels), strides in floats."""
    _fields_ = [("base", ctypes.c_void_p), ("dims", ctypes.c_int32 * 5), ("strides", ctypes.c_int64 * 5)]


_P5 = ctypes.POINTER(Tensor5)
_lib = None

# name -> (restype, argtypes); every symbol include/gelib_b200.h declares
_PART3 = [_P5, _P5, _P5, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
_PART5 = [_P5, _P5, _P5, _P5, _P5, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
_VEC3 = [ctypes.c_int, _P5, ctypes.c_int, _P5, ctypes.c_int, _P5, ctypes.c_int, ctypes.c_void_p]
_VEC5 = [ctypes.c_int, _P5, ctypes.c_int, _P5, ctypes.c_int, _P5, _P5, _P5, ctypes.c_int, ctypes.c_void_p]
_IP = ctypes.POINTER(ctypes.c_int)
SYMBOLS = {
    "gelib_version": (ctypes.c_char_p, []),
    "gelib_last_error": (ctypes.c_char_p, []),
    "gelib_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "gelib_CGcoefficient": (ctypes.c_double, [ctypes.c_int] * 5),
    "gelib_CGmatrix": (ctypes.c_int, [ctypes.c_int] * 3 + [ctypes.c_void_p]),
    "gelib_SO3type_CGproduct": (ctypes.c_int, [ctypes.c_int, _IP, _IP, ctypes.c_int, _IP, _IP, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_int, _IP, _IP]),
    "gelib_SO3vec_CGproduct_schedule": (ctypes.c_int, [ctypes.c_int, _IP, _IP, ctypes.c_int, _IP, _IP, ctypes.c_int,
                                                       _IP, ctypes.c_int, ctypes.c_int, _IP]),
    "gelib_SO3part_addCGproduct": (ctypes.c_int, _PART3),
    "gelib_SO3part_addCGproduct_back0": (ctypes.c_int, _PART3),
    "gelib_SO3part_addCGproduct_back1": (ctypes.c_int, _PART3),
    "gelib_SO3part_addCGproduct_back01": (ctypes.c_int, _PART5),
    "gelib_SO3part_addDiagCGproduct": (ctypes.c_int, _PART3),
    "gelib_SO3part_addDiagCGproduct_back0": (ctypes.c_int, _PART3),
    "gelib_SO3part_addDiagCGproduct_back1": (ctypes.c_int, _PART3),
    "gelib_SO3part_addDiagCGproduct_back01": (ctypes.c_int, _PART5),
    "gelib_SO3part_addSPharm": (ctypes.c_int, [_P5, _P5, ctypes.c_int, ctypes.c_void_p]),
    "gelib_SO3vec_addCGproduct": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addCGproduct_static": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addCGproduct_back0": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addCGproduct_back1": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addCGproduct_back01": (ctypes.c_int, _VEC5),
    "gelib_SO3vec_addDiagCGproduct": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addDiagCGproduct_back0": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addDiagCGproduct_back1": (ctypes.c_int, _VEC3),
    "gelib_SO3vec_addDiagCGproduct_back01": (ctypes.c_int, _VEC5),
    "gelib_SO3vec_addSPharm": (ctypes.c_int, [ctypes.c_int, _P5, _P5, ctypes.c_int, ctypes.c_void_p]),
    "gelib_SO3vec_addCGproduct_spharm": (ctypes.c_int, [ctypes.c_int, _P5, _P5, ctypes.c_int, ctypes.c_int, _P5, ctypes.c_int,
                                                        ctypes.c_void_p]),
    "gelib_SO3vec_addCGproduct_spharm_back1": (ctypes.c_int, [ctypes.c_int, _P5, ctypes.c_int, _P5, _P5, ctypes.c_int,
                                                              ctypes.c_int, ctypes.c_void_p]),
    "gelib_add_gather": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "gelib_SO3part_mix": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "gelib_SO3part_mix_back_w": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                                                ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "gelib_SO3irrep_matrix": (ctypes.c_int, [ctypes.c_int, ctypes.c_double, ctypes.c_double, ctypes.c_double, ctypes.c_void_p]),
    "gelib_SO3part_apply": (ctypes.c_int, [_P5, _P5, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "gelib_kernel_launch_count": (ctypes.c_longlong, []),
    "gelib_set_option": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p]),
    "gelib_async_status": (ctypes.c_int, []),
    "gelib_probe_fp32_tflops": (ctypes.c_double, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
}


def lib():
    """The loaded library.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "gelib_b200: %s not found. Build it with `python -m gelib_b200.build` (needs nvcc); "
                "there is no CPU fallback." % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def last_error():
    return lib().gelib_last_error().decode()


def set_option(name, value):
    """Pins the kernel choice ("fwd", "bwd") or a test switch ("inject_timeout"); see include/gelib_b200.h."""
    check(lib().gelib_set_option(name.encode(), str(value).encode()))


def async_status():
    """Raises if a kernel with bounded waits gave up since the last check (call after synchronising)."""
    check(lib().gelib_async_status())


def check(status):
    """Maps a status code onto the reference's behaviour: a GELIB_SKIP prints its message and the call
    returns without computing (include/GElib_base.hpp:36); everything else raises RuntimeError, as the
    reference's std::runtime_error does through pybind11."""
    if status == GELIB_OK:
        return True
    msg = last_error()
    if status == GELIB_SKIPPED:
        sys.stderr.write(msg + "\n")
        return False
    raise RuntimeError(msg)


# ---- descriptors -----------------------------------------------------------------------------------


def _fuse(dims, strides):
    """Fuses grid dimensions into one if their strides allow it (core/Gpart.hpp:462-468)."""
    dims, strides = list(dims), list(strides)
    keep = [(d, s) for d, s in zip(dims, strides) if d != 1]
    if not keep:
        return 1, 0
    for (d0, s0), (d1, s1) in zip(keep[:-1], keep[1:]):
        if s0 != s1 * d1:
            raise RuntimeError("GElib error: grid dimensions cannot be fused into the 5-D canonical form.")
    n = 1
    for d, _ in keep:
        n *= d
    return n, keep[-1][1]


def descriptor(t, real=False):
    """``gelib_tensor5`` of a torch tensor in the reference's 5-D canonical form (core/Gpart.hpp:450-469).

    Complex tensors (b, [grid...], 2l+1, n) are viewed as interleaved floats, so strides double
    (cuda/GPUtensor.hpp:31-38).  ``real=True`` is for the (b, [grid...], 3, n) float input of spharm.
    """
    if not t.is_cuda:
        raise RuntimeError("gelib_b200 computes on CUDA tensors only (this build has no CPU path); got a %s tensor"
                           % t.device.type)
    if real:
        if t.dtype != torch.float32:
            raise RuntimeError("expected a float32 tensor")
        scale = 1
    else:
        if t.dtype != torch.complex64:
            raise RuntimeError("expected a complex64 tensor (an SO3part)")
        scale = 2
    d = t.dim()
    if d < 3:
        raise RuntimeError("an SO3part has at least 3 dimensions (batch, 2l+1, channels)")
    dims, strides = list(t.shape), [s * scale for s in t.stride()]
    if d == 3:
        D = [dims[0], 1, 1, dims[1], dims[2]]
        S = [strides[0], 0, 0, strides[1], strides[2]]
    elif d == 4:
        D = [dims[0], dims[1], 1, dims[2], dims[3]]
        S = [strides[0], strides[1], 0, strides[2], strides[3]]
    elif d == 5:
        D, S = dims, strides
    else:
        g, s = _fuse(dims[1:d - 2], strides[1:d - 2])
        D = [dims[0], g, 1, dims[d - 2], dims[d - 1]]
        S = [strides[0], s, 0, strides[d - 2], strides[d - 1]]
    out = Tensor5()
    out.base = t.data_ptr()
    for i in range(5):
        out.dims[i] = D[i]
        out.strides[i] = S[i]
    return out


def descriptor_array(tensors, real=False):
    arr = (Tensor5 * max(1, len(tensors)))()
    for i, t in enumerate(tensors):
        arr[i] = descriptor(t, real)
    return arr


def device_guard(t):
    """Context manager making t's device current; raises for anything that is not a CUDA tensor."""
    if not t.is_cuda:
        raise RuntimeError("gelib_b200 computes on CUDA tensors only (this build has no CPU path); got a %s tensor"
                           % t.device.type)
    return torch.cuda.device(t.device)


def stream_of(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
