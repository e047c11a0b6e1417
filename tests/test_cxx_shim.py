"""The C++ binding a GElib maintainer adds (include/SO3part_b200.cpp, which replaces four files of GElib's cuda/).

The file is compiled as it is with g++ against include/gelib_b200.h and a stand-in for the two cnine / GElib types it
touches (tests/cxx/SO3part.hpp), linked with the library, and driven through the four reference signatures
(SO3/SO3part.hpp:33-39 of GElib): forward, back0, back1, spherical harmonics.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from util import crandn, frandn, np_c, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CXX = os.path.join(ROOT, "tests", "cxx")
OUT = os.path.join(CXX, "build")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_shim():
    from gelib_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(ROOT, "include", "SO3part_b200.cpp")
    so = os.path.join(OUT, "libgelib_shim.so")
    libdir = os.path.dirname(_lib.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-I", CXX, "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA, "include"), src, os.path.join(CXX, "shim_driver.cpp"), "-o", so,
           "-L", libdir, "-lgelib_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return so


def test_binding_listing_compiles_and_links():
    so = build_shim()
    syms = subprocess.run(["nm", "-D", "--defined-only", so], capture_output=True, text=True).stdout
    for name in ("SO3part_addCGproduct_cu", "SO3part_addCGproduct_back0_cu", "SO3part_addCGproduct_back1_cu",
                 "addSPharm_cu", "SO3part_addDiagCGproduct_cu", "shim_product", "shim_spharm"):
        assert name in syms, name


@pytest.mark.gpu
def test_binding_runs_the_four_reference_signatures(oracle):
    assert torch.cuda.is_available()
    L = ctypes.CDLL(build_shim())
    I, P = ctypes.c_int, ctypes.c_void_p
    L.shim_product.argtypes = [I, P, P, P] + [I] * 8
    L.shim_spharm.argtypes = [P, P, I, I, I]
    B, l1, l2, l, n1, n2 = 5, 2, 3, 4, 32, 32
    x, y, g = crandn(1, B, 2 * l1 + 1, n1), crandn(2, B, 2 * l2 + 1, n2), crandn(3, B, 2 * l + 1, n1 * n2 + 6)
    xd, yd, gd = x.cuda(), y.cuda(), g.cuda()
    offs = 6
    r = torch.zeros(B, 2 * l + 1, n1 * n2 + offs, dtype=torch.complex64, device="cuda")
    assert L.shim_product(0, r.data_ptr(), xd.data_ptr(), yd.data_ptr(), B, l, n1 * n2 + offs, l1, n1, l2, n2, offs) == 0
    want = np.zeros(r.shape, np.complex64)
    oracle.add_CGproduct(want, np_c(x), np_c(y), offs=offs)
    assert rel_err(r, want) < 1e-5
    xg, yg = torch.zeros_like(xd), torch.zeros_like(yd)
    assert L.shim_product(1, xg.data_ptr(), gd.data_ptr(), yd.data_ptr(), B, l1, n1, l, n1 * n2 + offs, l2, n2, offs) == 0
    assert L.shim_product(2, yg.data_ptr(), gd.data_ptr(), xd.data_ptr(), B, l2, n2, l, n1 * n2 + offs, l1, n1, offs) == 0
    xg_w, yg_w = np.zeros(x.shape, np.complex64), np.zeros(y.shape, np.complex64)
    oracle.add_CGproduct_back0(xg_w, np_c(g), np_c(y), offs=offs)
    oracle.add_CGproduct_back1(yg_w, np_c(g), np_c(x), offs=offs)
    assert rel_err(xg, xg_w) < 1e-4 and rel_err(yg, yg_w) < 1e-4
    X = frandn(4, 9, 3, 2)
    s = torch.zeros(9, 7, 2, dtype=torch.complex64, device="cuda")
    Xd = X.cuda()
    assert L.shim_spharm(s.data_ptr(), Xd.data_ptr(), 9, 3, 2) == 0
    ws = np.zeros((9, 7, 2), np.complex64)
    oracle.add_spharm(ws, np_c(X))
    assert rel_err(s, ws) < 2e-6
    # what the reference GELIB_SKIPs is printed and skipped, not thrown: l = 7 is not in 2 x 3
    bad = torch.zeros(B, 15, n1 * n2, dtype=torch.complex64, device="cuda")
    assert L.shim_product(0, bad.data_ptr(), xd.data_ptr(), yd.data_ptr(), B, 7, n1 * n2, l1, n1, l2, n2, 0) == 0
    assert float(bad.abs().max()) == 0.0
