"""catccos_b200: B200 (sm_100a) implementation of CATCCOS's MXFP8 quantise + AllGather-Matmul path.

The product is libcatccos_b200.so (hand-written CUDA kernels behind a C ABI, include/catccos_b200.h)
and the C++ operator surface under catccos_b200/host/.  This Python package is the thin harness the
tests and the benchmark use to reach the C ABI.
"""
from . import capi, workloads  # noqa: F401
