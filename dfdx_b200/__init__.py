"""dfdx_b200 — the matmul / conv2d hot path of dfdx's `Cuda` device, re-built for B200 (sm_100a).

`dfdx_b200.Cuda` is the host-side mirror of the reference device for this path; all arithmetic runs
in libdfdx_b200.so (hand-written CUDA: tcgen05 + TMA tensor-core GEMMs, exact SIMT GEMMs for odd
layouts, conv2d unfold kernels) through the C ABI declared in include/dfdx_b200.h.
"""
from . import _lib
from ._lib import (AMP_F16, F16, F32, F64, PATH_AUTO, PATH_SIMT, PATH_TENSOR, B200Error, Conv2DOp)
from .cuda import Cuda, ShapeMismatch, conv2d_out_dim

__all__ = ["Cuda", "ShapeMismatch", "conv2d_out_dim", "Conv2DOp", "B200Error", "F32", "F64", "F16", "AMP_F16",
           "PATH_AUTO", "PATH_SIMT", "PATH_TENSOR", "_lib"]
