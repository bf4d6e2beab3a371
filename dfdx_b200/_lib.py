"""ctypes binding of libdfdx_b200.so (the C ABI in include/dfdx_b200.h).

Loading fails loudly: there is no CPU or library fallback behind this module.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libdfdx_b200.so"

# b200_dtype
F32, F64, F16, AMP_F16 = 0, 1, 2, 3
# b200_path
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2
# b200_status
OK = 0
ERR_SHAPE, ERR_STRIDE, ERR_DTYPE, ERR_NULL, ERR_WORKSPACE = -1, -2, -3, -4, -5
ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_UNSUPPORTED, ERR_NOT_CONTIGUOUS, ERR_LIMIT = -6, -7, -8, -9, -10


# b200_activation
ACT_NONE, ACT_RELU = 0, 1


class Epilogue(C.Structure):
    """`b200_epilogue`: out = activation(alpha * sum + bias[j])."""
    _fields_ = [("alpha", C.c_double), ("bias", C.c_void_p), ("activation", C.c_int)]


class Conv2DOp(C.Structure):
    """Bit-identical to dfdx's `Conv2DOp` (dfdx-core/src/tensor_ops/conv2d/mod.rs:14-29)."""
    _fields_ = [(n, C.c_size_t) for n in (
        "kernel", "stride", "padding", "dilation", "groups", "batch",
        "chan_in", "chan_out", "h_in", "h_out", "w_in", "w_out")]


class Conv1DOp(C.Structure):
    """Bit-identical to dfdx's `Conv1DOp` (dfdx-core/src/tensor_ops/conv1d/mod.rs:12-23)."""
    _fields_ = [(n, C.c_size_t) for n in (
        "kernel", "stride", "padding", "dilation", "groups", "batch", "chan_in", "chan_out", "l_in", "l_out")]


_sz, _vp, _i, _d = C.c_size_t, C.c_void_p, C.c_int, C.c_double
_szp = C.POINTER(C.c_size_t)

# name -> (restype, argtypes); every function declared in include/dfdx_b200.h.
SIGNATURES = {
    "b200_init": (_i, [_i]),
    "b200_strerror": (C.c_char_p, [_i]),
    "b200_last_cuda_error": (C.c_char_p, []),
    "b200_device_status": (_i, [_vp]),
    "b200_set_path": (_i, [_i]),
    "b200_set_tf32_split_mode": (_i, [_i]),
    "b200_set_tile_n": (_i, [_i]),
    "b200_set_mn_single_box": (_i, [_i]),
    "b200_set_cta_pair_mode": (_i, [_i]),
    "b200_set_store_mode": (_i, [_i]),
    "b200_set_conv_lowering": (_i, [_i, _sz]),
    "b200_set_split_k": (_i, [_i]),
    "b200_set_capture_split_k": (_i, [_i]),
    "b200_set_wait_limit": (_i, [C.c_longlong]),
    "b200_set_max_ctas": (_i, [_i]),
    "b200_set_tail_split": (_i, [_i]),
    "b200_selftest_bounded_wait": (_i, [C.c_longlong, C.POINTER(C.c_longlong), _vp]),
    "b200_launch_count": (C.c_uint64, []),
    "b200_tensor_launch_count": (C.c_uint64, []),
    "b200_conv_implicit_count": (C.c_uint64, []),
    "b200_gemm": (_i, [_i, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _d, _vp, _szp, _vp]),
    "b200_gemm_batch": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _d, _vp, _szp, _vp]),
    "b200_matmat_forward": (_i, [_i, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _vp]),
    "b200_matmat_backward": (_i, [_i, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp, _vp, _vp, _vp]),
    "b200_matmat_br_forward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _vp]),
    "b200_matmat_br_backward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp, _vp, _vp, _vp]),
    "b200_matmat_br_backward_overwrite": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp, _vp, _vp]),
    "b200_matmat_br_grad_rhs_f32": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp]),
    "b200_matmat_batch3_forward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _vp]),
    "b200_matmat_batch3_backward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp, _vp, _vp, _vp]),
    "b200_matmat_batch4_forward": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _vp]),
    "b200_matmat_batch4_backward": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _vp, _szp, _vp, _vp, _vp, _vp]),
    "b200_gemm_batch_fused": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, C.POINTER(Epilogue), _vp, _szp, _vp]),
    "b200_linear_forward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _i, _vp, _vp]),
    "b200_matmat_batch4_forward_scaled": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _d, _vp, _vp]),
    "b200_attention_forward": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _szp, _d, _vp, _szp, _vp, _vp]),
    "b200_layer_norm_forward": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _vp, _d, _vp, _sz, _vp, _vp]),
    "b200_layer_norm_backward": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _vp, _vp, _sz, _vp, _sz, _i, _vp, _vp, _vp]),
    "b200_layer_norm_backward_sum": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _vp]),
    "b200_add_layer_norm_forward": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _vp, C.c_double, _vp, _sz, _vp, _vp]),
    "b200_relu_backward_bias_grad": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _vp]),
    "b200_bias_grad": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _vp]),
    "b200_softmax_forward": (_i, [_i, _sz, _sz, _vp, _sz, _d, _vp, _sz, _vp]),
    "b200_softmax_backward": (_i, [_i, _sz, _sz, _vp, _sz, _vp, _sz, _d, _vp, _sz, _i, _vp]),
    "b200_attention_backward_workspace_bytes": (_sz, [_sz, _sz, _sz]),
    "b200_attention_backward": (_i, [_i, _sz, _sz, _sz, _sz, _sz, _vp, _szp, _vp, _szp, _vp, _szp, _d, _vp, _szp, _vp,
                                     _vp, _szp, _vp, _szp, _vp, _szp, _vp, _szp, _i, _vp, _sz, _vp]),
    "b200_conv2d_workspace_bytes": (_sz, [_i, C.POINTER(Conv2DOp), _i]),
    "b200_conv2d_forward": (_i, [_i, C.POINTER(Conv2DOp), _vp, _szp, _vp, _vp, _vp, _sz, _vp]),
    "b200_conv2d_backward": (_i, [_i, C.POINTER(Conv2DOp), _vp, _vp, _vp, _szp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "b200_convtrans2d_workspace_bytes": (_sz, [_i, C.POINTER(Conv2DOp), _i]),
    "b200_convtrans2d_forward": (_i, [_i, C.POINTER(Conv2DOp), _vp, _vp, _szp, _vp, _vp, _sz, _vp]),
    "b200_convtrans2d_backward": (_i, [_i, C.POINTER(Conv2DOp), _vp, _vp, _vp, _szp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "b200_conv1d_workspace_bytes": (_sz, [_i, C.POINTER(Conv1DOp), _i]),
    "b200_conv1d_forward": (_i, [_i, C.POINTER(Conv1DOp), _vp, _szp, _vp, _vp, _vp, _sz, _vp]),
    "b200_conv1d_backward": (_i, [_i, C.POINTER(Conv1DOp), _vp, _vp, _vp, _szp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "b200_conv2d_forward_noalloc": (_i, [_i, C.POINTER(Conv2DOp), _vp, _szp, _vp, _vp, _vp]),
}

# Capacity of the library-resident scratch of b200_conv2d_forward_noalloc (include/dfdx_b200.h).
CONV2D_NOALLOC_SCRATCH_BYTES = 32 << 20

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and types every entry point.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m dfdx_b200.build` "
            "(the library has no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def strides(seq):
    return (C.c_size_t * len(seq))(*[int(s) for s in seq])


class B200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.b200_strerror(status).decode()
        detail = lib.b200_last_cuda_error().decode() if status == ERR_CUDA else ""
        super().__init__(f"{where}: {msg} [{status}]" + (f" — {detail}" if detail else ""))
        self.status = status


def check(status: int, where: str) -> None:
    if status != OK:
        raise B200Error(status, where)
