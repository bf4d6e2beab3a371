"""The C-ABI library loads without a GPU, exports every symbol include/dfdx_b200.h declares, and
rejects malformed calls before touching a device (the reference's pre-launch panics)."""
import ctypes as C
import re
from pathlib import Path

import pytest

from dfdx_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "dfdx_b200.h"


@pytest.fixture(scope="module")
def lib():
    from dfdx_b200 import build
    build.build()
    return _lib.load()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"


def test_strerror(lib):
    assert lib.b200_strerror(0) == b"ok"
    for code in range(-10, 0):
        assert lib.b200_strerror(code) not in (b"", b"unknown status")
    assert lib.b200_strerror(-99) == b"unknown status"


def _gemm(lib, dtype, ls, rs, os_, beta=0.0, ptr=0x1000):
    return lib.b200_gemm(dtype, 4, 3, 2, ptr, _lib.strides(ls), ptr, _lib.strides(rs), beta, ptr,
                         _lib.strides(os_), None)


def test_gemm_validation_before_launch(lib):
    # matmul/mod.rs:323 "At least a single stride must be 1 for cublas"
    assert _gemm(lib, _lib.F32, [2, 3], [2, 1], [2, 1]) == _lib.ERR_STRIDE
    assert _gemm(lib, _lib.F32, [3, 1], [5, 7], [2, 1]) == _lib.ERR_STRIDE
    assert _gemm(lib, _lib.F32, [3, 1], [2, 1], [0, 3]) == _lib.ERR_STRIDE
    assert _gemm(lib, 17, [3, 1], [2, 1], [2, 1]) == _lib.ERR_DTYPE
    assert _gemm(lib, _lib.F32, [3, 1], [2, 1], [2, 1], beta=0.5) == _lib.ERR_UNSUPPORTED
    assert _gemm(lib, _lib.F32, [3, 1], [2, 1], [2, 1], ptr=None) == _lib.ERR_NULL


def test_gemm_batch_validation(lib):
    p = 0x1000
    # assert_ne!(out_strides[0], 0), cuda_kernel.rs:208
    rc = lib.b200_gemm_batch(_lib.F32, 2, 4, 3, 2, p, _lib.strides([12, 3, 1]), p, _lib.strides([0, 2, 1]), 0.0, p,
                             _lib.strides([0, 2, 1]), None)
    assert rc == _lib.ERR_STRIDE
    # MatMatBatch3 / Batch4 assert non-zero operand batch strides (cuda_kernel.rs:400-401, :474-477)
    rc = lib.b200_matmat_batch3_forward(_lib.F32, 2, 4, 3, 2, p, _lib.strides([0, 3, 1]), p,
                                        _lib.strides([6, 2, 1]), p, None)
    assert rc == _lib.ERR_STRIDE
    rc = lib.b200_matmat_batch4_forward(_lib.F32, 2, 2, 4, 3, 2, p, _lib.strides([24, 12, 3, 1]), p,
                                        _lib.strides([12, 0, 2, 1]), p, None)
    assert rc == _lib.ERR_STRIDE


def test_conv2d_workspace_and_validation(lib):
    op = _lib.Conv2DOp(kernel=3, stride=1, padding=1, dilation=1, groups=1, batch=32, chan_in=64, chan_out=128,
                       h_in=56, h_out=56, w_in=56, w_out=56)
    fwd = lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 0)
    assert fwd == 32 * 64 * 9 * 56 * 56 * 4          # the (B, C, K, K, OH, OW) patch buffer
    bwd = lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 1)
    assert bwd >= 32 * 128 * 9 * 56 * 56 * 4 + (1 + 32) * 128 * 64 * 9 * 4
    p = 0x1000
    rc = lib.b200_conv2d_forward(_lib.F32, C.byref(op), p, _lib.strides([1, 1, 1, 1]), p, p, p, fwd - 1, None)
    assert rc == _lib.ERR_WORKSPACE
    bad = _lib.Conv2DOp(kernel=3, stride=1, padding=1, dilation=1, groups=3, batch=1, chan_in=4, chan_out=6,
                        h_in=5, h_out=5, w_in=5, w_out=5)
    assert lib.b200_conv2d_forward(_lib.F32, C.byref(bad), p, _lib.strides([1, 1, 1, 1]), p, p, p, 1 << 20,
                                   None) == _lib.ERR_SHAPE
    assert lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(bad), 0) == 0


def test_conv2d_op_layout():
    # 12 x usize, #[repr(C)] (conv2d/mod.rs:14-29)
    assert C.sizeof(_lib.Conv2DOp) == 12 * C.sizeof(C.c_size_t)
    assert [f[0] for f in _lib.Conv2DOp._fields_] == [
        "kernel", "stride", "padding", "dilation", "groups", "batch", "chan_in", "chan_out", "h_in", "h_out",
        "w_in", "w_out"]


def test_path_selector_and_counters(lib):
    assert lib.b200_set_path(_lib.PATH_SIMT) == 0
    assert lib.b200_set_path(_lib.PATH_AUTO) == 0
    assert lib.b200_set_path(7) == _lib.ERR_UNSUPPORTED
    assert lib.b200_launch_count() >= lib.b200_tensor_launch_count()


def test_conv_workspace_overflow_is_reported(lib):
    # extents whose product wraps a size_t: SIZE_MAX from the size query, ERR_LIMIT from the entry points
    big = 1 << 31
    op = _lib.Conv2DOp(kernel=3, stride=1, padding=1, dilation=1, groups=1, batch=big, chan_in=big, chan_out=1,
                       h_in=4, h_out=4, w_in=4, w_out=4)
    size_max = (1 << (8 * C.sizeof(C.c_size_t))) - 1
    assert lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 0) == size_max
    assert lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 1) == size_max
    p = 0x1000
    one = _lib.strides([1, 1, 1, 1])
    assert lib.b200_conv2d_forward(_lib.F32, C.byref(op), p, one, p, p, p, size_max, None) == _lib.ERR_LIMIT
    assert lib.b200_conv2d_forward_noalloc(_lib.F32, C.byref(op), p, one, p, p, None) == _lib.ERR_LIMIT
    assert lib.b200_conv2d_backward(_lib.F32, C.byref(op), p, p, p, one, p, p, p, size_max, None, None) == _lib.ERR_LIMIT


def test_testing_hooks_reject_unknown_modes(lib):
    # the f32 operand-split hook has two modes, both correct; nothing else is accepted
    for mode in range(2, 16):
        assert lib.b200_set_tf32_split_mode(mode) == _lib.ERR_UNSUPPORTED
    assert lib.b200_set_tf32_split_mode(-1) == _lib.ERR_UNSUPPORTED
    assert lib.b200_set_tf32_split_mode(0) == 0
    assert lib.b200_set_tf32_split_mode(1) == 0
    assert lib.b200_set_capture_split_k(1) == 0
    assert lib.b200_set_capture_split_k(0) == 0
