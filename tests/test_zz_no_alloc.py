"""conv2d forward through the allocation-free entry point (`b200_conv2d_forward_noalloc`).

That entry point exists for callers that cannot get scratch memory where they run (their own arena
owns the GPU's memory, or a device-synchronising cudaMalloc is not acceptable in their loop): the patch
buffer is a fixed array inside the library.  The test calls it through the C ABI twice in a row — the
second time on a different, smaller problem, so stale contents of the shared array would show — and
compares each result with the workspace-taking entry point and with the CPU oracle; free device memory
must be the same before and after a call.  It is collected last so that a failure here cannot hide
the rest of the suite behind `-x`.
"""
import ctypes as C

import pytest
import torch

from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu


def _both(dev, oracle, x, w, dtype, **kw):
    op = dev.conv2d_op(x, w, kw.get("stride", 1), kw.get("padding", 0), kw.get("dilation", 1), kw.get("groups", 1))
    shape = (op.batch, op.chan_out, op.h_out, op.w_out)
    ref = torch.full(shape, float("nan"), dtype=dtype, device=dev.device)
    dev.conv2d_forward(op, x, w, ref)                       # existing entry point, caller-provided workspace
    got = torch.full(shape, float("nan"), dtype=dtype, device=dev.device)
    dev.synchronize()
    free_before = torch.cuda.mem_get_info(dev.device)[0]
    rc = dev.lib.b200_conv2d_forward_noalloc(dev._dtype(x), C.byref(op), x.data_ptr(), _lib.strides(x.stride()),
                                             w.data_ptr(), got.data_ptr(), dev._stream())
    assert rc == 0, dev.lib.b200_strerror(rc)
    dev.synchronize()
    assert torch.cuda.mem_get_info(dev.device)[0] == free_before, "the call changed the amount of free device memory"
    assert not torch.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= FROB_TOL[dtype]
    want, _ = oracle.conv2d(x.cpu(), w.cpu(), stride=kw.get("stride", 1), padding=kw.get("padding", 0),
                            dilation=kw.get("dilation", 1), groups=kw.get("groups", 1))
    assert oracle.rel_frobenius(got, want) <= FROB_TOL[dtype]
    return got


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_noalloc_matches_workspace_entry_point_twice(cuda_dev, oracle, dtype):
    dev = cuda_dev
    g = torch.Generator().manual_seed(77)
    # call 1: tensor-core sized problem (patch buffer 8*16*9*24*24 elements)
    x1 = (torch.randn(8, 16, 24, 24, generator=g) * 0.5).to(dtype).to(dev.device)
    w1 = (torch.randn(32, 16, 3, 3, generator=g) * 0.2).to(dtype).to(dev.device)
    _both(dev, oracle, x1, w1, dtype, stride=1, padding=1)
    # call 2, straight after: smaller, strided, padded, grouped -> different layout of the same scratch
    x2 = (torch.randn(2, 8, 10, 11, generator=g) * 0.5).to(dtype).to(dev.device)
    w2 = (torch.randn(4, 4, 3, 3, generator=g) * 0.2).to(dtype).to(dev.device)
    _both(dev, oracle, x2, w2, dtype, stride=2, padding=2, groups=2)


def test_noalloc_rejects_oversized_problem(cuda_dev):
    """Beyond the fixed capacity the call fails cleanly before any launch.  Real buffers of the stated shapes
    are passed, so a regression of the limit check shows as a wrong return code, not as a wild access."""
    dev = cuda_dev
    op = _lib.Conv2DOp(kernel=3, stride=1, padding=1, dilation=1, groups=1, batch=32, chan_in=64, chan_out=128,
                       h_in=56, h_out=56, w_in=56, w_out=56)
    assert dev.lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 0) > _lib.CONV2D_NOALLOC_SCRATCH_BYTES
    x = torch.zeros(32, 64, 56, 56, device=dev.device)
    w = torch.zeros(128, 64, 3, 3, device=dev.device)
    out = torch.zeros(32, 128, 56, 56, device=dev.device)
    before = dev.lib.b200_launch_count()
    rc = dev.lib.b200_conv2d_forward_noalloc(_lib.F32, C.byref(op), x.data_ptr(), _lib.strides(x.stride()),
                                             w.data_ptr(), out.data_ptr(), None)
    assert rc == _lib.ERR_LIMIT
    assert dev.lib.b200_launch_count() == before


def test_noalloc_rejects_wrapping_extents(cuda_dev):
    """Extents whose product wraps around a size_t must not slip under the capacity test."""
    dev = cuda_dev
    big = 1 << 31
    # batch * chan_in * 9 * h_out * w_out * 4 = 2^31 * 2^31 * 9 * 4 * ... wraps to a small number without a checked product
    op = _lib.Conv2DOp(kernel=3, stride=1, padding=1, dilation=1, groups=1, batch=big, chan_in=big, chan_out=1,
                       h_in=4, h_out=4, w_in=4, w_out=4)
    assert dev.lib.b200_conv2d_workspace_bytes(_lib.F32, C.byref(op), 0) == (1 << 64) - 1
    x = torch.zeros(64, device=dev.device)
    before = dev.lib.b200_launch_count()
    rc = dev.lib.b200_conv2d_forward_noalloc(_lib.F32, C.byref(op), x.data_ptr(), _lib.strides([1, 1, 1, 1]),
                                             x.data_ptr(), x.data_ptr(), None)
    assert rc == _lib.ERR_LIMIT
    assert dev.lib.b200_launch_count() == before
