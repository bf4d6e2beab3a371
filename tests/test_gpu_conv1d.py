"""GPU parity of conv1d (the conv2d lowering over an image of height 1) against the f64 oracle, through the C ABI.
Tolerances: relative Frobenius error <= 1e-5 (f32), <= 2e-3 (f16), 1e-12 (f64)."""
import pytest
import torch

import dfdx_b200
from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu

# (batch, chan_in, chan_out, length, kernel, stride, padding, dilation, groups)
CASES = [(1, 1, 2, 2, 2, 1, 0, 1, 1), (2, 3, 5, 28, 6, 1, 0, 1, 1), (3, 4, 6, 37, 3, 2, 1, 2, 2),
         (2, 8, 8, 64, 5, 1, 2, 1, 4), (1, 16, 24, 256, 3, 1, 1, 1, 1), (4, 32, 16, 128, 7, 3, 3, 1, 1),
         (2, 6, 6, 40, 4, 2, 0, 3, 3)]


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_conv1d_forward_backward(cuda_dev, oracle, dtype, case):
    b, c, o, l, k, stride, pad, dil, groups = case
    g = gen(sum(case))
    x = torch.randn(b, c, l, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    w = (torch.randn(o, c // groups, k, generator=g, dtype=torch.float64) * 0.3).to(dtype).to(cuda_dev.device)
    kw = dict(stride=stride, padding=pad, dilation=dil, groups=groups)
    y, bwd = cuda_dev.conv1d(x, w, **kw)
    want, wbwd = oracle.conv1d(x.cpu(), w.cpu(), **kw)
    assert y.shape == want.shape
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[dtype]
    go = torch.randn(*y.shape, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    gx, gw = bwd(go)
    wx, ww = wbwd(go.cpu())
    assert oracle.rel_frobenius(gx, wx) <= FROB_TOL[dtype]
    assert oracle.rel_frobenius(gw, ww) <= FROB_TOL[dtype]
    assert cuda_dev.device_status() == 0


def test_batched_conv1d_equals_per_image(cuda_dev):
    """conv1d/tests.rs:133-165: the batched result and gradient equal the per-image ones."""
    g = gen(5)
    x = torch.randn(3, 28, generator=g).to(cuda_dev.device)
    w = torch.randn(5, 3, 6, generator=g).to(cuda_dev.device)
    y1, bwd1 = cuda_dev.conv1d(x, w)
    xb = x.unsqueeze(0).expand(10, 3, 28).contiguous()
    yb, bwdb = cuda_dev.conv1d(xb, w)
    assert yb.shape == (10, 5, 23)
    for i in range(10):
        assert torch.allclose(yb[i], y1, rtol=1e-5, atol=1e-6)
    gx1, gw1 = bwd1(torch.ones_like(y1))
    gxb, gwb = bwdb(torch.ones_like(yb))
    assert torch.allclose(gwb, 10.0 * gw1, rtol=1e-4, atol=1e-4)
    for i in range(10):
        assert torch.allclose(gxb[i], gx1, rtol=1e-5, atol=1e-6)


def test_conv1d_errors(cuda_dev):
    lib = cuda_dev.lib
    op = _lib.Conv1DOp(kernel=3, stride=1, padding=0, dilation=1, groups=2, batch=1, chan_in=3, chan_out=4, l_in=8, l_out=6)
    assert lib.b200_conv1d_workspace_bytes(_lib.F32, op, 0) == 0            # 3 channels in 2 groups
    x = torch.zeros(1, 4, 8, device=cuda_dev.device)
    w = torch.zeros(4, 2, 3, device=cuda_dev.device)
    op = _lib.Conv1DOp(kernel=3, stride=1, padding=0, dilation=1, groups=2, batch=1, chan_in=4, chan_out=4, l_in=8, l_out=6)
    need = lib.b200_conv1d_workspace_bytes(_lib.F32, op, 0)
    assert need >= 1 * 4 * 3 * 6 * 4
    out = torch.zeros(1, 4, 6, device=cuda_dev.device)
    ws = torch.zeros(need, dtype=torch.uint8, device=cuda_dev.device)
    rc = lib.b200_conv1d_forward(_lib.F32, op, x.data_ptr(), _lib.strides(x.stride()), w.data_ptr(), out.data_ptr(),
                                 ws.data_ptr(), need - 1, None)
    assert rc == _lib.ERR_WORKSPACE
    with pytest.raises(dfdx_b200.ShapeMismatch):
        cuda_dev.conv1d(x.transpose(1, 2), w)
