"""GPU parity of convtrans2d (the data gradient of a conv2d, run forward) against the f64 oracle, through the C ABI.
Tolerances: relative Frobenius error <= 1e-5 (f32), <= 2e-3 (f16), 1e-12 (f64)."""
import pytest
import torch

import dfdx_b200
from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu

# (batch, chan_in, chan_out, h, w, kernel, stride, padding, dilation, groups)
CASES = [(1, 2, 3, 3, 4, 2, 1, 0, 1, 1), (2, 3, 4, 5, 5, 3, 2, 0, 1, 1), (2, 4, 6, 6, 7, 3, 1, 1, 1, 2),
         (1, 2, 2, 4, 4, 2, 1, 0, 2, 1), (3, 8, 8, 8, 8, 3, 3, 2, 1, 4), (2, 16, 8, 12, 12, 4, 2, 1, 1, 1)]


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_convtrans2d_forward_backward(cuda_dev, oracle, dtype, case):
    b, c, o, h, w_, k, stride, pad, dil, groups = case
    g = gen(sum(case))
    x = torch.randn(b, c, h, w_, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    w = (torch.randn(c, o // groups, k, k, generator=g, dtype=torch.float64) * 0.3).to(dtype).to(cuda_dev.device)
    kw = dict(stride=stride, padding=pad, dilation=dil, groups=groups)
    y, bwd = cuda_dev.convtrans2d(x, w, **kw)
    want, wbwd = oracle.convtrans2d(x.cpu(), w.cpu(), **kw)
    assert y.shape == want.shape
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[dtype]
    go = torch.randn(*y.shape, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    gx, gw = bwd(go)
    wx, ww = wbwd(go.cpu())
    assert oracle.rel_frobenius(gx, wx) <= FROB_TOL[dtype]
    assert oracle.rel_frobenius(gw, ww) <= FROB_TOL[dtype]
    assert cuda_dev.device_status() == 0


def test_batched_convtrans2d_equals_per_image(cuda_dev):
    """convtrans2d/tests.rs:280-311: stride 3, padding 2; batched output and gradients equal the per-image ones."""
    g = gen(6)
    x = torch.randn(3, 28, 28, generator=g).to(cuda_dev.device)
    w = torch.randn(3, 5, 6, 6, generator=g).to(cuda_dev.device)
    y1, bwd1 = cuda_dev.convtrans2d(x, w, stride=3, padding=2)
    xb = x.unsqueeze(0).expand(10, 3, 28, 28).contiguous()
    yb, bwdb = cuda_dev.convtrans2d(xb, w, stride=3, padding=2)
    assert yb.shape == (10, 5, 83, 83)
    for i in range(10):
        assert torch.allclose(yb[i], y1, rtol=1e-4, atol=1e-4)
    gx1, gw1 = bwd1(torch.ones_like(y1))
    gxb, gwb = bwdb(torch.ones_like(yb))
    assert torch.allclose(gwb, 10.0 * gw1, rtol=1e-3, atol=1e-2)
    for i in range(10):
        assert torch.allclose(gxb[i], gx1, rtol=1e-4, atol=1e-4)


def test_convtrans2d_errors(cuda_dev):
    lib = cuda_dev.lib
    x = torch.zeros(1, 4, 5, 5, device=cuda_dev.device)
    w = torch.zeros(4, 3, 3, 3, device=cuda_dev.device)
    op = _lib.Conv2DOp(kernel=3, stride=1, padding=0, dilation=1, groups=1, batch=1, chan_in=4, chan_out=3,
                       h_in=5, h_out=7, w_in=5, w_out=7)
    need = lib.b200_convtrans2d_workspace_bytes(_lib.F32, op, 0)
    assert need > 0
    out = torch.zeros(1, 3, 7, 7, device=cuda_dev.device)
    ws = torch.zeros(need, dtype=torch.uint8, device=cuda_dev.device)
    st = _lib.strides
    rc = lib.b200_convtrans2d_forward(_lib.F32, op, x.data_ptr(), w.data_ptr(), st(w.stride()), out.data_ptr(),
                                      ws.data_ptr(), need - 1, None)
    assert rc == _lib.ERR_WORKSPACE
    wt = w.permute(0, 1, 3, 2)                                                # filters must be dense for grad_img
    rc = lib.b200_convtrans2d_backward(_lib.F32, op, x.data_ptr(), x.data_ptr(), wt.data_ptr(), st((27, 9, 1, 3)),
                                       None, out.data_ptr(), ws.data_ptr(), need, None, None)
    assert rc == _lib.ERR_NOT_CONTIGUOUS
    with pytest.raises(dfdx_b200.ShapeMismatch):
        cuda_dev.convtrans2d(x, torch.zeros(5, 3, 3, 3, device=cuda_dev.device))
