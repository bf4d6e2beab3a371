"""GPU parity of the row-wise kernels (LayerNorm forward / backward, bias gradient) against the f64 oracle, through
the C ABI.  Tolerances as for the GEMMs: relative Frobenius error <= 1e-5 (f32), <= 2e-3 (f16)."""
import pytest
import torch

import dfdx_b200
from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu

SHAPES = [(5, 3), (300, 512), (77, 520), (33, 1000), (64, 37), (4, 16, 128), (2050, 1024), (9, 2048)]


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_layer_norm_forward_backward(cuda_dev, oracle, dtype, shape):
    cols = shape[-1]
    if dtype == torch.float32 and cols > 1024:
        pytest.skip("backward limit for f32 is 1024 columns")
    g = gen(sum(shape))
    x = (torch.randn(*shape, generator=g, dtype=torch.float64) * 2 + 0.5).to(dtype).to(cuda_dev.device)
    gamma = (1 + 0.3 * torch.randn(cols, generator=g, dtype=torch.float64)).to(dtype).to(cuda_dev.device)
    beta = torch.randn(cols, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    go = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    y, stats = cuda_dev.layer_norm_forward(x, gamma, beta, 1e-5, want_stats=True)
    want, bwd = oracle.layer_norm(x, gamma, beta, 1e-5)
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[dtype]
    gg = torch.full((cols,), 1.0, dtype=torch.float32, device=cuda_dev.device)      # sums are ADDED to these
    gb = torch.full((cols,), -2.0, dtype=torch.float32, device=cuda_dev.device)
    gx = cuda_dev.layer_norm_backward(x, gamma, stats, go, gg, gb)
    wx, wg, wb = bwd(go)
    tol = FROB_TOL[dtype] * (4 if dtype == torch.float16 else 1)      # dx subtracts two row means from g * gamma
    assert oracle.rel_frobenius(gx, wx) <= tol
    assert oracle.rel_frobenius(gg - 1.0, wg) <= 1e-4
    assert oracle.rel_frobenius(gb + 2.0, wb) <= 1e-4


def test_layer_norm_limits_and_plain_normalize(cuda_dev, oracle):
    x = torch.randn(4, 4096, generator=gen(1)).half().to(cuda_dev.device)
    y, stats = cuda_dev.layer_norm_forward(x, None, None, 1e-5, want_stats=True)      # forward has no column limit
    want, _ = oracle.layer_norm(x, None, None, 1e-5)
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[torch.float16]
    with pytest.raises(dfdx_b200.B200Error) as e:
        cuda_dev.layer_norm_backward(x, None, stats, x)
    assert e.value.status == _lib.ERR_LIMIT
    x64 = torch.zeros(2, 8, dtype=torch.float64, device=cuda_dev.device)
    with pytest.raises(dfdx_b200.B200Error) as e:
        cuda_dev.layer_norm_forward(x64)
    assert e.value.status == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(7, 5), (1000, 37), (16384, 512), (3, 700, 2048), (129, 264)], ids=str)
def test_bias_grad(cuda_dev, oracle, dtype, shape):
    g = gen(sum(shape))
    go = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    out = torch.full((shape[-1],), 3.0, dtype=torch.float32, device=cuda_dev.device)
    cuda_dev.bias_grad(go, out)
    want = go.cpu().double().reshape(-1, shape[-1]).sum(0)
    assert oracle.rel_frobenius(out - 3.0, want) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(5, 3), (300, 512), (77, 520), (4, 16, 128), (2050, 256), (64, 37), (9, 2048)],
                         ids=lambda s: "x".join(map(str, s)))
def test_add_layer_norm_and_backward_with_sum(cuda_dev, oracle, dtype, shape):
    """`LayerNorm(a + b)` in one call (the sum comes back rounded as a separate add rounds it, the norm is taken of
    that rounded sum) and the backward that also returns the column sums of the grad_x it stores; shapes on both
    sides of the one-kernel path's limits."""
    dev = cuda_dev
    cols = shape[-1]
    if dtype == torch.float32 and cols > 1024:
        pytest.skip("backward limit for f32 is 1024 columns")
    g = gen(sum(shape) + 7)
    a = (torch.randn(*shape, generator=g, dtype=torch.float64) * 2 + 0.5).to(dtype).to(dev.device)
    b = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(dev.device)
    gamma = (1 + 0.3 * torch.randn(cols, generator=g, dtype=torch.float64)).to(dtype).to(dev.device)
    beta = torch.randn(cols, generator=g, dtype=torch.float64).to(dtype).to(dev.device)
    go = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(dev.device)
    y, total, stats = dev.add_layer_norm_forward(a, b, gamma, beta, 1e-5)
    want_sum = (a.cpu().double() + b.cpu().double()).to(dtype)
    assert torch.equal(total.cpu(), want_sum)                                    # one rounding, like the add op
    want, bwd = oracle.layer_norm(want_sum, gamma, beta, 1e-5)
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[dtype]
    y2, stats2 = dev.layer_norm_forward(total, gamma, beta, 1e-5, want_stats=True)
    assert torch.equal(y, y2) and torch.equal(stats, stats2)                     # same arithmetic as the two-step route
    gg = torch.full((cols,), 1.0, dtype=torch.float32, device=dev.device)
    gb = torch.full((cols,), -2.0, dtype=torch.float32, device=dev.device)
    gs = torch.full((cols,), 0.5, dtype=torch.float32, device=dev.device)
    gx = dev.layer_norm_backward_sum(total, gamma, stats, go, gg, gb, gs)
    wx, wg, wb = bwd(go)
    tol = FROB_TOL[dtype] * (4 if dtype == torch.float16 else 1)
    assert oracle.rel_frobenius(gx, wx) <= tol
    assert oracle.rel_frobenius(gg - 1.0, wg) <= 1e-4
    assert oracle.rel_frobenius(gb + 2.0, wb) <= 1e-4
    # the sums are those of the stored (rounded) gradient
    assert oracle.rel_frobenius(gs - 0.5, gx.cpu().double().reshape(-1, cols).sum(0)) <= 1e-5
    assert torch.equal(gx, dev.layer_norm_backward(total, gamma, stats, go))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(7, 5), (1000, 37), (4096, 2048), (3, 700, 520), (129, 264)], ids=str)
def test_relu_backward_bias_grad(cuda_dev, oracle, dtype, shape):
    """ReLU's backward in place plus the bias gradient: bit-exact mask (zeros where y <= 0, NaN-free), f32 sums."""
    dev = cuda_dev
    g = gen(sum(shape) + 3)
    y = torch.relu(torch.randn(*shape, generator=g, dtype=torch.float64)).to(dtype).to(dev.device)
    go = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(dev.device)
    want = torch.where(y > 0, go, torch.zeros_like(go))
    out = torch.full((shape[-1],), 3.0, dtype=torch.float32, device=dev.device)
    got = go.clone()
    dev.relu_backward_bias_grad(y, got, out)
    assert torch.equal(got, want)
    assert oracle.rel_frobenius(out - 3.0, want.cpu().double().reshape(-1, shape[-1]).sum(0)) <= 1e-5
    got2 = go.clone()
    dev.relu_backward_bias_grad(y, got2, None)                                   # mask only
    assert torch.equal(got2, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(5, 3), (300, 512), (77, 520), (33, 1000), (64, 37), (4, 16, 128), (2050, 1024),
                                   (9, 2048), (3, 5000)], ids=lambda s: "x".join(map(str, s)))
def test_softmax_forward_backward(cuda_dev, oracle, dtype, shape):
    """softmax over the last axis with the preceding scalar multiply folded in, forward and backward (written and
    accumulated), against the f64 restatement of dfdx's op sequence; rows keep their sum of 1."""
    g = gen(sum(shape) + 1)
    alpha = 0.125
    x = (torch.randn(*shape, generator=g, dtype=torch.float64) * 6).to(dtype).to(cuda_dev.device)
    go = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(cuda_dev.device)
    y = cuda_dev.softmax_forward(x, alpha)
    want, bwd = oracle.softmax(x, alpha)
    assert oracle.rel_frobenius(y, want) <= FROB_TOL[dtype]
    assert (y.double().sum(-1) - 1).abs().max().item() <= (2e-2 if dtype == torch.float16 else 1e-5)
    # the backward reads the stored (rounded) y: the oracle is given the same y
    wx = alpha * y.cpu().double() * (go.cpu().double() - (go.cpu().double() * y.cpu().double()).sum(-1, keepdim=True))
    gx = cuda_dev.softmax_backward(y, go, alpha)
    tol = FROB_TOL[dtype] * (2 if dtype == torch.float16 else 1)
    assert oracle.rel_frobenius(gx, wx) <= tol
    assert oracle.rel_frobenius(gx, bwd(go)) <= (8e-3 if dtype == torch.float16 else 1e-5)
    acc = torch.ones_like(gx)
    cuda_dev.softmax_backward(y, go, alpha, accumulate_into=acc)
    assert oracle.rel_frobenius(acc, wx + 1.0) <= tol


def test_softmax_extremes_and_strided_rows(cuda_dev, oracle):
    """Large magnitudes do not overflow (the row maximum is subtracted first), and rows may be padded views."""
    dev = cuda_dev
    x = torch.tensor([[1e4, 1e4 - 1.0, -1e4, 0.0], [-3e4, -3e4, -3e4, -3e4]], device=dev.device)
    y = dev.softmax_forward(x)
    want, _ = oracle.softmax(x)
    assert torch.isfinite(y).all()
    assert oracle.rel_frobenius(y, want) <= 1e-5
    base = torch.randn(40, 72, generator=gen(5)).to(dev.device)
    view = base[:, :65]                                           # leading dimension 72, 65 columns: element-wise path
    y = dev.softmax_forward(view)
    want, _ = oracle.softmax(view)
    assert oracle.rel_frobenius(y, want) <= 1e-5
    x64 = torch.zeros(2, 8, dtype=torch.float64, device=dev.device)
    with pytest.raises(dfdx_b200.B200Error) as e:
        dev.softmax_forward(x64)
    assert e.value.status == _lib.ERR_UNSUPPORTED
