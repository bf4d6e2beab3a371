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
