"""GPU parity of the GEMMs with a fused epilogue (scale, bias, ReLU) against the f64 oracle, through the C ABI.

The oracle applies the reference's op sequence step by step (matmul, `* scalar`, `Bias1D`, `ReLU`);
the device applies the same work to the f32 accumulator before the single rounding, so the tolerances
of the plain GEMMs hold: relative Frobenius error <= 1e-5 (f32), <= 2e-3 (f16), 1e-12 (f64).
"""
import itertools
import math

import pytest
import torch

import dfdx_b200
from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator().manual_seed(seed)


def rand(shape, dtype, g, device):
    return torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype).to(device)


EPILOGUES = [dict(alpha=1.0, bias=True, relu=False), dict(alpha=1.0, bias=True, relu=True),
             dict(alpha=0.125, bias=False, relu=False), dict(alpha=-0.5, bias=True, relu=True),
             dict(alpha=1.0, bias=False, relu=True)]
SHAPES = [(2, 3, 128, 64, 64), (1, 2, 200, 136, 72), (1, 1, 264, 520, 296), (2, 1, 64, 72, 520)]


def run_case(dev, oracle, dtype, b0, b1, m, k, n, ep, rhs_t, seed, bcast_rhs=False):
    g = gen(seed)
    lhs = rand((b0, b1, m, k), dtype, g, dev.device)
    if rhs_t:       # rhs stored (n, k), consumed as the permuted (k, n) view, like Linear's weight
        rhs = rand((1, 1, n, k) if bcast_rhs else (b0, b1, n, k), dtype, g, dev.device).permute(0, 1, 3, 2)
    else:
        rhs = rand((1, 1, k, n) if bcast_rhs else (b0, b1, k, n), dtype, g, dev.device)
    if bcast_rhs:
        rhs = rhs.expand(b0, b1, k, n)
    bias = rand((n,), dtype, g, dev.device) if ep["bias"] else None
    out = torch.full((b0, b1, m, n), float("nan"), dtype=dtype, device=dev.device)
    dev.gemm_batch_fused(lhs, rhs, out, alpha=ep["alpha"], bias=bias, relu=ep["relu"])
    dev.synchronize()
    want = oracle.fused_matmul(lhs.cpu(), rhs.cpu(), ep["alpha"], None if bias is None else bias.cpu(), ep["relu"])
    err = oracle.rel_frobenius(out, want)
    assert err <= FROB_TOL[dtype], f"{(b0, b1, m, k, n)} {ep} rhs_t={rhs_t}: rel frobenius {err:.3e}"
    if ep["relu"]:
        assert float(out.min()) >= 0.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float64])
def test_fused_simt(cuda_dev, oracle, dtype):
    cuda_dev.set_path(dfdx_b200.PATH_SIMT)
    try:
        for i, ((b0, b1, m, k, n), ep) in enumerate(itertools.product(SHAPES[:2] + [(1, 1, 5, 3, 7)], EPILOGUES)):
            run_case(cuda_dev, oracle, dtype, b0, b1, m, k, n, ep, rhs_t=bool(i & 1), seed=500 + i)
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("store", [pytest.param(0, id="auto"), pytest.param(1, id="rowstore"), pytest.param(2, id="colstore")])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_fused_tensor_core(cuda_dev, oracle, dtype, tile_n, store):
    """tcgen05 path forced: every tile width, both store orientations (the column-store orientation indexes the
    bias by the kernel's row or column depending on which problem it transposed), ragged extents, batch
    strides incl. a broadcast rhs."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_tile_n(tile_n) == 0
    assert cuda_dev.lib.b200_set_store_mode(store) == 0
    try:
        before = cuda_dev.lib.b200_tensor_launch_count()
        cases = list(itertools.product(SHAPES, EPILOGUES))
        for i, ((b0, b1, m, k, n), ep) in enumerate(cases):
            run_case(cuda_dev, oracle, dtype, b0, b1, m, k, n, ep, rhs_t=bool(i & 1), seed=700 + i,
                     bcast_rhs=(i % 3 == 0))
        assert cuda_dev.lib.b200_tensor_launch_count() - before == len(cases)
    finally:
        cuda_dev.lib.b200_set_tile_n(0)
        cuda_dev.lib.b200_set_store_mode(0)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


def test_fused_unaligned_bias_is_served(cuda_dev, oracle):
    """A bias that is not 16-byte aligned cannot use the tensor-core epilogue's vector loads: the forced tensor
    path says so, the product path serves the call on the SIMT kernel."""
    g = gen(9)
    x = rand((1, 1, 128, 64), torch.float32, g, cuda_dev.device)
    w = rand((1, 1, 64, 128), torch.float32, g, cuda_dev.device)
    bias = rand((129,), torch.float32, g, cuda_dev.device)[1:]
    out = torch.empty(1, 1, 128, 128, device=cuda_dev.device)
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    try:
        with pytest.raises(dfdx_b200.B200Error) as e:
            cuda_dev.gemm_batch_fused(x, w, out, bias=bias)
        assert e.value.status == _lib.ERR_UNSUPPORTED
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)
    cuda_dev.gemm_batch_fused(x, w, out, bias=bias)
    assert oracle.rel_frobenius(out, oracle.fused_matmul(x.cpu(), w.cpu(), 1.0, bias.cpu())) <= FROB_TOL[torch.float32]


def test_fused_rejects_unknown_activation(cuda_dev):
    x = torch.zeros(1, 8, 8, device=cuda_dev.device)
    w = torch.zeros(8, 8, device=cuda_dev.device)
    out = torch.zeros(1, 8, 8, device=cuda_dev.device)
    rc = cuda_dev.lib.b200_linear_forward(_lib.F32, 1, 8, 8, 8, x.data_ptr(), _lib.strides(x.stride()), w.data_ptr(),
                                          _lib.strides(w.stride()), None, 7, out.data_ptr(), None)
    assert rc == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_linear_forward_encoder_shapes(cuda_dev, oracle, dtype):
    """`Linear` (+ReLU) of the Transformer feed-forward block at configuration 5's widths (512 -> 2048 -> 512,
    batch 4 x seq 512): sampled output rows against the oracle, and equality with the unfused sequence."""
    g = gen(31)
    b, s, i, o = 4, 512, 512, 2048
    x = rand((b, s, i), dtype, g, cuda_dev.device)
    w = (rand((o, i), dtype, g, cuda_dev.device) / math.sqrt(i)).to(dtype)
    bias = rand((o,), dtype, g, cuda_dev.device)
    before = cuda_dev.lib.b200_tensor_launch_count()
    y = cuda_dev.linear_forward(x, w.permute(1, 0), bias, relu=True)
    assert cuda_dev.lib.b200_tensor_launch_count() - before == 1
    rows = torch.tensor([0, 1, 127, 128, 700, 1023, 2047])
    xs = x.reshape(b * s, i)[rows.to(x.device)]
    want = oracle.fused_matmul(xs.cpu(), w.permute(1, 0).cpu(), 1.0, bias.cpu(), True)
    assert oracle.rel_frobenius(y.reshape(b * s, o)[rows.to(x.device)], want) <= FROB_TOL[dtype]
    # the unfused sequence rounds after every op; the fused one once
    y_mm, _ = cuda_dev.matmul(x, w.permute(1, 0))
    unfused = torch.relu(y_mm + bias)
    assert oracle.rel_frobenius(y, unfused) <= (2e-3 if dtype == torch.float16 else 1e-6)


def test_attention_scores_scaled(cuda_dev, oracle):
    """`q.matmul(k) * 1/sqrt(d)` with MultiHeadAttention's zero-copy permuted views, f16."""
    g = gen(32)
    b, s, h, d = 2, 256, 8, 64
    q = rand((b, s, h, d), torch.float16, g, cuda_dev.device).permute(0, 2, 1, 3)
    k = rand((b, s, h, d), torch.float16, g, cuda_dev.device).permute(0, 2, 3, 1)
    got = cuda_dev.matmat_batch4_forward_scaled(q, k, 1.0 / math.sqrt(d))
    want = oracle.fused_matmul(q.cpu(), k.cpu(), 1.0 / math.sqrt(d))
    assert oracle.rel_frobenius(got, want) <= FROB_TOL[torch.float16]


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float64])
def test_matmat_br_backward_overwrite(cuda_dev, oracle, dtype):
    """The first-accumulation variant writes what the accumulating one adds into zeros; the buffers are never read
    (NaN-poisoned here); views with aliased elements are rejected."""
    g = gen(41)
    b, m, k, n = 3, 136, 72, 200
    x = rand((b, m, k), dtype, g, cuda_dev.device)
    w = rand((n, k), dtype, g, cuda_dev.device).permute(1, 0)              # (k, n) view of a stored (n, k) weight
    go = rand((b, m, n), dtype, g, cuda_dev.device)
    gx = torch.full((b * m * k,), float("nan"), dtype=dtype, device=cuda_dev.device)
    gw = torch.full((n * k,), float("nan"), dtype=dtype, device=cuda_dev.device)
    cuda_dev.matmat_br_backward_overwrite(x, gx, w, gw, go)
    _, bwd = oracle.matmul(x.cpu(), w.cpu())
    want_x, want_w = bwd(go.cpu())
    assert oracle.rel_frobenius(cuda_dev.grad_view(gx, x), want_x) <= FROB_TOL[dtype]
    assert oracle.rel_frobenius(cuda_dev.grad_view(gw, w), want_w) <= FROB_TOL[dtype]
    xb = x[:1].expand(b, m, k)                                              # broadcast lhs: its gradient is a sum
    with pytest.raises(dfdx_b200.B200Error) as e:
        cuda_dev.matmat_br_backward_overwrite(xb, gx, w, gw, go)
    assert e.value.status == _lib.ERR_STRIDE
