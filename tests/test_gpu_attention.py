"""GPU parity of the fused attention kernel against the f64 oracle's step-by-step op sequence
(matmul, scale, softmax, matmul), through the C ABI.  Tolerance: relative Frobenius error <= 2e-3 (f16
output), log-sum-exp within 2e-3 absolute."""
import math

import pytest
import torch

import dfdx_b200
from dfdx_b200 import _lib
from helpers import FROB_TOL

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator().manual_seed(seed)


def mha_views(b, h, s1, s2, d, g, device, spread=1.0):
    """q, k, v as MultiHeadAttention builds them: (B,S,H,D) buffers viewed through permutes, no copy."""
    q = (torch.randn(b, s1, h, d, generator=g, dtype=torch.float64) * spread).half().to(device).permute(0, 2, 1, 3)
    k = (torch.randn(b, s2, h, d, generator=g, dtype=torch.float64) * spread).half().to(device).permute(0, 2, 3, 1)
    v = torch.randn(b, s2, h, d, generator=g, dtype=torch.float64).half().to(device).permute(0, 2, 1, 3)
    return q, k, v


SHAPES = [(1, 1, 128, 128, 64), (2, 3, 200, 136, 64), (1, 2, 384, 520, 32), (1, 1, 128, 256, 128),
          (2, 2, 72, 72, 16), (1, 2, 8, 1000, 64), (1, 1, 300, 8, 40), (1, 2, 130, 257, 96)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_attention_forward(cuda_dev, oracle, shape):
    b, h, s1, s2, d = shape
    q, k, v = mha_views(b, h, s1, s2, d, gen(sum(shape)), cuda_dev.device)
    alpha = 1.0 / math.sqrt(d)
    before = cuda_dev.lib.b200_tensor_launch_count()
    out, lse = cuda_dev.attention_forward(q, k, v, alpha, want_lse=True)
    cuda_dev.synchronize()
    assert cuda_dev.lib.b200_tensor_launch_count() - before == 1
    assert out.shape == (b, h, s1, d) and out.permute(0, 2, 1, 3).is_contiguous()
    want, want_lse = oracle.attention(q.cpu(), k.cpu(), v.cpu(), alpha)
    err = oracle.rel_frobenius(out, want)
    assert err <= FROB_TOL[torch.float16], f"rel frobenius {err:.3e}"
    assert float((lse.cpu().double() - want_lse).abs().max()) <= 2e-3


def test_attention_peaked_scores_and_negative_scale(cuda_dev, oracle):
    """Large score spread (the running maximum moves by hundreds between key tiles) and a negative scale."""
    q, k, v = mha_views(1, 2, 256, 640, 64, gen(5), cuda_dev.device, spread=4.0)
    for alpha in (1.0, -0.5):
        out, lse = cuda_dev.attention_forward(q, k, v, alpha, want_lse=True)
        want, want_lse = oracle.attention(q.cpu(), k.cpu(), v.cpu(), alpha)
        assert oracle.rel_frobenius(out, want) <= FROB_TOL[torch.float16]
        assert float(((lse.cpu().double() - want_lse).abs() / want_lse.abs().clamp_min(1.0)).max()) <= 2e-3
        assert bool(torch.isfinite(out).all())


def test_attention_output_layouts(cuda_dev, oracle):
    """A caller-provided contiguous (B,H,S1,D) output (what `weights.matmul(v)` allocates) gives the same values."""
    q, k, v = mha_views(2, 4, 160, 160, 64, gen(6), cuda_dev.device)
    a, _ = cuda_dev.attention_forward(q, k, v, 0.125)
    out = torch.empty(2, 4, 160, 64, dtype=torch.float16, device=cuda_dev.device)
    b_, _ = cuda_dev.attention_forward(q, k, v, 0.125, out=out)
    assert torch.equal(a.contiguous(), b_)


def test_attention_matches_unfused_sequence(cuda_dev):
    """Against this library's own unfused path (two batched GEMMs + torch softmax), configuration 3's shape."""
    q, k, v = mha_views(16, 16, 512, 512, 64, gen(7), cuda_dev.device)
    out, _ = cuda_dev.attention_forward(q, k, v, 0.125)
    scores = cuda_dev.matmat_batch4_forward_scaled(q, k, 0.125)
    ref = cuda_dev.matmat_batch4_forward(torch.softmax(scores.float(), dim=-1).half(), v)
    err = (out.float() - ref.float()).norm() / ref.float().norm()
    assert float(err) <= 2e-3


def test_attention_rejects_what_it_cannot_address(cuda_dev):
    dev = cuda_dev
    q, k, v = mha_views(1, 1, 64, 64, 64, gen(8), dev.device)
    with pytest.raises(dfdx_b200.B200Error) as e:                     # unit stride must be along D
        dev.attention_forward(q.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2), k, v, 1.0)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    q32 = q.float()
    with pytest.raises(dfdx_b200.B200Error) as e:                     # f16 only
        dev.attention_forward(q32, k.float(), v.float(), 1.0)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    qd, kd, vd = mha_views(1, 1, 64, 64, 12, gen(9), dev.device)      # D not a multiple of 8
    with pytest.raises(dfdx_b200.B200Error) as e:
        dev.attention_forward(qd, kd, vd, 1.0)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    assert dev.device_status() == 0


# ----------------------------------------------------------------------------------------------- backward
BWD_SHAPES = [(1, 1, 128, 128, 64), (2, 3, 200, 136, 64), (1, 2, 384, 520, 32), (1, 1, 128, 256, 128),
              (2, 2, 72, 72, 16), (1, 2, 8, 300, 64), (1, 1, 300, 8, 40), (1, 2, 130, 257, 96)]


@pytest.mark.parametrize("shape", BWD_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_attention_backward(cuda_dev, oracle, shape):
    """dQ, dK, dV against the oracle's op-by-op backward; gradients land in the operands' base layouts
    ((B,S,H,D) buffers) through the views' strides, as dfdx stores them."""
    b, h, s1, s2, d = shape
    g = gen(1000 + sum(shape))
    q, k, v = mha_views(b, h, s1, s2, d, g, cuda_dev.device)
    alpha = 1.0 / math.sqrt(d)
    out, lse = cuda_dev.attention_forward(q, k, v, alpha, want_lse=True)
    go = torch.randn(b, s1, h, d, generator=g, dtype=torch.float64).half().to(cuda_dev.device).permute(0, 2, 1, 3)
    before = cuda_dev.lib.b200_tensor_launch_count()
    gq, gk, gv = cuda_dev.attention_backward(q, k, v, alpha, out, lse, go)
    cuda_dev.synchronize()
    assert cuda_dev.lib.b200_tensor_launch_count() - before == 2
    assert gq.stride() == q.stride() and gk.stride() == k.stride() and gv.stride() == v.stride()
    wq, wk, wv = oracle.attention_backward(q.cpu(), k.cpu(), v.cpu(), alpha, go.cpu())
    for name, got, want in (("dQ", gq, wq), ("dK", gk, wk), ("dV", gv, wv)):
        err = oracle.rel_frobenius(got, want)
        assert err <= 2 * FROB_TOL[torch.float16], f"{name}: rel frobenius {err:.3e}"
    assert cuda_dev.device_status() == 0


@pytest.mark.parametrize("shape", [(40, 8, 256, 256, 64), (20, 8, 200, 264, 128), (30, 6, 300, 136, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_attention_many_work_items_per_cta(cuda_dev, oracle, shape):
    """More work items than SMs: each CTA of the forward and of both backward kernels walks several (batch, head,
    row tile) items, its barriers, shared-memory rings and tensor-memory buffers counting on across them (d <= 64:
    the backward's double-buffered accumulator sets; d = 128: one set; s1 = 300: the forward's one-CTA-per-item
    launch, because the last pair of query tiles of a head holds one tile only)."""
    b, h, s1, s2, d = shape
    dev = cuda_dev
    sms = torch.cuda.get_device_properties(dev.device).multi_processor_count
    assert b * h * ((s2 + 127) // 128) > sms and b * h * ((s1 + 127) // 128) > sms
    g = gen(2000 + sum(shape))
    q, k, v = mha_views(b, h, s1, s2, d, g, dev.device)
    alpha = 1.0 / math.sqrt(d)
    out, lse = dev.attention_forward(q, k, v, alpha, want_lse=True)
    go = torch.randn(b, s1, h, d, generator=g, dtype=torch.float64).half().to(dev.device).permute(0, 2, 1, 3)
    gq, gk, gv = dev.attention_backward(q, k, v, alpha, out, lse, go)
    dev.synchronize()
    want, want_lse = oracle.attention(q.cpu(), k.cpu(), v.cpu(), alpha)
    assert oracle.rel_frobenius(out, want) <= FROB_TOL[torch.float16]
    assert float((lse.cpu().double() - want_lse).abs().max()) <= 2e-3
    wq, wk, wv = oracle.attention_backward(q.cpu(), k.cpu(), v.cpu(), alpha, go.cpu())
    for name, got, ref in (("dQ", gq, wq), ("dK", gk, wk), ("dV", gv, wv)):
        err = oracle.rel_frobenius(got, ref)
        assert err <= 2 * FROB_TOL[torch.float16], f"{name}: rel frobenius {err:.3e}"
    # every item separately: the per-(batch, head) errors, not only the norm over all of them
    per_item = (out.float().cpu() - want.float()).flatten(2).norm(dim=2) / want.float().flatten(2).norm(dim=2)
    assert float(per_item.max()) <= 2 * FROB_TOL[torch.float16]
    per_item = (gk.float().cpu() - wk.float()).permute(0, 1, 3, 2).flatten(2).norm(dim=2) / \
        wk.float().permute(0, 1, 3, 2).flatten(2).norm(dim=2)
    assert float(per_item.max()) <= 4 * FROB_TOL[torch.float16]
    assert dev.device_status() == 0


def test_attention_backward_accumulates(cuda_dev, oracle):
    """accumulate = 1 adds to what the gradient buffers hold (two calls give twice the gradient)."""
    g = gen(77)
    q, k, v = mha_views(1, 2, 192, 160, 64, g, cuda_dev.device)
    out, lse = cuda_dev.attention_forward(q, k, v, 0.125, want_lse=True)
    go = torch.randn(1, 192, 2, 64, generator=g).half().to(cuda_dev.device).permute(0, 2, 1, 3)
    once = cuda_dev.attention_backward(q, k, v, 0.125, out, lse, go)
    bufs = (cuda_dev.alloc_grad(q), cuda_dev.alloc_grad(k), cuda_dev.alloc_grad(v))
    cuda_dev.attention_backward(q, k, v, 0.125, out, lse, go, accumulate_into=bufs)
    twice = cuda_dev.attention_backward(q, k, v, 0.125, out, lse, go, accumulate_into=bufs)
    for a, b2 in zip(once, twice):
        assert oracle.rel_frobenius(b2, 2.0 * a.double()) <= 1e-3


def test_attention_backward_workspace_is_checked(cuda_dev):
    g = gen(78)
    q, k, v = mha_views(1, 1, 64, 64, 64, g, cuda_dev.device)
    out, lse = cuda_dev.attention_forward(q, k, v, 0.125, want_lse=True)
    lib = cuda_dev.lib
    need = lib.b200_attention_backward_workspace_bytes(1, 1, 64)
    assert need == 64 * 8
    ws = torch.empty(need, dtype=torch.uint8, device=cuda_dev.device)
    gq, gk, gv = cuda_dev.alloc_grad(q), cuda_dev.alloc_grad(k), cuda_dev.alloc_grad(v)
    st = _lib.strides
    rc = lib.b200_attention_backward(_lib.F16, 1, 1, 64, 64, 64, q.data_ptr(), st(q.stride()), k.data_ptr(), st(k.stride()),
                                     v.data_ptr(), st(v.stride()), 0.125, out.data_ptr(), st(out.stride()), lse.data_ptr(),
                                     out.data_ptr(), st(out.stride()), gq.data_ptr(), st(q.stride()), gk.data_ptr(),
                                     st(k.stride()), gv.data_ptr(), st(v.stride()), 0, ws.data_ptr(), need - 1, None)
    assert rc == _lib.ERR_WORKSPACE
