"""Pins the oracle beyond the literal vectors: against torch's CPU f64 matmul / conv2d on seeded
random inputs (the reference's own goldens were produced with PyTorch, README.md:178-180), over the
stride patterns the path meets (permuted, broadcast, batched), and the properties the reference tests
(matmul/mod.rs:412-527; conv2d/tests.rs:218-250, :404-464)."""
import pytest
import torch
import torch.nn.functional as F

from helpers import OracleBackend, d_exp_mean, d_exp_sum, d_square_mean, d_sum

TOL = 1e-11


def gen(seed):
    return torch.Generator().manual_seed(seed)


def _grads(x, w, y_fn, dy_fn):
    x = x.clone().requires_grad_(True)
    w = w.clone().requires_grad_(True)
    y = y_fn(x, w)
    y.backward(dy_fn(y.detach()))
    return y.detach(), x.grad, w.grad


@pytest.mark.parametrize("shapes", [
    ((4, 3), (3, 2)), ((5, 4, 3), (3, 2)), ((5, 3, 2), (5, 2, 4)), ((7, 5, 3, 2), (7, 5, 2, 4)),
    ((3,), (3, 2)), ((5,), (3,)), ((4, 3), (3,)), ((33, 17), (17, 29)),
])
def test_matmul_matches_torch(oracle, shapes):
    be = OracleBackend(oracle)
    g = gen(1)
    a, b = be.randn(*shapes[0], gen=g), be.randn(*shapes[1], gen=g)
    out, bwd = be.matmul(a, b)
    if a.dim() == 1 and b.dim() == 1:
        fn = lambda x, w: torch.outer(x, w)
    else:
        fn = lambda x, w: torch.matmul(x, w)
    y, ga_t, gb_t = _grads(a, b, fn, d_exp_mean)
    assert (out - y).abs().max() < TOL
    ga, gb = bwd(d_exp_mean(out))
    assert (ga - ga_t).abs().max() < TOL and (gb - gb_t).abs().max() < TOL


def test_matmul_transpose_property(oracle):
    """matmul/mod.rs:412-426: (b^T a^T) yields the same gradients as (a b)."""
    be = OracleBackend(oracle)
    g = gen(2)
    a, b = be.randn(4, 3, gen=g), be.randn(3, 2, gen=g)
    c, bwd = be.matmul(a, b)
    ga1, gb1 = bwd(d_exp_mean(c))
    c2, bwd2 = be.matmul(b.permute(1, 0), a.permute(1, 0))
    gb2_view, ga2_view = bwd2(d_exp_mean(c2))
    assert (ga1 - ga2_view.permute(1, 0)).abs().max() < TOL
    assert (gb1 - gb2_view.permute(1, 0)).abs().max() < TOL


def test_matmul_broadcast_properties(oracle):
    """matmul/mod.rs:428-473: broadcast-rhs equals per-item 2-D matmuls; rhs gradient sums over the batch.
    Also :454-473: an expanded (stride-0) rhs through the batch-3 kernel accumulates into one buffer."""
    be = OracleBackend(oracle)
    g = gen(3)
    a, b = be.randn(5, 4, 3, gen=g), be.randn(3, 2, gen=g)
    r, bwd = be.matmul(a, b)
    ga, gb = bwd(d_sum(r))
    gb_sum = torch.zeros_like(gb)
    for i in range(5):
        ri, bwdi = be.matmul(a[i].contiguous(), b)
        assert (ri - r[i]).abs().max() < TOL
        gai, gbi = bwdi(d_sum(ri))
        assert (gai - ga[i]).abs().max() < TOL
        gb_sum += gbi
    assert (gb_sum - gb).abs().max() < TOL


@pytest.mark.parametrize("cfg", [
    dict(x=(2, 3, 7, 6), w=(4, 3, 2, 2), stride=1, padding=0, dilation=1, groups=1),
    dict(x=(1, 5, 7, 6), w=(3, 5, 2, 2), stride=4, padding=3, dilation=1, groups=1),
    dict(x=(3, 3, 28, 28), w=(5, 3, 6, 6), stride=3, padding=2, dilation=1, groups=1),
    dict(x=(2, 4, 9, 8), w=(6, 4, 3, 3), stride=2, padding=1, dilation=2, groups=1),
    dict(x=(2, 9, 14, 14), w=(15, 3, 3, 3), stride=1, padding=0, dilation=1, groups=3),
    dict(x=(2, 8, 10, 11), w=(4, 4, 3, 3), stride=2, padding=2, dilation=1, groups=2),
])
def test_conv2d_matches_torch(oracle, cfg):
    be = OracleBackend(oracle)
    g = gen(4)
    x, w = be.randn(*cfg["x"], gen=g), be.randn(*cfg["w"], gen=g)
    kw = {k: cfg[k] for k in ("stride", "padding", "dilation", "groups")}
    y, bwd = be.conv2d(x, w, **kw)
    yt, gxt, gwt = _grads(x, w, lambda a, b: F.conv2d(a, b, None, **kw), d_square_mean)
    assert y.shape == yt.shape
    assert (y - yt).abs().max() < TOL
    gx, gw = bwd(d_square_mean(y))
    assert (gx - gxt).abs().max() < TOL and (gw - gwt).abs().max() < TOL


def test_conv2d_grouped_equals_slices(oracle):
    """conv2d/tests.rs:404-464."""
    be = OracleBackend(oracle)
    g = gen(5)
    x, w = be.randn(2, 9, 14, 14, gen=g), be.randn(15, 3, 3, 3, gen=g)
    y, bwd = be.conv2d(x, w, groups=3)
    gx, gw = bwd(d_exp_sum(y))
    for i in range(3):
        xg, wg = x[:, 3 * i:3 * i + 3].contiguous(), w[5 * i:5 * i + 5].contiguous()
        yg, bwdg = be.conv2d(xg, wg)
        assert (yg - y[:, 5 * i:5 * i + 5]).abs().max() < TOL
        gxg, gwg = bwdg(d_exp_sum(yg))
        assert (gxg - gx[:, 3 * i:3 * i + 3]).abs().max() < TOL
        assert (gwg - gw[5 * i:5 * i + 5]).abs().max() < TOL


def test_out_dim_formula(oracle):
    assert oracle.conv2d_out_dim(56, 3, 1, 1, 1) == 56
    assert oracle.conv2d_out_dim(28, 6, 3, 2, 1) == 9
    assert oracle.conv2d_out_dim(7, 2, 4, 3, 1) == 3
    with pytest.raises(AssertionError):
        oracle.conv2d_out_dim(1, 5, 1, 0, 1)


def test_cpu_baseline_port_matches_oracle(oracle):
    """The timed CPU stand-in (oracle/cpu_baseline.c) computes the same MatMatBr forward / backward."""
    import ctypes as C
    import numpy as np
    L = oracle.baseline_lib()
    if not L.cpu_baseline_supported():
        pytest.skip("host CPU lacks AVX2/FMA")
    g = gen(9)
    b, m, k, n = 3, 37, 70, 45
    x = torch.randn(b, m, k, generator=g)
    w = torch.randn(n, k, generator=g)
    dy = torch.randn(b, m, n, generator=g)
    want_y, bwd = oracle.matmul(x, w.permute(1, 0))
    want_gx, want_gw = bwd(dy)
    fp = lambda t: t.numpy().ctypes.data_as(C.POINTER(C.c_float))
    st = lambda *v: (C.c_size_t * len(v))(*v)
    y = torch.empty(b, m, n)
    gx, gw = torch.zeros(b, m, k), torch.zeros(n, k)
    L.cpu_matmat_br_forward(b, m, k, n, fp(x), st(m * k, k, 1), fp(w), st(1, k), fp(y))
    L.cpu_matmat_br_backward(b, m, k, n, fp(x), st(m * k, k, 1), fp(gx), fp(w), st(1, k), fp(gw), fp(dy))
    assert oracle.rel_frobenius(y, want_y) < 1e-6
    assert oracle.rel_frobenius(gx, want_gx) < 1e-6
    assert oracle.rel_frobenius(gw.permute(1, 0), want_gw) < 1e-6


# ---- restatements added for the fused / neighbouring ops: each against torch's own f64 implementation ----------
def test_attention_oracle_matches_torch_autograd(oracle):
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, 20, 3, 16, generator=g, dtype=torch.float64).permute(0, 2, 1, 3).requires_grad_(True)
    k = torch.randn(2, 24, 3, 16, generator=g, dtype=torch.float64).permute(0, 2, 3, 1).requires_grad_(True)
    v = torch.randn(2, 24, 3, 16, generator=g, dtype=torch.float64).permute(0, 2, 1, 3).requires_grad_(True)
    go = torch.randn(2, 3, 20, 16, generator=g, dtype=torch.float64)
    ref = torch.softmax(q @ k * 0.25, -1) @ v
    ref.backward(go)
    out, lse = oracle.attention(q.detach(), k.detach(), v.detach(), 0.25)
    assert torch.allclose(out, ref.detach(), atol=1e-12)
    assert torch.allclose(lse, torch.logsumexp(q.detach() @ k.detach() * 0.25, -1), atol=1e-12)
    gq, gk, gv = oracle.attention_backward(q.detach(), k.detach(), v.detach(), 0.25, go)
    assert torch.allclose(gq, q.grad, atol=1e-12) and torch.allclose(gk, k.grad, atol=1e-12)
    assert torch.allclose(gv, v.grad, atol=1e-12)


def test_layer_norm_oracle_matches_torch(oracle):
    g = torch.Generator().manual_seed(12)
    x = torch.randn(7, 5, 33, generator=g, dtype=torch.float64, requires_grad=True)
    gamma = torch.randn(33, generator=g, dtype=torch.float64, requires_grad=True)
    beta = torch.randn(33, generator=g, dtype=torch.float64, requires_grad=True)
    go = torch.randn(7, 5, 33, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.layer_norm(x, (33,), gamma, beta, 1e-5)
    ref.backward(go)
    y, bwd = oracle.layer_norm(x.detach(), gamma.detach(), beta.detach(), 1e-5)
    gx, gg, gb = bwd(go)
    assert torch.allclose(y, ref.detach(), atol=1e-12)
    assert torch.allclose(gx, x.grad, atol=1e-12)
    assert torch.allclose(gg, gamma.grad, atol=1e-12) and torch.allclose(gb, beta.grad, atol=1e-12)


@pytest.mark.parametrize("case", [(2, 4, 6, 19, 3, 2, 1, 2, 2), (1, 3, 5, 28, 6, 1, 0, 1, 1), (3, 6, 6, 17, 4, 3, 2, 1, 3)])
def test_conv1d_oracle_matches_torch(oracle, case):
    b, c, o, l, k, stride, pad, dil, groups = case
    g = torch.Generator().manual_seed(sum(case))
    x = torch.randn(b, c, l, generator=g, dtype=torch.float64, requires_grad=True)
    w = torch.randn(o, c // groups, k, generator=g, dtype=torch.float64, requires_grad=True)
    ref = torch.nn.functional.conv1d(x, w, None, stride, pad, dil, groups)
    go = torch.randn(*ref.shape, generator=g, dtype=torch.float64)
    ref.backward(go)
    y, bwd = oracle.conv1d(x.detach(), w.detach(), stride=stride, padding=pad, dilation=dil, groups=groups)
    gx, gw = bwd(go)
    assert torch.allclose(y, ref.detach(), atol=1e-12)
    assert torch.allclose(gx, x.grad, atol=1e-12) and torch.allclose(gw, w.grad, atol=1e-12)


@pytest.mark.parametrize("case", [(2, 4, 6, 5, 6, 3, 2, 1, 1, 2), (1, 3, 2, 4, 4, 2, 1, 0, 2, 1), (2, 6, 3, 5, 5, 3, 3, 2, 1, 3)])
def test_convtrans2d_oracle_matches_torch(oracle, case):
    b, c, o, h, w_, k, stride, pad, dil, groups = case
    g = torch.Generator().manual_seed(sum(case))
    x = torch.randn(b, c, h, w_, generator=g, dtype=torch.float64, requires_grad=True)
    w = torch.randn(c, o // groups, k, k, generator=g, dtype=torch.float64, requires_grad=True)
    ref = torch.nn.functional.conv_transpose2d(x, w, None, stride, pad, 0, groups, dil)
    go = torch.randn(*ref.shape, generator=g, dtype=torch.float64)
    ref.backward(go)
    y, bwd = oracle.convtrans2d(x.detach(), w.detach(), stride=stride, padding=pad, dilation=dil, groups=groups)
    gx, gw = bwd(go)
    assert y.shape == ref.shape
    assert torch.allclose(y, ref.detach(), atol=1e-12)
    assert torch.allclose(gx, x.grad, atol=1e-12) and torch.allclose(gw, w.grad, atol=1e-12)
