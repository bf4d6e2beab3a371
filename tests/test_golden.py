"""The reference's literal known-answer tests for the path, re-stated over the extracted vectors
(tests/golden/*.json, produced by tests/golden/make_golden.py from dfdx's Rust test sources).

Each test body follows the dfdx test of the same name:
  matmul  — dfdx-core/src/tensor_ops/matmul/mod.rs:367-410, :529-702
  linear  — dfdx/src/nn/layers/linear.rs:97-204   (x.matmul(weight.permute()) + bias)
  conv2d  — dfdx-core/src/tensor_ops/conv2d/tests.rs:11-196, :252-402
  softmax — dfdx-core/src/tensor_ops/softmax.rs:111-196
and runs on the CPU oracle (pins the oracle; no GPU) and on the CUDA device (marked gpu) with the
reference's absolute tolerances (1e-6 for f32/f64, 1e-2 for f16; dfdx-core/src/lib.rs:236-270).
"""
import math

import pytest
import torch

from helpers import (ABS_TOL, CudaBackend, OracleBackend, assert_close, d_exp_mean, d_exp_sum, d_mean,
                     d_square_mean, golden)

BACKENDS = [
    pytest.param(("oracle", torch.float64), id="oracle-f64"),
    pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", torch.float64), id="cuda-f64", marks=pytest.mark.gpu),
    pytest.param(("cuda", torch.float16), id="cuda-f16", marks=pytest.mark.gpu),
]


@pytest.fixture(params=BACKENDS)
def be(request):
    kind, dtype = request.param
    if kind == "oracle":
        return OracleBackend(request.getfixturevalue("oracle"), dtype)
    return CudaBackend(request.getfixturevalue("cuda_dev"), dtype)


def _split(events):
    tensors = [e["value"] for e in events if e["kind"] == "tensor"]
    asserts = [e for e in events if e["kind"] == "assert"]
    return tensors, asserts


def _check(be, got, a, shape_like=None):
    tol = a["tol"] if a["tol"] is not None else ABS_TOL[be.dtype]
    tol = max(tol, ABS_TOL[be.dtype])
    want = torch.tensor(a["value"], dtype=torch.float64)
    if be.dtype == torch.float16:
        # f16 storage: allow a few ulps (2^-10 relative each) of the largest expected value
        tol = max(tol, 4e-3 * float(want.abs().max()))
    elif be.dtype == torch.float32:
        # the literals were computed by PyTorch in f32: allow two f32 ulps of the largest value
        tol = max(tol, 2.4e-7 * float(want.abs().max()))
    assert_close(be.host(got).reshape(want.shape), want, tol, a["expr"])


def _mm_case(be, a, b, asserts, loss, a_view=None, b_view=None):
    """r = a_view.matmul(b_view); checks r, g(a), g(b).  Gradients are compared in the BASE layout
    of a / b (dfdx stores a permuted view's gradient in the base tensor's buffer)."""
    av = a if a_view is None else a_view(a)
    bv = b if b_view is None else b_view(b)
    r, bwd = be.matmul(av, bv)
    if asserts[0]["value"] is not None:
        _check(be, r, asserts[0])
    ga, gb = bwd(loss(be.host(r)))
    ga = ga if a_view is None else a_view(ga)   # permute is an involution for rank 2
    gb = gb if b_view is None else b_view(gb)
    if asserts[1]["value"] is not None:
        _check(be, ga, asserts[1])
    if asserts[2]["value"] is not None:
        _check(be, gb, asserts[2])
    return r, ga, gb


def permute(t):
    return t.permute(1, 0)


# ------------------------------------------------------------------------------------------ matmul
def test_matmul_normal(be):
    t, a = _split(golden("matmul")["test_matmul_normal"])
    _mm_case(be, be.tensor(t[0]), be.tensor(t[1]), a, d_exp_mean)


def test_matmul_vec_normal(be):
    t, a = _split(golden("matmul")["test_matmul_vec_normal"])
    _mm_case(be, be.tensor(t[0]), be.tensor(t[1]), a, d_exp_mean)


def test_matmul_vec_transpose(be):
    t, a = _split(golden("matmul")["test_matmul_vec_transpose"])
    _mm_case(be, be.tensor(t[0]), be.tensor(t[1]), a, d_exp_mean, b_view=permute)


def test_vecvec(be):
    t, a = _split(golden("matmul")["test_vecvec"])
    x, y = be.tensor(t[0]), be.tensor(t[1])
    c, _, _ = _mm_case(be, x, y, a, d_exp_mean)
    c_t, _ = be.matmul(y, x)
    assert torch.equal(be.host(c), be.host(c_t).permute(1, 0))


def test_small_matmul_vv(be):
    t, a = _split(golden("matmul")["test_small_matmul_vv"])
    _mm_case(be, be.tensor(t[0]), be.tensor(t[1]), a, d_exp_sum)


def test_small_matmul_vm(be):
    t, a = _split(golden("matmul")["test_small_matmul_vm"])
    x, y = be.tensor(t[0]), be.tensor(t[1])
    _mm_case(be, x, y, a[0:3], d_exp_sum)                       # 1 * 1x1
    _mm_case(be, x, y, a[3:6], d_exp_sum, b_view=permute)       # 1 * 1x1 (permuted)
    e = [1.0, 2.0]
    ga_want = math.exp(e[0]) * 2.0 + math.exp(e[1]) * 4.0
    for tensors, asserts, view in ((t[2:4], a[6:9], None), (t[4:6], a[9:12], permute)):
        x, y = be.tensor(tensors[0]), be.tensor(tensors[1])
        r, ga, _ = _mm_case(be, x, y, asserts, d_exp_sum, b_view=view)
        assert_close(be.host(r), e, ABS_TOL[be.dtype], "c")
        assert_close(be.host(ga), [ga_want], max(1e-4, ABS_TOL[be.dtype] * 4), "g.get(&a)")


def test_small_matmul_mm(be):
    t, a = _split(golden("matmul")["test_small_matmul_mm"])
    views = [(None, None), (None, None), (permute, None), (None, permute)]
    for i, (av, bv) in enumerate(views):
        _mm_case(be, be.tensor(t[2 * i]), be.tensor(t[2 * i + 1]), a[3 * i:3 * i + 3], d_exp_sum,
                 a_view=av, b_view=bv)


# ------------------------------------------------------------------------------------------ linear
@pytest.mark.parametrize("name", ["test_forward_1d", "test_forward_2d", "test_forward_3d"])
def test_linear(be, name):
    t, a = _split(golden("linear")[name])
    weight, bias, x = be.tensor(t[0]), be.tensor(t[1]), be.tensor(t[2])
    y_mm, bwd = be.matmul(x, weight.permute(1, 0))              # linear.rs:82-89
    y = be.host(y_mm) + be.host(bias)                            # Bias1D, host side
    _check(be, y, a[0])
    dy = d_square_mean(y)
    _, gw_view = bwd(dy)
    _check(be, gw_view.permute(1, 0), a[1])                      # gradient in the (O, I) base layout
    _check(be, dy.reshape(-1, dy.shape[-1]).sum(0), a[2])


@pytest.mark.parametrize("name", ["test_forward_1d", "test_forward_2d", "test_forward_3d"])
def test_linear_fused_forward(be, name):
    """The same known answers through the one-launch Linear forward (matmul + bias in the epilogue)."""
    t, a = _split(golden("linear")[name])
    weight, bias, x = be.tensor(t[0]), be.tensor(t[1]), be.tensor(t[2])
    _check(be, be.linear(x, weight.permute(1, 0), bias), a[0])
    y_relu = be.host(be.linear(x, weight.permute(1, 0), bias, relu=True))
    want = torch.clamp_min(torch.tensor(a[0]["value"], dtype=torch.float64), 0.0)
    _check(be, y_relu, dict(a[0], value=want.tolist()))


# ------------------------------------------------------------------------------------------ conv1d
CONV1D_CASES = {
    "test_conv1d_default_stride_and_padding": dict(stride=1, padding=0, dilation=1, groups=1),
    "test_conv1d_all": dict(stride=2, padding=1, dilation=2, groups=1),
    "test_conv1d_all_grouped": dict(stride=2, padding=1, dilation=2, groups=2),
}


@pytest.mark.parametrize("name", list(CONV1D_CASES))
def test_conv1d(be, name):
    """dfdx-core/src/tensor_ops/conv1d/tests.rs:4-131: result, then g = result.exp().mean().backward()."""
    t, a = _split(golden("conv1d")[name])
    order = (1, 0) if name == "test_conv1d_all_grouped" else (0, 1)       # that test builds x before w
    weight, x = be.tensor(t[order[0]]), be.tensor(t[order[1]])
    y, bwd = be.conv1d(x, weight, **CONV1D_CASES[name])
    _check(be, y, a[0])
    gx, gw = bwd(d_exp_mean(be.host(y)))
    _check(be, gx, a[1])
    _check(be, gw, a[2])


# ------------------------------------------------------------------------------------------ convtrans2d
CONVTRANS2D_CASES = {
    "test_convtrans2d_default": dict(stride=1, padding=0, dilation=1, groups=1),
    "test_convtrans2d_stride_2": dict(stride=2, padding=0, dilation=1, groups=1),
    "test_convtrans2d_padded": dict(stride=1, padding=1, dilation=1, groups=1),
    "test_convtrans2d_grouped": dict(stride=1, padding=0, dilation=1, groups=2),
    "test_convtrans2d_dilated": dict(stride=1, padding=0, dilation=2, groups=1),
}


@pytest.mark.parametrize("name", list(CONVTRANS2D_CASES))
def test_convtrans2d(be, name):
    """dfdx-core/src/tensor_ops/convtrans2d/tests.rs:4-516: y, then g = y.exp().mean().backward()."""
    t, a = _split(golden("convtrans2d")[name])
    x, w = be.tensor(t[0]), be.tensor(t[1])
    y, bwd = be.convtrans2d(x, w, **CONVTRANS2D_CASES[name])
    _check(be, y, a[0])
    gx, gw = bwd(d_exp_mean(be.host(y)))
    _check(be, gx, a[1])
    _check(be, gw, a[2])


# ------------------------------------------------------------------------------------------ normalize
@pytest.mark.parametrize("name", ["test_1d_normalize_axis_last", "test_2d_normalize_axis_last"])
def test_normalize_last_axis(be, name):
    """dfdx-core/src/tensor_ops/normalize.rs:52-96: r = a.normalize(1e-5); g = r.exp().mean().backward()."""
    if be.dtype == torch.float64 and be.name == "cuda":
        pytest.skip("the row-wise kernels serve f32 and f16")
    t, a = _split(golden("normalize")[name])
    x = be.tensor(t[0])
    r, bwd = be.normalize(x, 1e-5)
    _check(be, r, a[0])
    _check(be, bwd(d_exp_mean(be.host(r))), a[1])


# ------------------------------------------------------------------------------------------ softmax
@pytest.mark.parametrize("name,axis", [("test_softmax_1d", -1), ("test_softmax_2d", 1), ("test_softmax_2d_0th_axis", 0)])
def test_softmax(be, name, axis):
    """dfdx-core/src/tensor_ops/softmax.rs:111-196: r = a.softmax::<Axis>(); l = r * mask; g = l.mean().backward().
    The kernels reduce over the last axis; the 0th-axis test runs on the transposed matrix."""
    if be.dtype == torch.float64 and be.name == "cuda":
        pytest.skip("the row-wise kernels serve f32 and f16")
    t, a = _split(golden("softmax")[name])
    x, mask = be.tensor(t[0]), torch.tensor(t[1], dtype=torch.float64)
    tr = (lambda v: v.t()) if axis == 0 else (lambda v: v)
    r, bwd = be.softmax(tr(x))
    _check(be, tr(be.host(r)), a[0])
    _check(be, tr(be.host(r)) * mask, a[1])
    g = bwd(tr(mask / mask.numel()).contiguous())
    _check(be, tr(be.host(g)), a[2])


# ------------------------------------------------------------------------------------------ conv2d
CONV_BIAS_CASES = {
    "test_conv2d_default_stride_and_padding": dict(stride=1, padding=0),
    "test_conv2d_stride_2": dict(stride=2, padding=0),
    "test_conv2d_padding_1": dict(stride=1, padding=1),
    "test_conv2d_stride_3_padding_4": dict(stride=3, padding=4),
}


@pytest.mark.parametrize("name", list(CONV_BIAS_CASES))
def test_conv2d_with_bias(be, name):
    t, a = _split(golden("conv2d")[name])
    weight, bias, x = be.tensor(t[0]), be.tensor(t[1]), be.tensor(t[2])
    y, bwd = be.conv2d(x, weight, **CONV_BIAS_CASES[name])
    result = be.host(y) + be.host(bias).reshape(-1, 1, 1)        # bias.broadcast::<_, Axes2<1, 2>>()
    _check(be, result, a[0])
    d = d_exp_mean(result)
    gx, gw = bwd(d)
    _check(be, gx, a[1])
    _check(be, gw, a[2])
    _check(be, d.sum(dim=(1, 2)), a[3])


def test_conv2d_dilated(be):
    t, a = _split(golden("conv2d")["test_conv2d_dilated"])
    x, w = be.tensor(t[0]), be.tensor(t[1])
    y, bwd = be.conv2d(x, w, stride=1, padding=0, dilation=2, groups=1)
    # values reach 63.8: one f16 ulp there is 3.1e-2, so f16 gets a relative allowance
    tol_y = 5e-2 if be.dtype == torch.float16 else None
    if tol_y:
        assert_close(be.host(y), a[0]["value"], tol_y, "y")
    else:
        _check(be, y, a[0])
    gx, gw = bwd(d_mean(be.host(y)))
    _check(be, gx, a[1])
    if be.dtype == torch.float16:
        assert_close(be.host(gw), a[2]["value"], 2e-2, "grads.get(&w)")
    else:
        _check(be, gw, a[2])


def test_conv2d_grouped(be):
    t, a = _split(golden("conv2d")["test_conv2d_grouped"])
    x, w = be.tensor(t[0]), be.tensor(t[1])
    y, bwd = be.conv2d(x, w, stride=1, padding=0, dilation=1, groups=2)
    _check(be, y, a[0])
    gx, gw = bwd(d_exp_mean(be.host(y)))
    _check(be, gx, a[1])
    _check(be, gw, a[2])
