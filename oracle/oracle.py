"""TEST INFRASTRUCTURE — Python front-end of the CPU oracle (oracle.c) and the CPU baseline port.

Only tests/, `__graft_entry__.smoke()` and bench.py's CPU-baseline / reference arm may import this.
Tensors are torch CPU tensors (any dtype, any view); they are widened to f64 over their whole
storage so that strides keep their meaning, and results come back as f64 torch tensors.
The API mirrors `dfdx_b200.Cuda` (matmul / conv2d returning `(out, backward)`), which in turn
mirrors dfdx's `TryMatMul` / `TryConv2D`.

Restatements written directly in this file (f64, torch CPU ops + the C matmul): `fused_matmul`, `attention`,
`attention_backward`, `layer_norm`, `conv1d`, `convtrans2d`; each docstring names the reference lines it follows.
Parity is pinned: matmul, linear, conv2d, conv1d, convtrans2d and normalize reproduce every literal known answer
the reference's tests hold for them (tests/golden/*.json, tests/test_golden.py); the attention restatement is the
composition of pinned pieces (matmul, and softmax = exp(x - logsumexp)) and is checked against torch f64 autograd
(tests/test_oracle.py), because the reference's MultiHeadAttention tests draw their inputs from Rust's seeded RNG.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
_sz = C.c_size_t
_szp = C.POINTER(C.c_size_t)
_dp = C.POINTER(C.c_double)
_fp = C.POINTER(C.c_float)


class Conv2DOp(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in (
        "kernel", "stride", "padding", "dilation", "groups", "batch",
        "chan_in", "chan_out", "h_in", "h_out", "w_in", "w_out")]


def build() -> None:
    """Compiles liboracle.so and libcpu_baseline.so next to their sources (idempotent)."""
    res = subprocess.run(["make", "-C", str(HERE)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"oracle build failed:\n{res.stdout}\n{res.stderr}")


_oracle = None
_baseline = None


def lib() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not (HERE / "liboracle.so").exists():
            build()
        L = C.CDLL(str(HERE / "liboracle.so"))
        L.oracle_gemm.argtypes = [_sz, _sz, _sz, C.c_int, _dp, _szp, _dp, _szp, _dp, _szp]
        L.oracle_matmat_forward.argtypes = [_sz, _sz, _sz, _dp, _szp, _dp, _szp, _dp]
        L.oracle_matmat_backward.argtypes = [_sz, _sz, _sz, _dp, _szp, _dp, _dp, _szp, _dp, _dp]
        L.oracle_matmat_br_forward.argtypes = [_sz] * 4 + [_dp, _szp, _dp, _szp, _dp]
        L.oracle_matmat_br_backward.argtypes = [_sz] * 4 + [_dp, _szp, _dp, _dp, _szp, _dp, _dp]
        L.oracle_matmat_batch3_forward.argtypes = [_sz] * 4 + [_dp, _szp, _dp, _szp, _dp]
        L.oracle_matmat_batch3_backward.argtypes = [_sz] * 4 + [_dp, _szp, _dp, _dp, _szp, _dp, _dp]
        L.oracle_matmat_batch4_forward.argtypes = [_sz] * 5 + [_dp, _szp, _dp, _szp, _dp]
        L.oracle_matmat_batch4_backward.argtypes = [_sz] * 5 + [_dp, _szp, _dp, _dp, _szp, _dp, _dp]
        L.oracle_conv2d_out_dim.argtypes = [_sz] * 5
        L.oracle_conv2d_out_dim.restype = _sz
        L.oracle_conv2d_forward.argtypes = [C.POINTER(Conv2DOp), _dp, _szp, _dp, _dp]
        L.oracle_conv2d_forward.restype = C.c_int
        L.oracle_conv2d_backward.argtypes = [C.POINTER(Conv2DOp), _dp, _dp, _dp, _szp, _dp, _dp]
        L.oracle_conv2d_backward.restype = C.c_int
        _oracle = L
    return _oracle


def baseline_lib() -> C.CDLL:
    global _baseline
    if _baseline is None:
        if not (HERE / "libcpu_baseline.so").exists():
            build()
        L = C.CDLL(str(HERE / "libcpu_baseline.so"))
        L.cpu_baseline_supported.restype = C.c_int
        L.cpu_baseline_threads.restype = C.c_int
        L.cpu_sgemm.argtypes = [_sz, _sz, _sz, C.c_int, _fp, _szp, _fp, _szp, _fp, _szp]
        L.cpu_matmat_forward.argtypes = [_sz, _sz, _sz, _fp, _szp, _fp, _szp, _fp]
        L.cpu_matmat_backward.argtypes = [_sz, _sz, _sz, _fp, _szp, _fp, _fp, _szp, _fp, _fp]
        L.cpu_matmat_br_forward.argtypes = [_sz] * 4 + [_fp, _szp, _fp, _szp, _fp]
        L.cpu_matmat_br_backward.argtypes = [_sz] * 4 + [_fp, _szp, _fp, _fp, _szp, _fp, _fp]
        _baseline = L
    return _baseline


def _strides(seq):
    return (C.c_size_t * len(seq))(*[int(s) for s in seq])


class _Buf:
    """A tensor's whole storage widened to f64, plus the view (offset, shape, strides) into it."""

    def __init__(self, t: torch.Tensor):
        t = t.detach().cpu()
        n = t.untyped_storage().nbytes() // t.element_size()
        flat = torch.empty(0, dtype=t.dtype).set_(t.untyped_storage(), 0, (n,), (1,))
        self.data = flat.to(torch.float64).contiguous().numpy()
        self.offset = t.storage_offset()
        self.shape = tuple(t.shape)
        self.strides = tuple(t.stride())

    @property
    def ptr(self):
        return self.data[self.offset:].ctypes.data_as(_dp)

    def zeros_like_storage(self) -> np.ndarray:
        return np.zeros_like(self.data)

    def view_of(self, flat: np.ndarray) -> torch.Tensor:
        return torch.as_strided(torch.from_numpy(flat), self.shape, self.strides, self.offset)


def _out(shape) -> np.ndarray:
    return np.empty(int(np.prod(shape)) if len(shape) else 1, dtype=np.float64)


def _p(a: np.ndarray):
    return a.ctypes.data_as(_dp)


def gemm(mkn, lhs: _Buf, lhs_strides, rhs: _Buf, rhs_strides, accum: bool, out: np.ndarray, out_strides):
    m, k, n = mkn
    lib().oracle_gemm(m, k, n, int(accum), lhs.ptr, _strides(lhs_strides), rhs.ptr, _strides(rhs_strides),
                      _p(out), _strides(out_strides))


class ShapeMismatch(AssertionError):
    pass


def _assert_eq(a, b):
    if a != b:
        raise ShapeMismatch(f"left: {a}\n right: {b}")


_KINDS = {
    (2, 2): ("oracle_matmat", 0), (3, 2): ("oracle_matmat_br", 1),
    (3, 3): ("oracle_matmat_batch3", 1), (4, 4): ("oracle_matmat_batch4", 2),
}


def matmul(lhs: torch.Tensor, rhs: torch.Tensor):
    """Rank dispatch of `TryMatMul` (matmul/mod.rs:133-311) on the oracle.  Returns (out, backward);
    backward(grad_out) -> (grad_lhs, grad_rhs) as f64 views through the operands' strides."""
    ld, rd = lhs.dim(), rhs.dim()
    if ld == 1 and rd == 1:
        l2 = torch.as_strided(lhs, (lhs.shape[0], 1), (lhs.stride(0), 1), lhs.storage_offset())
        r2 = torch.as_strided(rhs, (1, rhs.shape[0]), (rhs.shape[0], rhs.stride(0)), rhs.storage_offset())
        return _run(l2, r2, lhs, rhs, None)
    if ld == 1 and rd == 2:
        _assert_eq(lhs.shape[0], rhs.shape[0])
        l2 = torch.as_strided(lhs, (1, lhs.shape[0]), (lhs.shape[0], lhs.stride(0)), lhs.storage_offset())
        return _run(l2, rhs, lhs, rhs, (rhs.shape[1],))
    if ld == 2 and rd == 1:
        _assert_eq(lhs.shape[1], rhs.shape[0])
        r2 = torch.as_strided(rhs, (rhs.shape[0], 1), (rhs.stride(0), 1), rhs.storage_offset())
        return _run(lhs, r2, lhs, rhs, (lhs.shape[0],))
    if (ld, rd) not in _KINDS:
        raise TypeError(f"matmul is not defined for ranks {ld} x {rd}")
    if ld == rd:
        for i in range(ld - 2):
            _assert_eq(lhs.shape[i], rhs.shape[i])
    _assert_eq(lhs.shape[-1], rhs.shape[-2])
    return _run(lhs, rhs, lhs, rhs, None)


def _run(l, r, l_orig, r_orig, out_shape):
    name, nbatch = _KINDS[(l.dim(), r.dim())]
    L = lib()
    lb, rb = _Buf(l), _Buf(r)
    batch = tuple(l.shape[:nbatch])
    m, k, n = l.shape[-2], l.shape[-1], r.shape[-1]
    oshape = batch + (m, n)
    out = _out(oshape)
    getattr(L, name + "_forward")(*batch, m, k, n, lb.ptr, _strides(lb.strides), rb.ptr, _strides(rb.strides), _p(out))
    out_t = torch.from_numpy(out).reshape(oshape)
    shaped = out_t if out_shape is None else out_t.reshape(out_shape)

    def backward(grad_out: torch.Tensor):
        go = np.ascontiguousarray(grad_out.detach().cpu().to(torch.float64).reshape(oshape).numpy())
        gl, gr = lb.zeros_like_storage(), rb.zeros_like_storage()
        getattr(L, name + "_backward")(*batch, m, k, n, lb.ptr, _strides(lb.strides),
                                       gl[lb.offset:].ctypes.data_as(_dp), rb.ptr, _strides(rb.strides),
                                       gr[rb.offset:].ctypes.data_as(_dp), _p(go))
        gl_v = torch.as_strided(torch.from_numpy(gl), l_orig.shape, l_orig.stride(), l_orig.storage_offset())
        gr_v = torch.as_strided(torch.from_numpy(gr), r_orig.shape, r_orig.stride(), r_orig.storage_offset())
        return gl_v, gr_v

    return shaped, backward


def conv2d_out_dim(dim, kernel, stride, padding, dilation) -> int:
    v = lib().oracle_conv2d_out_dim(dim, kernel, stride, padding, dilation)
    if v == (1 << 64) - 1:
        raise ShapeMismatch("called `Option::unwrap()` on a `None` value")
    return int(v)


def conv2d(img: torch.Tensor, filters: torch.Tensor, stride=1, padding=0, dilation=1, groups=1):
    """`TryConv2D` (conv2d/mod.rs:273-324) on the oracle.  Returns (out, backward)."""
    squeeze = img.dim() == 3
    x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
    if not x.is_contiguous() or not filters.is_contiguous():
        raise ShapeMismatch("Image & filter inputs to conv2d must be contiguous")
    b, c, h, w = x.shape
    o, cg, k, k2 = filters.shape
    _assert_eq(c, cg * groups)
    _assert_eq(k, k2)
    op = Conv2DOp(kernel=k, stride=stride, padding=padding, dilation=dilation, groups=groups, batch=b,
                  chan_in=c, chan_out=o, h_in=h, h_out=conv2d_out_dim(h, k, stride, padding, dilation),
                  w_in=w, w_out=conv2d_out_dim(w, k, stride, padding, dilation))
    L = lib()
    xb, fb = _Buf(x), _Buf(filters)
    oshape = (b, o, op.h_out, op.w_out)
    out = _out(oshape)
    rc = L.oracle_conv2d_forward(C.byref(op), xb.ptr, _strides(xb.strides), fb.ptr, _p(out))
    assert rc == 0
    out_t = torch.from_numpy(out).reshape(oshape)

    def backward(grad_out: torch.Tensor):
        go = np.ascontiguousarray(grad_out.detach().cpu().to(torch.float64).reshape(oshape).numpy())
        gx, gf = xb.zeros_like_storage(), fb.zeros_like_storage()
        rc2 = L.oracle_conv2d_backward(C.byref(op), xb.ptr, gx[xb.offset:].ctypes.data_as(_dp), fb.ptr,
                                       _strides(fb.strides), gf[fb.offset:].ctypes.data_as(_dp), _p(go))
        assert rc2 == 0
        return xb.view_of(gx).reshape(img.shape), fb.view_of(gf)

    return (out_t[0] if squeeze else out_t), backward


def conv1d(img: torch.Tensor, filters: torch.Tensor, stride=1, padding=0, dilation=1, groups=1):
    """`TryConv1D` on the oracle (dfdx-core/src/tensor_ops/conv1d/mod.rs:160-286; arithmetic of
    conv1d/cpu_kernel.rs:20-250: patches[c, k, l] = img[c, l*stride + k*dilation - padding] or 0 outside, then one
    matmul per image and group; backward = the transposed gather of grad_out times the transposed filters for the
    image, and img x patches(grad_out)^T summed over the batch for the filters), in f64.  Returns (out, backward)."""
    squeeze = img.dim() == 2
    x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
    if not x.is_contiguous() or not filters.is_contiguous():
        raise ShapeMismatch("Image & filter inputs to conv1d must be contiguous")
    b, c, l = x.shape
    o, cg, k = filters.shape
    _assert_eq(c, cg * groups)
    og = o // groups
    l_out = conv2d_out_dim(l, k, stride, padding, dilation)
    x64 = x.detach().cpu().to(torch.float64)
    w64 = filters.detach().cpu().to(torch.float64)

    def patches_of(t):                      # (B, C, L) -> (B, C, K, L_out) with zero padding
        p = torch.zeros(t.shape[0], t.shape[1], k, l_out, dtype=torch.float64)
        for kk in range(k):
            for lo in range(l_out):
                pos = lo * stride + kk * dilation - padding
                if 0 <= pos < l:
                    p[:, :, kk, lo] = t[:, :, pos]
        return p

    pat = patches_of(x64)
    out = torch.zeros(b, o, l_out, dtype=torch.float64)
    for g in range(groups):
        wg = w64[g * og:(g + 1) * og].reshape(og, cg * k)
        pg = pat[:, g * cg:(g + 1) * cg].reshape(b, cg * k, l_out)
        for i in range(b):
            out[i, g * og:(g + 1) * og], _ = matmul(wg, pg[i])

    def backward(grad_out: torch.Tensor):
        go = grad_out.detach().cpu().to(torch.float64).reshape(b, o, l_out)
        gx = torch.zeros(b, c, l, dtype=torch.float64)
        gw = torch.zeros(o, cg, k, dtype=torch.float64)
        for g in range(groups):
            wg = w64[g * og:(g + 1) * og].reshape(og, cg * k)
            for i in range(b):
                gp, _ = matmul(wg.t().contiguous(), go[i, g * og:(g + 1) * og])          # (cg*k, l_out)
                gp = gp.reshape(cg, k, l_out)
                for kk in range(k):
                    for lo in range(l_out):
                        pos = lo * stride + kk * dilation - padding
                        if 0 <= pos < l:
                            gx[i, g * cg:(g + 1) * cg, pos] += gp[:, kk, lo]
                d, _ = matmul(go[i, g * og:(g + 1) * og], pat[i, g * cg:(g + 1) * cg].reshape(cg * k, l_out).t().contiguous())
                gw[g * og:(g + 1) * og] += d.reshape(og, cg, k)
        return gx.reshape(img.shape), gw

    return (out[0] if squeeze else out), backward


def convtrans2d(img: torch.Tensor, filters: torch.Tensor, stride=1, padding=0, dilation=1, groups=1):
    """`TryConvTrans2D` on the oracle (dfdx-core/src/tensor_ops/convtrans2d/mod.rs:124-280; arithmetic of
    convtrans2d/cpu_kernel.rs:9-271): input pixel (y, x) feeds output pixel (y*stride + k1*dilation - padding,
    x*stride + k2*dilation - padding) through tap (k1, k2) when that lies inside the output (`unfold_idx`, :10-17);
    filters are (C, O/G, K, K).  f64.  Returns (out, backward)."""
    squeeze = img.dim() == 3
    x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
    if not x.is_contiguous() or not filters.is_contiguous():
        raise ShapeMismatch("Image & filter inputs to conv2d must be contiguous")
    b, c, h, w = x.shape
    c2, og, k, k2 = filters.shape
    _assert_eq(c, c2)
    _assert_eq(k, k2)
    o, cg = og * groups, c // groups
    h_out = (h - 1) * stride + dilation * (k - 1) + 1 - 2 * padding
    w_out = (w - 1) * stride + dilation * (k - 1) + 1 - 2 * padding
    x64 = x.detach().cpu().to(torch.float64)
    w64 = filters.detach().cpu().to(torch.float64)

    def taps():
        for k1 in range(k):
            for kk2 in range(k):
                for y in range(h):
                    oh = y * stride + k1 * dilation - padding
                    if not 0 <= oh < h_out:
                        continue
                    for xx in range(w):
                        ow = xx * stride + kk2 * dilation - padding
                        if 0 <= ow < w_out:
                            yield k1, kk2, y, xx, oh, ow

    out = torch.zeros(b, o, h_out, w_out, dtype=torch.float64)
    for g in range(groups):
        xs, ws = x64[:, g * cg:(g + 1) * cg], w64[g * cg:(g + 1) * cg]              # (B, cg, H, W), (cg, og, K, K)
        for k1, kk2, y, xx, oh, ow in taps():
            out[:, g * og:(g + 1) * og, oh, ow] += xs[:, :, y, xx] @ ws[:, :, k1, kk2]

    def backward(grad_out: torch.Tensor):
        go = grad_out.detach().cpu().to(torch.float64).reshape(b, o, h_out, w_out)
        gx = torch.zeros(b, c, h, w, dtype=torch.float64)
        gw = torch.zeros(c, og, k, k, dtype=torch.float64)
        for g in range(groups):
            xs, ws = x64[:, g * cg:(g + 1) * cg], w64[g * cg:(g + 1) * cg]
            gs = go[:, g * og:(g + 1) * og]
            for k1, kk2, y, xx, oh, ow in taps():
                gx[:, g * cg:(g + 1) * cg, y, xx] += gs[:, :, oh, ow] @ ws[:, :, k1, kk2].t()
                gw[g * cg:(g + 1) * cg, :, k1, kk2] += xs[:, :, y, xx].t() @ gs[:, :, oh, ow]
        return gx.reshape(img.shape), gw

    return (out[0] if squeeze else out), backward


def fused_matmul(lhs: torch.Tensor, rhs: torch.Tensor, alpha: float = 1.0, bias: torch.Tensor = None,
                 relu: bool = False) -> torch.Tensor:
    """The op sequences the fused epilogues stand for, step by step in f64: `matmul`, then `* scalar`
    (multi_head_attention.rs:136-137), then `Bias1D` = bias broadcast over the leading dims + add
    (nn/layers/bias1d.rs:66-79, called from linear.rs:82-89), then `ReLU` = max(x, 0)."""
    y, _ = matmul(lhs, rhs)
    y = y * float(alpha)
    if bias is not None:
        y = y + bias.detach().cpu().to(torch.float64)
    if relu:
        y = torch.clamp_min(y, 0.0)
    return y


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alpha: float):
    """The middle of `MultiHeadAttention::try_forward` (dfdx/src/nn/layers/multi_head_attention.rs:136-141) in
    f64: weights = softmax(q.matmul(k) * alpha) over the last axis (softmax.rs: exp(x - logsumexp(x))),
    tokens = weights.matmul(v).  q (B,H,S1,D), k (B,H,D,S2), v (B,H,S2,D).  Returns (tokens, logsumexp)."""
    scores, _ = matmul(q, k)
    scores = scores * float(alpha)
    lse = torch.logsumexp(scores, dim=-1)
    weights = torch.exp(scores - lse.unsqueeze(-1))
    tokens, _ = matmul(weights, v.detach().cpu().to(torch.float64))
    return tokens, lse


def attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alpha: float, grad_out: torch.Tensor):
    """Backward of `attention` as dfdx's tape runs it, op by op in f64: matmul backward (matmul/cpu_kernel.rs via
    `matmul`'s backward), softmax backward (softmax.rs: y * (g - sum(g * y))), scalar-mul backward, matmul backward.
    Returns (grad_q, grad_k, grad_v) viewed through the operands' strides."""
    scores, bwd_qk = matmul(q, k)
    scores = scores * float(alpha)
    weights = torch.softmax(scores, dim=-1)
    _, bwd_wv = matmul(weights, v.detach().cpu().to(torch.float64))
    g_w, g_v = bwd_wv(grad_out.detach().cpu().to(torch.float64))
    g_scores = weights * (g_w - (g_w * weights).sum(dim=-1, keepdim=True)) * float(alpha)
    g_q, g_k = bwd_qk(g_scores)
    return g_q, g_k, g_v


def softmax(x: torch.Tensor, alpha: float = 1.0):
    """`softmax` over the last axis as dfdx-core/src/tensor_ops/softmax.rs:70-83 computes it (subtract the row maximum,
    exp, divide by the row sum), applied to alpha * x (the scalar multiply MultiHeadAttention puts in front of it,
    multi_head_attention.rs:136-137), in f64.  Returns (y, backward); backward(grad_out) -> grad_x is the chain of the
    tape entries of div, sum, exp and the scalar multiply: alpha * y * (g - sum(g * y))."""
    t = x.detach().cpu().to(torch.float64) * float(alpha)
    t = t - t.max(dim=-1, keepdim=True).values
    e = torch.exp(t)
    y = e / e.sum(dim=-1, keepdim=True)

    def backward(grad_out: torch.Tensor):
        g = grad_out.detach().cpu().to(torch.float64)
        return float(alpha) * y * (g - (g * y).sum(dim=-1, keepdim=True))

    return y, backward


def layer_norm(x: torch.Tensor, gamma: torch.Tensor = None, beta: torch.Tensor = None, eps: float = 1e-5):
    """`normalize::<last axis>(epsilon)` step by step as dfdx-core/src/tensor_ops/normalize.rs:33-50 writes it (mean,
    subtract, square, mean, + epsilon, sqrt, divide), then `* gamma + beta` (dfdx/src/nn/layers/layer_norm1d.rs:87-91),
    in f64.  Returns (y, backward); backward(grad_out) -> (grad_x, grad_gamma, grad_beta)."""
    x64 = x.detach().cpu().to(torch.float64)
    mean = x64.mean(dim=-1, keepdim=True)
    centered = x64 - mean
    std = (centered.square().mean(dim=-1, keepdim=True) + float(eps)).sqrt()
    xhat = centered / std
    g64 = None if gamma is None else gamma.detach().cpu().to(torch.float64)
    y = xhat if g64 is None else xhat * g64
    if beta is not None:
        y = y + beta.detach().cpu().to(torch.float64)

    def backward(grad_out: torch.Tensor):
        go = grad_out.detach().cpu().to(torch.float64)
        gg = go if g64 is None else go * g64
        gx = (gg - gg.mean(dim=-1, keepdim=True) - xhat * (gg * xhat).mean(dim=-1, keepdim=True)) / std
        flat = go.reshape(-1, go.shape[-1])
        return gx, (flat * xhat.reshape(flat.shape)).sum(0), flat.sum(0)

    return y, backward


def rel_frobenius(got: torch.Tensor, want: torch.Tensor) -> float:
    """||got - want||_F / ||want||_F in f64 (0/0 -> 0)."""
    g = got.detach().cpu().to(torch.float64)
    w = want.detach().cpu().to(torch.float64)
    den = torch.linalg.vector_norm(w).item()
    num = torch.linalg.vector_norm(g - w).item()
    return num / den if den > 0 else num
