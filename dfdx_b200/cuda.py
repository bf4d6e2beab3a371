"""Host-side mirror of dfdx's `Cuda` device for the matmul / conv2d path.

The names follow the reference (dfdx v0.13.0): `Cuda.gemm` / `Cuda.gemm_batch`
(dfdx-core/src/tensor_ops/matmul/cuda_kernel.rs:153-237), the four kernel traits
`MatMatKernel`, `MatMatBrKernel`, `MatMatBatch3Kernel`, `MatMatBatch4Kernel` (:240-569), the
rank dispatch of `TryMatMul` (matmul/mod.rs:133-311) and `Conv2DKernel` / `TryConv2D`
(conv2d/mod.rs:31-53,273-324).  Tensors are torch CUDA tensors used purely as device buffers: the
element strides of a torch view are exactly dfdx's `Tensor::strides`, so `permute` / `expand` views
reach the kernels without a copy, like dfdx's zero-copy `permute` / `broadcast`.

Everything computes through the C ABI of libdfdx_b200.so; nothing here calls a torch math op.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import Conv1DOp, Conv2DOp, check, strides as _st

_DTYPES = {torch.float32: _lib.F32, torch.float64: _lib.F64, torch.float16: _lib.F16}


class ShapeMismatch(AssertionError):
    """Raised where the reference panics with `assertion left == right failed` before any launch."""


def _assert_eq(left, right):
    if left != right:
        raise ShapeMismatch(f"left: {left}\n right: {right}")


def conv2d_out_dim(dim: int, kernel: int, stride: int, padding: int, dilation: int) -> int:
    """conv2d/mod.rs:143-161."""
    span = dilation * (kernel - 1) + 1
    if dim + 2 * padding < span:
        raise ShapeMismatch("called `Option::unwrap()` on a `None` value")
    return (dim + 2 * padding - span) // stride + 1


class Cuda:
    """One device ordinal, like `Cuda::try_build(ordinal, seed)` (tensor/cuda/device.rs:72-91)."""

    def __init__(self, ordinal: int = 0, amp: bool = False, par_stream: bool = False):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("dfdx_b200.Cuda needs a CUDA device (there is no CPU fallback)")
        self.ordinal = ordinal
        self.device = torch.device("cuda", ordinal)
        self.amp = amp  # treat float16 as AMP<f16> (same arithmetic here: f32 accumulate either way)
        torch.cuda.set_device(ordinal)
        check(self.lib.b200_init(ordinal), "b200_init")
        self._workspace = None  # grow-only byte workspace (tensor/cuda/device.rs:108-122)
        # dfdx's second stream, forked from the default one (tensor/cuda/device.rs:30,84): when present, the
        # grad_lhs GEMM of every matmul backward runs on it beside the grad_rhs GEMM (matmul/cuda_kernel.rs:282-310)
        self.par_stream = torch.cuda.Stream(self.device) if par_stream else None

    # -- plumbing ---------------------------------------------------------------------------------
    def _dtype(self, t: torch.Tensor) -> int:
        try:
            d = _DTYPES[t.dtype]
        except KeyError:
            raise TypeError(f"unsupported dtype {t.dtype}") from None
        return _lib.AMP_F16 if (d == _lib.F16 and self.amp) else d

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _fork(self):
        """`par_stream.wait_for_default()`: returns the handle to pass as `par_stream` (None without one)."""
        if self.par_stream is None:
            return None
        self.par_stream.wait_stream(torch.cuda.current_stream(self.device))
        return self.par_stream.cuda_stream

    def _join(self) -> None:
        """`dev.wait_for(par_stream)`."""
        if self.par_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.par_stream)

    def get_workspace(self, nbytes: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)
        return self._workspace

    def set_path(self, path: int) -> None:
        check(self.lib.b200_set_path(path), "b200_set_path")

    def device_status(self) -> int:
        return self.lib.b200_device_status(self._stream())

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)
        check(self.device_status(), "device status")

    def alloc_grad(self, t: torch.Tensor) -> torch.Tensor:
        """Zeroed gradient buffer with the PHYSICAL length of t's storage
        (tensor/cuda/device.rs:259-266): a permuted view's gradient lands in the base layout, a
        broadcast view's gradient accumulates."""
        n = t.untyped_storage().nbytes() // t.element_size()
        return torch.zeros(n, dtype=t.dtype, device=t.device)

    @staticmethod
    def grad_view(grad: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        return torch.as_strided(grad, t.shape, t.stride())

    # -- Cuda::gemm / Cuda::gemm_batch --------------------------------------------------------------
    def gemm(self, mkn, lhs, lhs_strides, rhs, rhs_strides, beta, out, out_strides) -> None:
        m, k, n = mkn
        check(self.lib.b200_gemm(self._dtype(out), m, k, n, lhs.data_ptr(), _st(lhs_strides), rhs.data_ptr(),
                                 _st(rhs_strides), float(beta), out.data_ptr(), _st(out_strides), self._stream()),
              "b200_gemm")

    def gemm_batch(self, bmkn, lhs, lhs_strides, rhs, rhs_strides, beta, out, out_strides) -> None:
        b, m, k, n = bmkn
        check(self.lib.b200_gemm_batch(self._dtype(out), b, m, k, n, lhs.data_ptr(), _st(lhs_strides),
                                       rhs.data_ptr(), _st(rhs_strides), float(beta), out.data_ptr(),
                                       _st(out_strides), self._stream()), "b200_gemm_batch")

    # -- kernel traits ------------------------------------------------------------------------------
    def _empty(self, shape, like):
        return torch.empty(shape, dtype=like.dtype, device=like.device)  # alloc_empty: uninitialised

    def matmat_forward(self, lhs, rhs):
        (m, k), n = lhs.shape, rhs.shape[1]
        out = self._empty((m, n), lhs)
        check(self.lib.b200_matmat_forward(self._dtype(lhs), m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                           rhs.data_ptr(), _st(rhs.stride()), out.data_ptr(), self._stream()),
              "b200_matmat_forward")
        return out

    def matmat_backward(self, lhs, grad_lhs, rhs, grad_rhs, grad_out) -> None:
        (m, k), n = lhs.shape, rhs.shape[1]
        par = self._fork()
        check(self.lib.b200_matmat_backward(self._dtype(lhs), m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                            _ptr(grad_lhs), rhs.data_ptr(), _st(rhs.stride()), _ptr(grad_rhs),
                                            grad_out.data_ptr(), self._stream(), par), "b200_matmat_backward")
        self._join()

    def matmat_br_forward(self, lhs, rhs):
        (b, m, k), n = lhs.shape, rhs.shape[1]
        out = self._empty((b, m, n), lhs)
        check(self.lib.b200_matmat_br_forward(self._dtype(lhs), b, m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                              rhs.data_ptr(), _st(rhs.stride()), out.data_ptr(), self._stream()),
              "b200_matmat_br_forward")
        return out

    def matmat_br_backward(self, lhs, grad_lhs, rhs, grad_rhs, grad_out) -> None:
        (b, m, k), n = lhs.shape, rhs.shape[1]
        par = self._fork()
        check(self.lib.b200_matmat_br_backward(self._dtype(lhs), b, m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                               _ptr(grad_lhs), rhs.data_ptr(), _st(rhs.stride()), _ptr(grad_rhs),
                                               grad_out.data_ptr(), self._stream(), par),
              "b200_matmat_br_backward")
        self._join()

    def matmat_br_backward_overwrite(self, lhs, grad_lhs, rhs, grad_rhs, grad_out) -> None:
        """The first accumulation into fresh gradient buffers: they are written, need no zero fill and are not read."""
        (b, m, k), n = lhs.shape, rhs.shape[1]
        check(self.lib.b200_matmat_br_backward_overwrite(self._dtype(lhs), b, m, k, n, lhs.data_ptr(),
                                                         _st(lhs.stride()), _ptr(grad_lhs), rhs.data_ptr(),
                                                         _st(rhs.stride()), _ptr(grad_rhs), grad_out.data_ptr(),
                                                         self._stream()), "b200_matmat_br_backward_overwrite")

    def matmat_br_grad_rhs_f32(self, lhs, grad_out, grad_rhs32) -> None:
        """grad_rhs32 (an f32 (K, N) view, any of the two orientations) += sum_b lhs_b^T . grad_out_b for f16 lhs
        (B, M, K) and a contiguous f16 grad_out (B, M, N): the weight gradient of a broadcast-rhs matmul added in f32
        to an f32 gradient buffer, one launch (`b200_matmat_br_grad_rhs_f32`)."""
        (b, m, k), n = lhs.shape, grad_out.shape[-1]
        _assert_eq(tuple(grad_rhs32.shape), (k, n))
        if grad_rhs32.dtype != torch.float32:
            raise TypeError("grad_rhs32 must be an f32 tensor")
        check(self.lib.b200_matmat_br_grad_rhs_f32(self._dtype(lhs), b, m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                                   grad_out.data_ptr(), grad_rhs32.data_ptr(), _st(grad_rhs32.stride()),
                                                   self._stream()), "b200_matmat_br_grad_rhs_f32")

    def matmat_batch3_forward(self, lhs, rhs):
        (b, m, k), n = lhs.shape, rhs.shape[2]
        out = self._empty((b, m, n), lhs)
        check(self.lib.b200_matmat_batch3_forward(self._dtype(lhs), b, m, k, n, lhs.data_ptr(),
                                                  _st(lhs.stride()), rhs.data_ptr(), _st(rhs.stride()),
                                                  out.data_ptr(), self._stream()), "b200_matmat_batch3_forward")
        return out

    def matmat_batch3_backward(self, lhs, grad_lhs, rhs, grad_rhs, grad_out) -> None:
        (b, m, k), n = lhs.shape, rhs.shape[2]
        par = self._fork()
        check(self.lib.b200_matmat_batch3_backward(self._dtype(lhs), b, m, k, n, lhs.data_ptr(),
                                                   _st(lhs.stride()), _ptr(grad_lhs), rhs.data_ptr(),
                                                   _st(rhs.stride()), _ptr(grad_rhs), grad_out.data_ptr(),
                                                   self._stream(), par), "b200_matmat_batch3_backward")
        self._join()

    def matmat_batch4_forward(self, lhs, rhs):
        (b, s, m, k), n = lhs.shape, rhs.shape[3]
        out = self._empty((b, s, m, n), lhs)
        check(self.lib.b200_matmat_batch4_forward(self._dtype(lhs), b, s, m, k, n, lhs.data_ptr(),
                                                  _st(lhs.stride()), rhs.data_ptr(), _st(rhs.stride()),
                                                  out.data_ptr(), self._stream()), "b200_matmat_batch4_forward")
        return out

    def matmat_batch4_backward(self, lhs, grad_lhs, rhs, grad_rhs, grad_out) -> None:
        (b, s, m, k), n = lhs.shape, rhs.shape[3]
        par = self._fork()
        check(self.lib.b200_matmat_batch4_backward(self._dtype(lhs), b, s, m, k, n, lhs.data_ptr(),
                                                   _st(lhs.stride()), _ptr(grad_lhs), rhs.data_ptr(),
                                                   _st(rhs.stride()), _ptr(grad_rhs), grad_out.data_ptr(),
                                                   self._stream(), par), "b200_matmat_batch4_backward")

    # -- fused epilogues (API additions) -------------------------------------------------------------
        self._join()

    def gemm_batch_fused(self, lhs, rhs, out, alpha=1.0, bias=None, relu=False) -> None:
        """out[b0,b1] = act(alpha * lhs[b0,b1] @ rhs[b0,b1] + bias) for rank-4 views (batch strides of lhs / rhs
        may be 0); one launch, `out` is only written."""
        (b0, b1, m, k), n = lhs.shape, rhs.shape[3]
        _assert_eq(tuple(rhs.shape[:3]), (b0, b1, k))
        ep = _lib.Epilogue(float(alpha), _ptr(bias), _lib.ACT_RELU if relu else _lib.ACT_NONE)
        check(self.lib.b200_gemm_batch_fused(self._dtype(lhs), b0, b1, m, k, n, lhs.data_ptr(), _st(lhs.stride()),
                                             rhs.data_ptr(), _st(rhs.stride()), ep, out.data_ptr(),
                                             _st(out.stride()), self._stream()), "b200_gemm_batch_fused")

    def linear_forward(self, x, weight_view, bias=None, relu=False):
        """`Linear::try_forward` (+ optional ReLU) in one launch: x (B, S, I), weight_view the (I, O) view of the
        stored (O, I) weight, bias (O,) -> (B, S, O)."""
        (b, m, i), o = x.shape, weight_view.shape[1]
        _assert_eq(weight_view.shape[0], i)
        if bias is not None:
            _assert_eq(tuple(bias.shape), (o,))
        out = self._empty((b, m, o), x)
        check(self.lib.b200_linear_forward(self._dtype(x), b, m, i, o, x.data_ptr(), _st(x.stride()),
                                           weight_view.data_ptr(), _st(weight_view.stride()), _ptr(bias),
                                           _lib.ACT_RELU if relu else _lib.ACT_NONE, out.data_ptr(),
                                           self._stream()), "b200_linear_forward")
        return out

    def matmat_batch4_forward_scaled(self, lhs, rhs, alpha: float):
        """`q.matmul(k) * scalar` (multi_head_attention.rs:136-137) in one launch."""
        (b, s, m, k), n = lhs.shape, rhs.shape[3]
        _assert_eq(tuple(rhs.shape[:3]), (b, s, k))
        out = self._empty((b, s, m, n), lhs)
        check(self.lib.b200_matmat_batch4_forward_scaled(self._dtype(lhs), b, s, m, k, n, lhs.data_ptr(),
                                                         _st(lhs.stride()), rhs.data_ptr(), _st(rhs.stride()),
                                                         float(alpha), out.data_ptr(), self._stream()),
              "b200_matmat_batch4_forward_scaled")
        return out

    def attention_forward(self, q, k, v, alpha: float, out=None, want_lse: bool = False):
        """softmax(q.matmul(k) * alpha).matmul(v) in one kernel (multi_head_attention.rs:136-141).
        q (B,H,S1,D), k (B,H,D,S2), v (B,H,S2,D) views with unit stride along D.  `out` defaults to a
        (B,S1,H,D) buffer viewed as (B,H,S1,D), i.e. already in the layout the output projection reads.
        Returns (out, lse or None)."""
        b, h, s1, d = q.shape
        s2 = k.shape[3]
        _assert_eq(tuple(k.shape), (b, h, d, s2))
        _assert_eq(tuple(v.shape), (b, h, s2, d))
        if out is None:
            out = self._empty((b, s1, h, d), q).permute(0, 2, 1, 3)
        lse = torch.empty((b, h, s1), dtype=torch.float32, device=q.device) if want_lse else None
        check(self.lib.b200_attention_forward(self._dtype(q), b, h, s1, s2, d, q.data_ptr(), _st(q.stride()),
                                              k.data_ptr(), _st(k.stride()), v.data_ptr(), _st(v.stride()),
                                              float(alpha), out.data_ptr(), _st(out.stride()), _ptr(lse),
                                              self._stream()), "b200_attention_forward")
        return out, lse

    def attention_backward(self, q, k, v, alpha: float, out, lse, grad_out, accumulate_into=None, write_into=None):
        """Gradients of `attention_forward`.  Returns (grad_q, grad_k, grad_v) viewed through q's, k's and v's
        strides (zeroed buffers of the storages' physical length, as `Gradients::try_alloc_for` makes them),
        accumulates into the three given flat buffers, or writes into three given views shaped like q, k and v
        (`write_into`; their strides may differ from q's, k's and v's)."""
        b, h, s1, d = q.shape
        s2 = k.shape[3]
        if write_into is not None:
            gq, gk, gv = write_into
            if (gq.shape, gk.shape, gv.shape) != (q.shape, k.shape, v.shape):
                raise ValueError("write_into: views shaped like q, k and v are required")
            go = grad_out if grad_out.stride(3) == 1 else grad_out.contiguous()
            ws = self.get_workspace(self.lib.b200_attention_backward_workspace_bytes(b, h, s1))
            check(self.lib.b200_attention_backward(
                self._dtype(q), b, h, s1, s2, d, q.data_ptr(), _st(q.stride()), k.data_ptr(), _st(k.stride()),
                v.data_ptr(), _st(v.stride()), float(alpha), out.data_ptr(), _st(out.stride()), lse.data_ptr(),
                go.data_ptr(), _st(go.stride()), gq.data_ptr(), _st(gq.stride()), gk.data_ptr(), _st(gk.stride()),
                gv.data_ptr(), _st(gv.stride()), 0, ws.data_ptr(), ws.numel(), self._stream()), "b200_attention_backward")
            return gq, gk, gv
        # Fresh buffers are simply written (no zero fill, no read-modify-write) when every element of q, k and v
        # owns its storage element and the views cover their storages; a broadcast view (several elements aliasing
        # one storage element) or a partial view keeps dfdx's zero-then-accumulate.
        dense = all(st != 0 for t in (q, k, v) for st in t.stride()) and \
            all(t.numel() * t.element_size() == t.untyped_storage().nbytes() for t in (q, k, v))
        acc = 0 if (accumulate_into is None and dense) else 1
        if accumulate_into is not None:
            gq, gk, gv = accumulate_into
        elif acc == 0:
            gq, gk, gv = (torch.empty(t.untyped_storage().nbytes() // t.element_size(), dtype=t.dtype, device=t.device)
                          for t in (q, k, v))
        else:
            gq, gk, gv = self.alloc_grad(q), self.alloc_grad(k), self.alloc_grad(v)
        go = grad_out if grad_out.stride(3) == 1 else grad_out.contiguous()
        need = self.lib.b200_attention_backward_workspace_bytes(b, h, s1)
        ws = self.get_workspace(need)
        check(self.lib.b200_attention_backward(
            self._dtype(q), b, h, s1, s2, d, q.data_ptr(), _st(q.stride()), k.data_ptr(), _st(k.stride()),
            v.data_ptr(), _st(v.stride()), float(alpha), out.data_ptr(), _st(out.stride()), lse.data_ptr(),
            go.data_ptr(), _st(go.stride()), gq.data_ptr(), _st(q.stride()), gk.data_ptr(), _st(k.stride()),
            gv.data_ptr(), _st(v.stride()), acc, ws.data_ptr(), ws.numel(), self._stream()), "b200_attention_backward")
        return self.grad_view(gq, q), self.grad_view(gk, k), self.grad_view(gv, v)

    # -- row-wise neighbours of the GEMMs ---------------------------------------------------------------
    def layer_norm_forward(self, x, gamma=None, beta=None, eps: float = 1e-5, want_stats: bool = False):
        """`LayerNorm1D::try_forward` over the last axis of a contiguous tensor.  Returns (y, stats or None)."""
        cols = x.shape[-1]
        rows = x.numel() // max(cols, 1)
        y = self._empty(tuple(x.shape), x)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=x.device) if want_stats else None
        check(self.lib.b200_layer_norm_forward(self._dtype(x), rows, cols, x.data_ptr(), cols, _ptr(gamma), _ptr(beta),
                                               float(eps), y.data_ptr(), cols, _ptr(stats), self._stream()),
              "b200_layer_norm_forward")
        return y, stats

    def layer_norm_backward(self, x, gamma, stats, grad_out, grad_gamma=None, grad_beta=None):
        """Returns grad_x; adds the f32 column sums into grad_gamma / grad_beta (f32 tensors of `cols` elements)."""
        cols = x.shape[-1]
        rows = x.numel() // max(cols, 1)
        gx = self._empty(tuple(x.shape), x)
        check(self.lib.b200_layer_norm_backward(self._dtype(x), rows, cols, x.data_ptr(), cols, _ptr(gamma),
                                                stats.data_ptr(), grad_out.data_ptr(), cols, gx.data_ptr(), cols, 0,
                                                _ptr(grad_gamma), _ptr(grad_beta), self._stream()),
              "b200_layer_norm_backward")
        return gx

    def layer_norm_backward_sum(self, x, gamma, stats, grad_out, grad_gamma, grad_beta, grad_x_sum):
        """`layer_norm_backward` that also adds the column sums of the grad_x it returns into grad_x_sum (f32, `cols`
        elements): the bias gradient of a Linear whose output reached this LayerNorm through a residual add."""
        cols = x.shape[-1]
        rows = x.numel() // max(cols, 1)
        gx = self._empty(tuple(x.shape), x)
        check(self.lib.b200_layer_norm_backward_sum(self._dtype(x), rows, cols, x.data_ptr(), cols, _ptr(gamma),
                                                    stats.data_ptr(), grad_out.data_ptr(), cols, gx.data_ptr(), cols,
                                                    _ptr(grad_gamma), _ptr(grad_beta), grad_x_sum.data_ptr(),
                                                    self._stream()), "b200_layer_norm_backward_sum")
        return gx

    def add_layer_norm_forward(self, a, b, gamma=None, beta=None, eps: float = 1e-5):
        """`LayerNorm1D(a + b)` (ResidualAdd followed by the norm) in one kernel.  Returns (y, a + b, stats)."""
        cols = a.shape[-1]
        rows = a.numel() // max(cols, 1)
        _assert_eq(tuple(a.shape), tuple(b.shape))
        total, y = self._empty(tuple(a.shape), a), self._empty(tuple(a.shape), a)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=a.device)
        check(self.lib.b200_add_layer_norm_forward(self._dtype(a), rows, cols, a.data_ptr(), cols, b.data_ptr(), cols,
                                                   total.data_ptr(), cols, _ptr(gamma), _ptr(beta), float(eps),
                                                   y.data_ptr(), cols, stats.data_ptr(), self._stream()),
              "b200_add_layer_norm_forward")
        return y, total, stats

    def relu_backward_bias_grad(self, y, grad, grad_bias=None) -> None:
        """In place: grad = grad where y > 0 else 0 (ReLU's backward); grad_bias (f32) += column sums of the result."""
        cols = y.shape[-1]
        rows = y.numel() // max(cols, 1)
        _assert_eq(tuple(y.shape), tuple(grad.shape))
        check(self.lib.b200_relu_backward_bias_grad(self._dtype(y), rows, cols, y.data_ptr(), cols, grad.data_ptr(), cols,
                                                    _ptr(grad_bias), self._stream()), "b200_relu_backward_bias_grad")

    def softmax_forward(self, x, alpha: float = 1.0, out=None):
        """`(x * alpha).softmax::<last axis>()` (softmax.rs:36-84) in one pass; x (..., cols) with a unit last stride."""
        x2 = x.reshape(-1, x.shape[-1])
        y = self._empty(x2.shape, x) if out is None else out.reshape(x2.shape)
        check(self.lib.b200_softmax_forward(self._dtype(x), x2.shape[0], x2.shape[1], x2.data_ptr(), x2.stride(0), float(alpha),
                                            y.data_ptr(), y.stride(0), self._stream()), "b200_softmax_forward")
        return y.reshape(x.shape)

    def softmax_backward(self, y, grad_out, alpha: float = 1.0, accumulate_into=None):
        """grad_x (+)= alpha * y * (grad_out - sum(grad_out * y)) over the last axis."""
        y2, g2 = y.reshape(-1, y.shape[-1]), grad_out.reshape(-1, y.shape[-1])
        gx = self._empty(y2.shape, y) if accumulate_into is None else accumulate_into.reshape(y2.shape)
        check(self.lib.b200_softmax_backward(self._dtype(y), y2.shape[0], y2.shape[1], y2.data_ptr(), y2.stride(0), g2.data_ptr(),
                                             g2.stride(0), float(alpha), gx.data_ptr(), gx.stride(0),
                                             0 if accumulate_into is None else 1, self._stream()), "b200_softmax_backward")
        return gx.reshape(y.shape)

    def bias_grad(self, grad_out, grad_bias) -> None:
        """grad_bias (f32, `cols` elements) += column sums of the contiguous (..., cols) tensor grad_out."""
        cols = grad_out.shape[-1]
        rows = grad_out.numel() // max(cols, 1)
        check(self.lib.b200_bias_grad(self._dtype(grad_out), rows, cols, grad_out.data_ptr(), cols, grad_bias.data_ptr(),
                                      self._stream()), "b200_bias_grad")

    # -- TryMatMul (matmul/mod.rs:133-311) ---------------------------------------------------------
    def matmul(self, lhs: torch.Tensor, rhs: torch.Tensor):
        """Rank dispatch of `TryMatMul`.  Returns (out, backward) where
        `backward(grad_out) -> (grad_lhs, grad_rhs)` runs the trait's backward into freshly zeroed
        gradient buffers and returns them viewed through the operands' strides."""
        ld, rd = lhs.dim(), rhs.dim()
        if ld == 1 and rd == 1:       # outer product: (M,) x (N,) -> (M,1) x (1,N)   (mod.rs:139-158)
            l2 = torch.as_strided(lhs, (lhs.shape[0], 1), (lhs.stride(0), 1))
            r2 = torch.as_strided(rhs, (1, rhs.shape[0]), (rhs.shape[0], rhs.stride(0)))
            return self._traced(self.matmat_forward, self.matmat_backward, l2, r2, lhs, rhs, None)
        if ld == 1 and rd == 2:       # (K,) x (K,N) -> (N,)                            (mod.rs:160-174)
            _assert_eq(lhs.shape[0], rhs.shape[0])
            l2 = torch.as_strided(lhs, (1, lhs.shape[0]), (lhs.shape[0], lhs.stride(0)))
            return self._traced(self.matmat_forward, self.matmat_backward, l2, rhs, lhs, rhs, (rhs.shape[1],))
        if ld == 2 and rd == 1:       # (M,K) x (K,) -> (M,)                            (mod.rs:176-189)
            _assert_eq(lhs.shape[1], rhs.shape[0])
            r2 = torch.as_strided(rhs, (rhs.shape[0], 1), (rhs.stride(0), 1))
            return self._traced(self.matmat_forward, self.matmat_backward, lhs, r2, lhs, rhs, (lhs.shape[0],))
        if ld == 2 and rd == 2:
            _assert_eq(lhs.shape[1], rhs.shape[0])
            return self._traced(self.matmat_forward, self.matmat_backward, lhs, rhs, lhs, rhs, None)
        if ld == 3 and rd == 2:
            _assert_eq(lhs.shape[2], rhs.shape[0])
            return self._traced(self.matmat_br_forward, self.matmat_br_backward, lhs, rhs, lhs, rhs, None)
        if ld == 3 and rd == 3:
            _assert_eq(lhs.shape[0], rhs.shape[0])
            _assert_eq(lhs.shape[2], rhs.shape[1])
            return self._traced(self.matmat_batch3_forward, self.matmat_batch3_backward, lhs, rhs, lhs, rhs, None)
        if ld == 4 and rd == 4:
            _assert_eq(lhs.shape[0], rhs.shape[0])
            _assert_eq(lhs.shape[1], rhs.shape[1])
            _assert_eq(lhs.shape[3], rhs.shape[2])
            return self._traced(self.matmat_batch4_forward, self.matmat_batch4_backward, lhs, rhs, lhs, rhs, None)
        raise TypeError(f"matmul is not defined for ranks {ld} x {rd}")

    def _traced(self, fwd, bwd, l, r, l_orig, r_orig, out_shape):
        out = fwd(l, r)
        shaped = out if out_shape is None else out.reshape(out_shape)

        def backward(grad_out: torch.Tensor):
            go = grad_out.reshape(out.shape).contiguous()
            gl, gr = self.alloc_grad(l_orig), self.alloc_grad(r_orig)
            bwd(l, gl, r, gr, go)
            return self.grad_view(gl, l_orig), self.grad_view(gr, r_orig)

        return shaped, backward

    # -- Conv2DKernel / TryConv2D (conv2d/mod.rs:273-324) -----------------------------------------
    def conv2d_op(self, img, filters, stride, padding, dilation, groups) -> Conv2DOp:
        b, c, h, w = img.shape
        o, cg, k, k2 = filters.shape
        _assert_eq(c, cg * groups)
        _assert_eq(k, k2)
        if o % groups:
            raise ShapeMismatch("assertion failed: out_chan.size() % groups.size() == 0")
        return Conv2DOp(kernel=k, stride=stride, padding=padding, dilation=dilation, groups=groups, batch=b,
                        chan_in=c, chan_out=o, h_in=h, h_out=conv2d_out_dim(h, k, stride, padding, dilation),
                        w_in=w, w_out=conv2d_out_dim(w, k, stride, padding, dilation))

    def conv2d_forward(self, op: Conv2DOp, img, filters, out) -> None:
        dt = self._dtype(img)
        need = self.lib.b200_conv2d_workspace_bytes(dt, op, 0)
        ws = self.get_workspace(need)
        check(self.lib.b200_conv2d_forward(dt, op, img.data_ptr(), _st(img.stride()), filters.data_ptr(),
                                           out.data_ptr(), ws.data_ptr(), ws.numel(), self._stream()),
              "b200_conv2d_forward")

    def conv2d_backward(self, op: Conv2DOp, img, grad_img, filters, grad_filters, grad_out) -> None:
        dt = self._dtype(img)
        need = self.lib.b200_conv2d_workspace_bytes(dt, op, 1)
        ws = self.get_workspace(need)
        check(self.lib.b200_conv2d_backward(dt, op, img.data_ptr(), _ptr(grad_img), filters.data_ptr(),
                                            _st(filters.stride()), _ptr(grad_filters), grad_out.data_ptr(),
                                            ws.data_ptr(), ws.numel(), self._stream(), None),
              "b200_conv2d_backward")

    def conv2d(self, img, filters, stride=1, padding=0, dilation=1, groups=1):
        """`(img, filters).conv2d(stride, padding, dilation, groups)`; 3-D images are batch 1
        (conv2d/mod.rs:216-222).  Returns (out, backward)."""
        squeeze = img.dim() == 3
        x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
        if not x.is_contiguous() or not filters.is_contiguous():
            raise ShapeMismatch("Image & filter inputs to conv2d must be contiguous")
        op = self.conv2d_op(x, filters, stride, padding, dilation, groups)
        out = self._empty((op.batch, op.chan_out, op.h_out, op.w_out), x)
        self.conv2d_forward(op, x, filters, out)

        def backward(grad_out: torch.Tensor):
            go = grad_out.reshape(out.shape).contiguous()
            gx, gw = self.alloc_grad(x), self.alloc_grad(filters)
            self.conv2d_backward(op, x, gx, filters, gw, go)
            return self.grad_view(gx, x).reshape(img.shape), self.grad_view(gw, filters)

        return (out[0] if squeeze else out), backward


def _ptr(t):
    return None if t is None else t.data_ptr()


def _conv1d(self, img, filters, stride=1, padding=0, dilation=1, groups=1):
    """`(img, filters).conv1d(stride, padding, dilation, groups)` (conv1d/mod.rs:160-286); 2-D images are batch 1.
    Returns (out, backward)."""
    squeeze = img.dim() == 2
    x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
    if not x.is_contiguous() or not filters.is_contiguous():
        raise ShapeMismatch("Image & filter inputs to conv1d must be contiguous")
    b, c, l = x.shape
    o, cg, k = filters.shape
    _assert_eq(c, cg * groups)
    if o % groups:
        raise ShapeMismatch("assertion failed: out_chan.size() % groups.size() == 0")
    op = Conv1DOp(kernel=k, stride=stride, padding=padding, dilation=dilation, groups=groups, batch=b, chan_in=c,
                  chan_out=o, l_in=l, l_out=conv2d_out_dim(l, k, stride, padding, dilation))
    dt = self._dtype(x)
    out = self._empty((b, o, op.l_out), x)
    ws = self.get_workspace(self.lib.b200_conv1d_workspace_bytes(dt, op, 0))
    check(self.lib.b200_conv1d_forward(dt, op, x.data_ptr(), _st(x.stride()), filters.data_ptr(), out.data_ptr(),
                                       ws.data_ptr(), ws.numel(), self._stream()), "b200_conv1d_forward")

    def backward(grad_out: torch.Tensor):
        go = grad_out.reshape(out.shape).contiguous()
        gx, gw = self.alloc_grad(x), self.alloc_grad(filters)
        wsb = self.get_workspace(self.lib.b200_conv1d_workspace_bytes(dt, op, 1))
        check(self.lib.b200_conv1d_backward(dt, op, x.data_ptr(), gx.data_ptr(), filters.data_ptr(),
                                            _st(filters.stride()), gw.data_ptr(), go.data_ptr(), wsb.data_ptr(),
                                            wsb.numel(), self._stream(), None), "b200_conv1d_backward")
        return self.grad_view(gx, x).reshape(img.shape), self.grad_view(gw, filters)

    return (out[0] if squeeze else out), backward


def convtrans2d_out_dim(dim: int, kernel: int, stride: int, padding: int, dilation: int) -> int:
    """convtrans2d/mod.rs:108-121."""
    full = (dim - 1) * stride + dilation * (kernel - 1) + 1
    if full < 2 * padding:
        raise ShapeMismatch("called `Option::unwrap()` on a `None` value")
    return full - 2 * padding


def _convtrans2d(self, img, filters, stride=1, padding=0, dilation=1, groups=1):
    """`(img, filters).convtrans2d(stride, padding, dilation, groups)` (convtrans2d/mod.rs:124-280): img (B,C,H,W) or
    (C,H,W), filters (C, O/G, K, K).  Returns (out, backward)."""
    squeeze = img.dim() == 3
    x = img.reshape((1,) + tuple(img.shape)) if squeeze else img
    if not x.is_contiguous() or not filters.is_contiguous():
        raise ShapeMismatch("Image & filter inputs to conv2d must be contiguous")
    b, c, h, w = x.shape
    c2, og, k, k2 = filters.shape
    _assert_eq(c, c2)
    _assert_eq(k, k2)
    op = Conv2DOp(kernel=k, stride=stride, padding=padding, dilation=dilation, groups=groups, batch=b, chan_in=c,
                  chan_out=og * groups, h_in=h, h_out=convtrans2d_out_dim(h, k, stride, padding, dilation), w_in=w,
                  w_out=convtrans2d_out_dim(w, k, stride, padding, dilation))
    dt = self._dtype(x)
    out = self._empty((b, op.chan_out, op.h_out, op.w_out), x)
    ws = self.get_workspace(self.lib.b200_convtrans2d_workspace_bytes(dt, op, 0))
    check(self.lib.b200_convtrans2d_forward(dt, op, x.data_ptr(), filters.data_ptr(), _st(filters.stride()),
                                            out.data_ptr(), ws.data_ptr(), ws.numel(), self._stream()),
          "b200_convtrans2d_forward")

    def backward(grad_out: torch.Tensor):
        go = grad_out.reshape(out.shape).contiguous()
        gx, gw = self.alloc_grad(x), self.alloc_grad(filters)
        wsb = self.get_workspace(self.lib.b200_convtrans2d_workspace_bytes(dt, op, 1))
        check(self.lib.b200_convtrans2d_backward(dt, op, x.data_ptr(), gx.data_ptr(), filters.data_ptr(),
                                                 _st(filters.stride()), gw.data_ptr(), go.data_ptr(), wsb.data_ptr(),
                                                 wsb.numel(), self._stream(), None), "b200_convtrans2d_backward")
        return self.grad_view(gx, x).reshape(img.shape), self.grad_view(gw, filters)

    return (out[0] if squeeze else out), backward


Cuda.conv1d = _conv1d
Cuda.convtrans2d = _convtrans2d
