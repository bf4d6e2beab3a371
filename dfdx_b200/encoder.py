"""Transformer-encoder training step whose matrix multiplications all run on this library.

This is a measurement harness for benchmark configuration 5, not a re-implementation of dfdx's nn
stack: the block structure restates dfdx's `EncoderBlock` (dfdx/src/nn/layers/transformer.rs:24-47:
ResidualAdd(MultiHeadAttention) -> LayerNorm1D -> ResidualAdd(Linear, ReLU, Linear) -> LayerNorm1D)
and `MultiHeadAttention::try_forward` (multi_head_attention.rs:105-146: three Linear layers, the
(b,s,h,d) buffers viewed as (b,h,s,d) / (b,h,d,s) without a copy, q.matmul(k) * 1/sqrt(d), softmax,
.matmul(v), permute back, output Linear).  Every `matmul` goes through `dfdx_b200.Cuda`
(`MatMatBrKernel` for the Linear layers, `MatMatBatch4Kernel` for the attention products, forward and
backward).  With `fused="attention"` the whole scores / softmax / weighted-sum sequence additionally runs as the
fused attention kernels.  With `fused=True` (default) the ops that directly follow a GEMM in the forward pass — Linear's
bias add, the feed-forward ReLU, the 1/sqrt(d) scale of the scores — run in that GEMM's epilogue
(`b200_linear_forward`, `b200_matmat_batch4_forward_scaled`); with `fused=False` they are separate torch
ops, as they are separate kernels in dfdx; any fused mode also runs LayerNorm (forward and backward), the bias
gradient and, where attention is not one fused kernel (f32, head sizes the fused kernel does not serve), the softmax
on this library's row-wise kernels.  Residual adds, the MSE loss and Adam are plain torch ops either way.

Parameters are f32 master weights; each step computes in f16 (`AMP<f16>`-like: f16 storage, f32
accumulation inside the GEMMs) and Adam updates the f32 masters.  A `Trainer` keeps masters, f16 compute copies
and gradients in flat buffers and, in the fused modes, has the backward ops write parameter gradients straight
into them (dfdx's tape writes into `Gradients` storage the same way); modules used on their own take torch
autograd's route.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .cuda import Cuda


class _MatMul(torch.autograd.Function):
    """`TryMatMul` with its tape entry: forward through the kernel trait's forward, backward through its
    backward (gradients come back viewed through the operands' own strides, as dfdx stores them)."""

    @staticmethod
    def forward(ctx, dev: Cuda, lhs: torch.Tensor, rhs: torch.Tensor):
        if lhs.storage_offset() or not _dense(lhs):
            lhs = lhs.contiguous()
        if rhs.storage_offset() or not _dense(rhs):
            rhs = rhs.contiguous()
        out, bwd = dev.matmul(lhs, rhs)
        ctx.bwd = bwd
        return out

    @staticmethod
    def backward(ctx, grad_out):
        gl, gr = ctx.bwd(grad_out)
        return None, gl, gr


def _dense(t: torch.Tensor) -> bool:
    """True when t is a permutation of a contiguous buffer that starts at its storage's origin."""
    return t.numel() * t.element_size() == t.untyped_storage().nbytes()


def matmul(dev: Cuda, lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    return _MatMul.apply(dev, lhs, rhs)


class _FusedLinear(torch.autograd.Function):
    """`Linear` (+ optional ReLU) with the bias add and the activation done in the GEMM's epilogue
    (`b200_linear_forward`): one launch and one pass over the output where the unfused path runs three.
    Backward: ReLU's mask and the bias gradient (a column sum) are torch ops, the two GEMMs are
    `MatMatBrKernel::backward`."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, weight, bias, relu: bool):
        if x.storage_offset() or not _dense(x):
            x = x.contiguous()
        w_view = weight.permute(1, 0)                              # (O, I) stored, (I, O) consumed
        y = dev.linear_forward(x, w_view, bias, relu)
        ctx.dev, ctx.relu = dev, relu
        ctx.save_for_backward(x, weight, y if relu else None)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, y = ctx.saved_tensors
        dev, w_view = ctx.dev, weight.permute(1, 0)
        g = grad_out.contiguous()
        if ctx.relu:
            g = torch.ops.aten.threshold_backward(g, y, 0.0)
        # fresh gradient buffers: written by the first (and here only) backward op, no zero fill needed
        gx = torch.empty(x.untyped_storage().nbytes() // x.element_size(), dtype=x.dtype, device=x.device)
        gw = torch.empty(weight.numel(), dtype=weight.dtype, device=weight.device)
        dev.matmat_br_backward_overwrite(x, gx, w_view, gw, g)
        grad_bias = torch.zeros(g.shape[-1], dtype=torch.float32, device=g.device)
        dev.bias_grad(g, grad_bias)                                # f32 column sums, one pass over g
        grad_bias = grad_bias.to(g.dtype)
        return None, dev.grad_view(gx, x), gw.view_as(weight), grad_bias, None


class _Softmax(torch.autograd.Function):
    """softmax over the last axis on this library's row-wise kernels (`b200_softmax_forward` / `_backward`): one pass
    each way where dfdx's op sequence (softmax.rs:36-84) runs five kernels forward."""

    @staticmethod
    def forward(ctx, dev: Cuda, scores):
        y = dev.softmax_forward(scores.contiguous())
        ctx.dev = dev
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        (y,) = ctx.saved_tensors
        return None, ctx.dev.softmax_backward(y, grad_out.contiguous())


class _ScaledMatMul(torch.autograd.Function):
    """`q.matmul(k) * alpha` with the scale in the GEMM's epilogue (`b200_matmat_batch4_forward_scaled`)."""

    @staticmethod
    def forward(ctx, dev: Cuda, lhs, rhs, alpha: float):
        if lhs.storage_offset() or not _dense(lhs):
            lhs = lhs.contiguous()
        if rhs.storage_offset() or not _dense(rhs):
            rhs = rhs.contiguous()
        ctx.dev, ctx.alpha = dev, alpha
        ctx.save_for_backward(lhs, rhs)
        return dev.matmat_batch4_forward_scaled(lhs, rhs, alpha)

    @staticmethod
    def backward(ctx, grad_out):
        lhs, rhs = ctx.saved_tensors
        dev = ctx.dev
        g = (grad_out * ctx.alpha).contiguous()
        gl, gr = dev.alloc_grad(lhs), dev.alloc_grad(rhs)
        dev.matmat_batch4_backward(lhs, gl, rhs, gr, g)
        return None, dev.grad_view(gl, lhs), dev.grad_view(gr, rhs), None


class _FusedAttention(torch.autograd.Function):
    """softmax(q.matmul(k) * alpha).matmul(v) as one forward kernel and three backward launches
    (`b200_attention_forward` / `b200_attention_backward`): the (batch, heads, S, S) score tensor never reaches
    HBM, and the output is written straight in the (batch, S, heads * d) layout the output projection reads."""

    @staticmethod
    def forward(ctx, dev: Cuda, q, k, v, alpha: float):
        out, lse = dev.attention_forward(q, k, v, alpha, want_lse=True)
        ctx.dev, ctx.alpha = dev, alpha
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, lse = ctx.saved_tensors
        gq, gk, gv = ctx.dev.attention_backward(q, k, v, ctx.alpha, out, lse, grad_out)
        return None, gq, gk, gv, None


def _split_qkv(qkv: torch.Tensor, heads: int):
    """The q (b, h, s, d), k (b, h, d, s) and v (b, h, s, d) views of a (b, s, 3 * h * d) projection output."""
    m = qkv.shape[-1] // 3
    d = m // heads
    q = qkv[..., :m].unflatten(-1, (heads, d)).permute(0, 2, 1, 3)
    k = qkv[..., m:2 * m].unflatten(-1, (heads, d)).permute(0, 2, 3, 1)
    v = qkv[..., 2 * m:].unflatten(-1, (heads, d)).permute(0, 2, 1, 3)
    return q, k, v


class _FusedAttentionQKV(torch.autograd.Function):
    """`_FusedAttention` on the output of one (model -> 3 * model) projection, i.e. w_q, w_k and w_v applied as one
    GEMM over their adjacent weights: q, k and v are strided views of that output, and the backward kernels write
    their three gradients into the matching views of one buffer, so that the projection's backward is one data
    gradient GEMM, one weight gradient GEMM and one bias column sum instead of three of each plus two adds."""

    @staticmethod
    def forward(ctx, dev: Cuda, qkv, heads: int, alpha: float):
        q, k, v = _split_qkv(qkv, heads)
        out, lse = dev.attention_forward(q, k, v, alpha, want_lse=True)
        ctx.dev, ctx.alpha, ctx.heads = dev, alpha, heads
        ctx.save_for_backward(qkv, out, lse)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        qkv, out, lse = ctx.saved_tensors
        q, k, v = _split_qkv(qkv, ctx.heads)
        gqkv = torch.empty_like(qkv)
        ctx.dev.attention_backward(q, k, v, ctx.alpha, out, lse, grad_out, write_into=_split_qkv(gqkv, ctx.heads))
        return None, gqkv, None, None


class _LayerNorm(torch.autograd.Function):
    """`LayerNorm1D` as one forward and one backward kernel (`b200_layer_norm_forward` / `_backward`); gamma and beta
    are the f16 compute copies, their gradients come back as f32 column sums."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, gamma, beta, eps: float):
        x = x.contiguous()
        y, stats = dev.layer_norm_forward(x, gamma, beta, eps, want_stats=True)
        ctx.dev = dev
        ctx.save_for_backward(x, gamma, stats)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        x, gamma, stats = ctx.saved_tensors
        gg = torch.zeros(gamma.shape, dtype=torch.float32, device=x.device)
        gb = torch.zeros(gamma.shape, dtype=torch.float32, device=x.device)
        gx = ctx.dev.layer_norm_backward(x, gamma, stats, grad_out.contiguous(), gg, gb)
        return None, gx, gg.to(gamma.dtype), gb.to(gamma.dtype), None


class _DirectLinear(torch.autograd.Function):
    """`_FusedLinear` for parameters held in a trainer's flat buffers, with the gradients written the way dfdx's tape
    does it: straight into the parameter's gradient storage (`Gradients::get_or_alloc_mut`), not returned to
    an autograd engine that would copy, cast and add them.  `slot` = (f16 weight, f16 bias, f16 weight-gradient
    buffer, f32 bias-gradient buffer); the weight gradient is overwritten (each parameter is used once per
    step), the bias gradient is added into its zeroed f32 slot."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, slot, relu: bool):
        if x.storage_offset() or not _dense(x):
            x = x.contiguous()
        y = dev.linear_forward(x, slot[0].permute(1, 0), slot[1], relu)
        ctx.dev, ctx.relu, ctx.slot = dev, relu, slot
        ctx.save_for_backward(x, y if relu else None)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        x, y = ctx.saved_tensors
        dev, (w16, _, gw16, gb32) = ctx.dev, ctx.slot[:4]
        g = grad_out.contiguous()
        if ctx.relu:
            g = torch.ops.aten.threshold_backward(g, y, 0.0)
        gx = torch.empty(x.untyped_storage().nbytes() // x.element_size(), dtype=x.dtype, device=x.device)
        dev.matmat_br_backward_overwrite(x, gx, w16.permute(1, 0), gw16, g)
        dev.bias_grad(g, gb32)
        return None, dev.grad_view(gx, x), None, None


class _DirectLayerNorm(torch.autograd.Function):
    """`_LayerNorm` with gamma's and beta's gradients added straight into their f32 gradient slots.
    `slot` = (f16 gamma, f16 beta, f32 gamma-gradient buffer, f32 beta-gradient buffer)."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, slot, eps: float):
        x = x.contiguous()
        y, stats = dev.layer_norm_forward(x, slot[0], slot[1], eps, want_stats=True)
        ctx.dev, ctx.slot = dev, slot
        ctx.save_for_backward(x, stats)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        x, stats = ctx.saved_tensors
        g16, _, gg32, gb32 = ctx.slot
        return None, ctx.dev.layer_norm_backward(x, g16, stats, grad_out.contiguous(), gg32, gb32), None, None


def _weight_grad(dev: Cuda, x, slot, g) -> None:
    """The weight gradient of `Linear(x)` given the gradient g of its output: added in f32 straight into the f32
    gradient of the master weight where the slot carries it and the blocks are told to (one launch, no f16 copy of the
    gradient, no cast at the end of the step), else written as f16 into the slot's f16 gradient."""
    if _ACC32[0] and len(slot) > 4 and slot[4] is not None:
        dev.matmat_br_grad_rhs_f32(x, g, slot[4].permute(1, 0))
    else:
        dev.matmat_br_backward_overwrite(x, None, slot[0].permute(1, 0), slot[2], g)


_ACC32 = [False]        # set by the Trainer that owns f32 gradients and skips the f16 -> f32 copy in exchange


class _DirectAttentionBlock(torch.autograd.Function):
    """`norm1(x + w_o(attention(w_q x, w_k x, w_v x)))` (dfdx/src/nn/layers/transformer.rs:27-28: ResidualAdd around
    MultiHeadAttention, then LayerNorm1D) with the backward written out by hand, as dfdx's tape would replay it, so
    that the gradients that meet at x and at the residual add are summed inside kernels that run anyway:
    the residual add rides in the LayerNorm's forward kernel, the LayerNorm's backward also produces w_o's bias
    gradient (the column sums of its grad_x), and the q/k/v projection's data gradient is accumulated onto the
    residual branch's gradient by the GEMM (beta = 1) instead of by an add kernel.
    Slots as in `_DirectLinear` / `_DirectLayerNorm`; `qkv` is the merged (3 * model, model) projection."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, qkv, o, ln, heads: int, eps: float):
        if x.storage_offset() or not _dense(x) or not x.is_contiguous():
            x = x.contiguous()
        b, s, m = x.shape
        alpha = 1.0 / math.sqrt(m // heads)
        p = dev.linear_forward(x, qkv[0].permute(1, 0), qkv[1], False)             # (b, s, 3 m)
        q, k, v = _split_qkv(p, heads)
        out, lse = dev.attention_forward(q, k, v, alpha, want_lse=True)            # (b, h, s, d) view of a (b, s, m) buffer
        tokens = out.permute(0, 2, 1, 3).reshape(b, s, m)
        y = dev.linear_forward(tokens, o[0].permute(1, 0), o[1], False)
        z, total, stats = dev.add_layer_norm_forward(x, y, ln[0], ln[1], eps)
        ctx.dev, ctx.slots, ctx.heads, ctx.alpha = dev, (qkv, o, ln), heads, alpha
        ctx.save_for_backward(x, p, out, lse, tokens, total, stats)
        return z

    @staticmethod
    def backward(ctx, grad_out):
        x, p, out, lse, tokens, total, stats = ctx.saved_tensors
        dev, (qkv, o, ln), heads = ctx.dev, ctx.slots, ctx.heads
        b, s, m = x.shape
        # LayerNorm: gs is the gradient of x + y, i.e. of both; its column sums are w_o's bias gradient
        gs = dev.layer_norm_backward_sum(total, ln[0], stats, grad_out.contiguous(), ln[2], ln[3], o[3])
        g_tokens = torch.empty_like(tokens)
        dev.matmat_br_backward_overwrite(tokens, g_tokens, o[0].permute(1, 0), None, gs)
        _weight_grad(dev, tokens, o, gs)
        gp = torch.empty_like(p)
        q, k, v = _split_qkv(p, heads)
        dev.attention_backward(q, k, v, ctx.alpha, out, lse, g_tokens.view(b, s, heads, m // heads).permute(0, 2, 1, 3),
                               write_into=_split_qkv(gp, heads))
        _weight_grad(dev, x, qkv, gp)
        dev.matmat_br_backward(x, gs, qkv[0].permute(1, 0), None, gp)                    # gs += gp . W_qkv
        dev.bias_grad(gp, qkv[3])
        return None, gs, None, None, None, None, None


class _DirectFeedForwardBlock(torch.autograd.Function):
    """`norm2(x + l2(relu(l1 x)))` (transformer.rs:29-30) with the backward written out by hand, see
    `_DirectAttentionBlock`: l2's bias gradient comes out of the LayerNorm's backward, ReLU's backward and l1's bias
    gradient are one pass, and l1's data gradient is accumulated onto the residual branch's gradient by the GEMM."""

    @staticmethod
    def forward(ctx, dev: Cuda, x, l1, l2, ln, eps: float):
        if x.storage_offset() or not _dense(x) or not x.is_contiguous():
            x = x.contiguous()
        h = dev.linear_forward(x, l1[0].permute(1, 0), l1[1], True)
        y = dev.linear_forward(h, l2[0].permute(1, 0), l2[1], False)
        z, total, stats = dev.add_layer_norm_forward(x, y, ln[0], ln[1], eps)
        ctx.dev, ctx.slots = dev, (l1, l2, ln)
        ctx.save_for_backward(x, h, total, stats)
        return z

    @staticmethod
    def backward(ctx, grad_out):
        x, h, total, stats = ctx.saved_tensors
        dev, (l1, l2, ln) = ctx.dev, ctx.slots
        gs = dev.layer_norm_backward_sum(total, ln[0], stats, grad_out.contiguous(), ln[2], ln[3], l2[3])
        gh = torch.empty_like(h)
        dev.matmat_br_backward_overwrite(h, gh, l2[0].permute(1, 0), None, gs)
        _weight_grad(dev, h, l2, gs)
        dev.relu_backward_bias_grad(h, gh, l1[3])
        _weight_grad(dev, x, l1, gh)
        dev.matmat_br_backward(x, gs, l1[0].permute(1, 0), None, gh)                    # gs += gh . W_1
        return None, gs, None, None, None, None


class _Attach(torch.autograd.Function):
    """Puts a tensor that needs no gradient on the tape (the ops above take their parameters outside autograd, so
    the first layer's input is what makes their backward run); nothing flows back through it."""

    @staticmethod
    def forward(ctx, x, anchor):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad_out):
        return None, None


class Linear(torch.nn.Module):
    """dfdx `Linear`: weight stored (O, I), consumed as the permuted (I, O) view; uniform(+-1/sqrt(I)) init
    (dfdx/src/nn/layers/linear.rs:65-89)."""

    def __init__(self, dev: Cuda, i: int, o: int, gen: torch.Generator, fused: bool = True):
        super().__init__()
        self.dev, self.fused = dev, fused
        self.slot = None                                           # set by a Trainer that owns the parameters' storage
        b = 1.0 / math.sqrt(i)
        self.weight = torch.nn.Parameter(((torch.rand(o, i, generator=gen) * 2 - 1) * b).to(dev.device))
        self.bias = torch.nn.Parameter(((torch.rand(o, generator=gen) * 2 - 1) * b).to(dev.device))

    def forward(self, x, relu: bool = False):
        if self.slot is not None and self.fused:
            return _DirectLinear.apply(self.dev, x, self.slot, relu)
        w = self.weight.half()                                     # f16 compute copy of the f32 master
        if self.fused:
            return _FusedLinear.apply(self.dev, x, w, self.bias.half(), relu)
        y = matmul(self.dev, x, w.permute(1, 0)) + self.bias.half()
        return torch.relu(y) if relu else y


class MultiHeadAttention(torch.nn.Module):
    def __init__(self, dev: Cuda, model: int, heads: int, gen: torch.Generator, fused: bool = True):
        super().__init__()
        self.dev, self.heads, self.fused = dev, heads, fused
        self.w_q, self.w_k = Linear(dev, model, model, gen, fused), Linear(dev, model, model, gen, fused)
        self.w_v, self.w_o = Linear(dev, model, model, gen, fused), Linear(dev, model, model, gen, fused)
        self.qkv_slot = None        # set by a Trainer that stores w_q, w_k, w_v (and their biases) next to each other

    def forward(self, x):
        b, s, m = x.shape
        h, d = self.heads, m // self.heads
        if self.qkv_slot is not None and self.fused == "attention" and x.dtype == torch.float16 and d % 8 == 0 and d <= 128:
            qkv = _DirectLinear.apply(self.dev, x, self.qkv_slot, False)
            tokens = _FusedAttentionQKV.apply(self.dev, qkv, h, 1.0 / math.sqrt(d))
            return self.w_o(tokens.permute(0, 2, 1, 3).reshape(b, s, m))
        v = self.w_v(x).reshape(b, s, h, d).permute(0, 2, 1, 3)
        k = self.w_k(x).reshape(b, s, h, d).permute(0, 2, 3, 1)
        q = self.w_q(x).reshape(b, s, h, d).permute(0, 2, 1, 3)
        if self.fused == "attention" and x.dtype == torch.float16 and d % 8 == 0 and d <= 128:
            tokens = _FusedAttention.apply(self.dev, q, k, v, 1.0 / math.sqrt(d))
            return self.w_o(tokens.permute(0, 2, 1, 3).reshape(b, s, m))
        if self.fused:
            scores = _ScaledMatMul.apply(self.dev, q, k, 1.0 / math.sqrt(d))
            weights = _Softmax.apply(self.dev, scores)
        else:
            scores = matmul(self.dev, q, k) * (1.0 / math.sqrt(d))
            weights = torch.softmax(scores, dim=-1)
        tokens = matmul(self.dev, weights, v).permute(0, 2, 1, 3).reshape(b, s, m)
        return self.w_o(tokens)


class EncoderBlock(torch.nn.Module):
    def __init__(self, dev: Cuda, model: int, heads: int, ff: int, gen: torch.Generator, fused: bool = True):
        super().__init__()
        self.attn = MultiHeadAttention(dev, model, heads, gen, fused)
        self.norm1 = torch.nn.LayerNorm(model, device=dev.device)
        self.l1, self.l2 = Linear(dev, model, ff, gen, fused), Linear(dev, ff, model, gen, fused)
        self.norm2 = torch.nn.LayerNorm(model, device=dev.device)

    def _norm(self, ln, x):
        if self.attn.fused and getattr(ln, "slot", None) is not None:
            return _DirectLayerNorm.apply(self.attn.dev, x, ln.slot, ln.eps)
        if self.attn.fused:
            return _LayerNorm.apply(self.attn.dev, x, ln.weight.half(), ln.bias.half(), ln.eps)
        return F.layer_norm(x, ln.normalized_shape, ln.weight.half(), ln.bias.half(), ln.eps)

    def forward(self, x):
        a = self.attn
        d = x.shape[-1] // a.heads
        if (a.qkv_slot is not None and a.fused == "attention" and x.dtype == torch.float16 and d % 8 == 0 and d <= 128
                and getattr(self.norm1, "slot", None) is not None):
            x = _DirectAttentionBlock.apply(a.dev, x, a.qkv_slot, a.w_o.slot, self.norm1.slot, a.heads, self.norm1.eps)
            return _DirectFeedForwardBlock.apply(a.dev, x, self.l1.slot, self.l2.slot, self.norm2.slot, self.norm2.eps)
        x = self._norm(self.norm1, x + self.attn(x))
        return self._norm(self.norm2, x + self.l2(self.l1(x, relu=True)))


class Encoder(torch.nn.Module):
    """`layers` encoder blocks (benchmark configuration 5: 6 x (d_model 512, 8 heads, ffn 2048))."""

    def __init__(self, dev: Cuda, layers=6, model=512, heads=8, ff=2048, seed=0, fused=True):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.blocks = torch.nn.ModuleList(EncoderBlock(dev, model, heads, ff, gen, fused) for _ in range(layers))
        self.attach = False                                        # set by a Trainer in direct-gradient mode

    def forward(self, x):
        if self.attach and not x.requires_grad:
            # a fresh leaf every step: a long-lived one would tie the backward pass to the stream it was made on
            x = _Attach.apply(x, torch.zeros(1, device=x.device, requires_grad=True))
        for blk in self.blocks:
            x = blk(x)
        return x


class Trainer:
    """One data-parallel training step: forward, MSE loss, backward, gradient all-reduce, Adam.

    The eager step is bound by host-side launch overhead (about 300 small launches), so `capture()` records
    the whole step once into a CUDA graph and `step()` then replays it on static input buffers."""

    def __init__(self, dev: Cuda, world: int = 1, direct: bool = True, **model_kw):
        self.dev, self.world = dev, world
        self.model = Encoder(dev, **model_kw)
        linears = [m for m in self.model.modules() if isinstance(m, Linear)]
        weights = [m.weight for m in linears]
        seen = {id(p) for p in weights}
        params = weights + [p for p in self.model.parameters() if id(p) not in seen]
        total = sum(p.numel() for p in params)
        # one flat f32 master buffer and one flat f32 gradient buffer (a single NCCL all-reduce per step), the
        # Linear weights first
        self.flat_param = torch.empty(total, device=dev.device)
        self.flat_grad = torch.zeros(total, device=dev.device)
        spans, off = {}, 0
        for p in params:
            spans[id(p)] = (off, off + p.numel())
            self.flat_param[off:off + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.flat_param[off:off + p.numel()].view_as(p)
            p.grad = self.flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
        # Direct-gradient mode (fused modes only): the f16 compute copies of all parameters are one flat buffer
        # refreshed by one cast per step; the GEMMs write the f16 weight gradients into one flat buffer that one
        # cast folds into the f32 gradients; bias / LayerNorm gradients (f32 column sums) are added straight into
        # their f32 slots.  Otherwise every parameter takes torch's route: a cast per use, and per gradient a
        # cast and an add.
        self.direct = bool(direct and model_kw.get("fused", True))
        if self.direct:
            self.n_weights = sum(p.numel() for p in weights)
            self.flat16 = torch.empty(total, dtype=torch.float16, device=dev.device)
            self.flat_gw16 = torch.zeros(self.n_weights, dtype=torch.float16, device=dev.device)

            def v16(p):
                lo, hi = spans[id(p)]
                return self.flat16[lo:hi].view_as(p)
            for m in linears:
                lo, hi = spans[id(m.weight)]
                m.slot = (v16(m.weight), v16(m.bias), self.flat_gw16[lo:hi].view_as(m.weight), m.bias.grad, m.weight.grad)
            for blk in self.model.blocks:
                for ln in (blk.norm1, blk.norm2):
                    ln.slot = (v16(ln.weight), v16(ln.bias), ln.weight.grad, ln.bias.grad)
                # w_q, w_k, w_v lie next to each other in the flat buffers (so do their biases): one (3 * model, model)
                # weight whose rows are the three projections' outputs
                a = blk.attn
                ws = [spans[id(l.weight)] for l in (a.w_q, a.w_k, a.w_v)]
                bs = [spans[id(l.bias)] for l in (a.w_q, a.w_k, a.w_v)]
                if all(ws[i][1] == ws[i + 1][0] and bs[i][1] == bs[i + 1][0] for i in range(2)):
                    o3, i_ = 3 * a.w_q.weight.shape[0], a.w_q.weight.shape[1]
                    a.qkv_slot = (self.flat16[ws[0][0]:ws[2][1]].view(o3, i_), self.flat16[bs[0][0]:bs[2][1]],
                                  self.flat_gw16[ws[0][0]:ws[2][1]].view(o3, i_), self.flat_grad[bs[0][0]:bs[2][1]],
                                  self.flat_grad[ws[0][0]:ws[2][1]].view(o3, i_))
            self.model.attach = True
        # With every Linear inside the hand-written blocks (f16 input, fused attention, head size the kernel takes) the
        # weight gradients are added in f32 straight into flat_grad; the f16 gradient buffer and its cast are not used.
        blocks = list(self.model.blocks)
        a0 = blocks[0].attn if blocks else None
        self.acc32 = bool(self.direct and a0 is not None and a0.fused == "attention" and len(linears) == 6 * len(blocks)
                          and all(b.attn.qkv_slot is not None for b in blocks)
                          and (a0.w_q.weight.shape[0] // a0.heads) % 8 == 0 and a0.w_q.weight.shape[0] // a0.heads <= 128
                          and all(d % 8 == 0 for m in linears for d in m.weight.shape))
        # Adam is element-wise, so it runs on the one flat buffer (a single fused kernel per step) instead of on the
        # hundred parameter views into it; `params` keeps the views for inspection
        self.params = params
        self.flat_p = torch.nn.Parameter(self.flat_param, requires_grad=False)
        self.flat_p.grad = self.flat_grad
        self.opt = torch.optim.Adam([self.flat_p], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, fused=True, capturable=True)
        self.graph = None

    def _step(self, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        self.flat_grad.zero_()
        _ACC32[0] = self.acc32
        if self.acc32 and x.dtype != torch.float16:
            raise TypeError("this trainer's blocks take f16 inputs")
        if self.direct:
            self.flat16.copy_(self.flat_param)
        loss = F.mse_loss(self.model(x).float(), target.float())
        loss.backward()
        if self.direct and not self.acc32:
            self.flat_grad[:self.n_weights].copy_(self.flat_gw16)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(self.flat_grad)
            self.flat_grad.div_(self.world)
        self.opt.step()
        return loss

    def capture(self, x: torch.Tensor, target: torch.Tensor) -> bool:
        """Records the step into a CUDA graph (after three eager steps on a side stream).  Returns False and
        stays eager if the capture fails."""
        self._x, self._t = x.clone(), target.clone()
        try:
            side = torch.cuda.Stream(self.dev.device)
            side.wait_stream(torch.cuda.current_stream(self.dev.device))
            with torch.cuda.stream(side):
                for _ in range(3):
                    self._step(self._x, self._t)
            torch.cuda.current_stream(self.dev.device).wait_stream(side)
            torch.cuda.synchronize(self.dev.device)
            graph = torch.cuda.CUDAGraph()
            # The trainer replays its graph on the one stream that carries all of its other work on this library, so
            # the f16 GEMMs inside the capture may keep their split-K (see b200_set_capture_split_k).
            self.dev.lib.b200_set_capture_split_k(1)
            try:
                with torch.cuda.graph(graph):
                    self._loss = self._step(self._x, self._t)
            finally:
                self.dev.lib.b200_set_capture_split_k(0)
            self.graph = graph
            return True
        except Exception as exc:  # noqa: BLE001 - any capture failure means: stay eager
            self.capture_error = repr(exc)
            self.graph = None
            torch.cuda.synchronize(self.dev.device)
            return False

    def step(self, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        if self.graph is None:
            return self._step(x, target)
        self._x.copy_(x, non_blocking=True)
        self._t.copy_(target, non_blocking=True)
        self.graph.replay()
        return self._loss
