"""Shared test plumbing: backends with one interface over the CPU oracle and the CUDA device, the
golden-vector loader, and the upstream gradients implied by the losses dfdx's tests use."""
from __future__ import annotations

import json
from pathlib import Path

import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

# dfdx-core/src/lib.rs:236-270: absolute tolerance 1e-6 for f32/f64, 1e-2 for f16.
ABS_TOL = {torch.float32: 1e-6, torch.float64: 1e-6, torch.float16: 1e-2}
# Relative Frobenius error bound against the f64 oracle for large shapes.
FROB_TOL = {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 2e-3}


def golden(name: str) -> dict:
    return json.loads((GOLDEN / f"{name}.json").read_text())["tests"]


class OracleBackend:
    """dfdx's `Cpu` device restated (oracle/oracle.c), f64 arithmetic."""
    name = "oracle"

    def __init__(self, oracle, dtype=torch.float64):
        self.o = oracle
        self.dtype = dtype

    def tensor(self, value):
        return torch.tensor(value, dtype=torch.float64).to(self.dtype)

    def randn(self, *shape, gen):
        return torch.randn(*shape, generator=gen, dtype=torch.float64).to(self.dtype)

    def matmul(self, a, b):
        return self.o.matmul(a, b)

    def conv2d(self, x, w, **kw):
        return self.o.conv2d(x, w, **kw)

    def conv1d(self, x, w, **kw):
        return self.o.conv1d(x, w, **kw)

    def convtrans2d(self, x, w, **kw):
        return self.o.convtrans2d(x, w, **kw)

    def normalize(self, x, eps):
        y, bwd = self.o.layer_norm(x, None, None, eps)
        return y, lambda go: bwd(go)[0]

    def softmax(self, x):
        return self.o.softmax(x)

    def linear(self, x, weight_view, bias, relu=False):
        return self.o.fused_matmul(x, weight_view, 1.0, bias, relu)

    def host(self, t):
        return t.detach().cpu().to(torch.float64)


class CudaBackend:
    """The device under test, through the C ABI."""
    name = "cuda"

    def __init__(self, dev, dtype):
        self.dev = dev
        self.dtype = dtype

    def tensor(self, value):
        return torch.tensor(value, dtype=torch.float64).to(self.dtype).to(self.dev.device)

    def randn(self, *shape, gen):
        return torch.randn(*shape, generator=gen, dtype=torch.float64).to(self.dtype).to(self.dev.device)

    def matmul(self, a, b):
        out, bwd = self.dev.matmul(a, b)

        def backward(go):
            return bwd(go.to(self.dtype).to(self.dev.device))
        return out, backward

    def linear(self, x, weight_view, bias, relu=False):
        """`Linear::try_forward` through the fused entry point (x of rank 1..3 is viewed as rank 3)."""
        x3 = x.reshape((1,) * (3 - x.dim()) + tuple(x.shape))
        return self.dev.linear_forward(x3, weight_view, bias, relu).reshape(tuple(x.shape[:-1]) + (weight_view.shape[1],))

    def convtrans2d(self, x, w, **kw):
        out, bwd = self.dev.convtrans2d(x, w, **kw)

        def backward(go):
            return bwd(go.to(self.dtype).to(self.dev.device))
        return out, backward

    def conv1d(self, x, w, **kw):
        out, bwd = self.dev.conv1d(x, w, **kw)

        def backward(go):
            return bwd(go.to(self.dtype).to(self.dev.device))
        return out, backward

    def normalize(self, x, eps):
        """`normalize` over the last axis through the LayerNorm kernels (gamma = beta = NULL)."""
        y, stats = self.dev.layer_norm_forward(x, None, None, eps, want_stats=True)
        return y, lambda go: self.dev.layer_norm_backward(x, None, stats, go.to(self.dtype).to(self.dev.device).contiguous())

    def conv2d(self, x, w, **kw):
        out, bwd = self.dev.conv2d(x, w, **kw)

        def backward(go):
            return bwd(go.to(self.dtype).to(self.dev.device))
        return out, backward

    def softmax(self, x):
        """softmax over the last axis through the row-wise kernels."""
        xc = x.contiguous()
        y = self.dev.softmax_forward(xc)
        return y, lambda go: self.dev.softmax_backward(y, go.to(self.dtype).to(self.dev.device).contiguous())

    def host(self, t):
        return t.detach().cpu().to(torch.float64)


# Upstream gradients of the scalar losses used by the reference's tests, as functions of the op output
# (host f64).
def d_exp_mean(r):
    return torch.exp(r) / r.numel()


def d_exp_sum(r):
    return torch.exp(r)


def d_sum(r):
    return torch.ones_like(r)


def d_square_mean(r):
    return 2.0 * r / r.numel()


def d_mean(r):
    return torch.full_like(r, 1.0 / r.numel())


def assert_close(got, want, tol, what=""):
    got = got.detach().cpu().to(torch.float64)
    want = torch.as_tensor(want, dtype=torch.float64)
    assert tuple(got.shape) == tuple(want.shape), f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs().max().item() if got.numel() else 0.0
    assert err <= tol, f"{what}: max abs err {err:.3e} > {tol:.1e}\n got {got}\nwant {want}"
