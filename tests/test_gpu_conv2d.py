"""GPU parity of conv2d (unfold + GEMM lowering) against the CPU oracle, through the C ABI.

Cases follow dfdx-core/src/tensor_ops/conv2d/tests.rs: stride / padding / dilation / groups
variants, batched vs single image (:218-250), grouped vs sliced (:404-464), plus benchmark configuration 4 at
full size on sampled output channels / pixels.
"""
import pytest
import torch

import dfdx_b200
from helpers import FROB_TOL, CudaBackend, OracleBackend, d_exp_sum, d_square_mean

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator().manual_seed(seed)


CASES = [
    dict(x=(2, 3, 7, 6), w=(4, 3, 2, 2), stride=1, padding=0, dilation=1, groups=1),
    dict(x=(1, 5, 7, 6), w=(3, 5, 2, 2), stride=4, padding=3, dilation=1, groups=1),
    dict(x=(3, 3, 28, 28), w=(5, 3, 6, 6), stride=3, padding=2, dilation=1, groups=1),
    dict(x=(2, 4, 9, 8), w=(6, 4, 3, 3), stride=2, padding=1, dilation=2, groups=1),
    dict(x=(2, 9, 14, 14), w=(15, 3, 3, 3), stride=1, padding=0, dilation=1, groups=3),
    dict(x=(2, 8, 10, 11), w=(4, 4, 3, 3), stride=2, padding=2, dilation=1, groups=2),
    dict(x=(4, 16, 24, 24), w=(32, 16, 3, 3), stride=1, padding=1, dilation=1, groups=1),
    dict(x=(2, 32, 16, 16), w=(64, 8, 3, 3), stride=1, padding=1, dilation=1, groups=4),
]


@pytest.mark.parametrize("path", [pytest.param(dfdx_b200.PATH_SIMT, id="simt"),
                                  pytest.param(dfdx_b200.PATH_AUTO, id="auto")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_conv2d_forward_backward(cuda_dev, oracle, case, dtype, path):
    cfg = CASES[case]
    kw = {k: cfg[k] for k in ("stride", "padding", "dilation", "groups")}
    g = gen(40 + case)
    x = (torch.randn(*cfg["x"], generator=g, dtype=torch.float64) * 0.5).to(dtype)
    w = (torch.randn(*cfg["w"], generator=g, dtype=torch.float64) * 0.2).to(dtype)
    want, obwd = OracleBackend(oracle, dtype).conv2d(x, w, **kw)
    cuda_dev.set_path(path)
    try:
        got, cbwd = CudaBackend(cuda_dev, dtype).conv2d(x.to(cuda_dev.device), w.to(cuda_dev.device), **kw)
        go = d_square_mean(want) * want.numel() / 64.0
        gx, gw = cbwd(go)
        cuda_dev.synchronize()
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)
    wgx, wgw = obwd(go.to(dtype))
    tol = FROB_TOL[dtype]
    assert oracle.rel_frobenius(got, want) <= tol
    assert oracle.rel_frobenius(gx, wgx) <= tol
    assert oracle.rel_frobenius(gw, wgw) <= tol


def test_batched_conv2d_property(cuda_dev):
    """conv2d/tests.rs:218-250: a batch of 10 copies of one image gives 10 copies of the output, the same
    filter gradient (mean loss) and 1/10 of the image gradient per copy."""
    cb = CudaBackend(cuda_dev, torch.float32)
    g = gen(60)
    x, w = cb.randn(3, 28, 28, gen=g), cb.randn(5, 3, 6, 6, gen=g)
    y0, bwd0 = cb.conv2d(x, w, stride=3, padding=2)
    gx0, gw0 = bwd0(d_square_mean(cb.host(y0)))
    xb = x.expand(10, 3, 28, 28).contiguous()
    y, bwd = cb.conv2d(xb, w, stride=3, padding=2)
    gx, gw = bwd(d_square_mean(cb.host(y)))
    for i in range(10):
        assert (cb.host(y[i]) - cb.host(y0)).abs().max() <= 1e-6
        assert (cb.host(gx[i]) * 10.0 - cb.host(gx0)).abs().max() <= 1e-6
    assert (cb.host(gw) - cb.host(gw0)).abs().max() <= 1e-3


def test_grouped_equals_slices_property(cuda_dev):
    """conv2d/tests.rs:404-464."""
    cb = CudaBackend(cuda_dev, torch.float32)
    g = gen(61)
    x, w = cb.randn(2, 9, 14, 14, gen=g), cb.randn(15, 3, 3, 3, gen=g)
    y, bwd = cb.conv2d(x, w, groups=3)
    gx, gw = bwd(d_exp_sum(cb.host(y)).clamp(max=1e4))
    for i in range(3):
        xg, wg = x[:, 3 * i:3 * i + 3].contiguous(), w[5 * i:5 * i + 5].contiguous()
        yg, bwdg = cb.conv2d(xg, wg)
        assert (cb.host(yg) - cb.host(y[:, 5 * i:5 * i + 5])).abs().max() <= 1e-5
        gxg, gwg = bwdg(d_exp_sum(cb.host(yg)).clamp(max=1e4))
        ref_x, ref_w = cb.host(gx[:, 3 * i:3 * i + 3]), cb.host(gw[5 * i:5 * i + 5])
        assert (cb.host(gxg) - ref_x).abs().max() <= 1e-5 * max(1.0, ref_x.abs().max().item())
        assert (cb.host(gwg) - ref_w).abs().max() <= 1e-5 * max(1.0, ref_w.abs().max().item())


def test_not_contiguous_is_rejected(cuda_dev):
    """conv2d/mod.rs:287-289."""
    x = torch.zeros(2, 6, 6, 3, device=cuda_dev.device).permute(0, 3, 1, 2)
    w = torch.zeros(4, 3, 2, 2, device=cuda_dev.device)
    with pytest.raises(dfdx_b200.ShapeMismatch, match="must be contiguous"):
        cuda_dev.conv2d(x, w)


def test_config4_conv2d_f32_full_size(cuda_dev, oracle):
    """x[32,64,56,56], w[128,64,3,3], stride 1, padding 1.  Images 0 and 31 are checked in full against
    the oracle (forward and grad_input); grad_weight against the oracle on a 2-image sub-batch plus
    additivity over the batch."""
    dev = cuda_dev
    g = gen(0xD0FD + 4)
    x = torch.randn(32, 64, 56, 56, generator=g, dtype=torch.float32)
    bound = 1.0 / (64 * 9) ** 0.5
    w = ((torch.rand(128, 64, 3, 3, generator=g, dtype=torch.float64) * 2 - 1) * bound).to(torch.float32)
    dy = torch.randn(32, 128, 56, 56, generator=g, dtype=torch.float32)
    xd, wd, dyd = x.to(dev.device), w.to(dev.device), dy.to(dev.device)
    y, bwd = dev.conv2d(xd, wd, stride=1, padding=1)
    gx, gw = bwd(dyd)
    dev.synchronize()
    for i in (0, 31):
        want, obwd = oracle.conv2d(x[i:i + 1], w, stride=1, padding=1)
        assert oracle.rel_frobenius(y[i:i + 1], want) <= 1e-5
        wgx, _ = obwd(dy[i:i + 1])
        assert oracle.rel_frobenius(gx[i:i + 1], wgx) <= 1e-5
    # grad_weight: sub-batch {0, 31} against the oracle ...
    sub = torch.tensor([0, 31])
    _, obwd2 = oracle.conv2d(x[sub], w, stride=1, padding=1)
    _, wgw2 = obwd2(dy[sub])
    _, bwd2 = dev.conv2d(xd[sub.to(dev.device)].contiguous(), wd, stride=1, padding=1)
    _, gw2 = bwd2(dyd[sub.to(dev.device)].contiguous())
    assert oracle.rel_frobenius(gw2, wgw2) <= 1e-5
    # ... and additivity: grad_w(batch) == grad_w(first half) + grad_w(second half)
    _, bwd_a = dev.conv2d(xd[:16].contiguous(), wd, stride=1, padding=1)
    _, bwd_b = dev.conv2d(xd[16:].contiguous(), wd, stride=1, padding=1)
    _, gwa = bwd_a(dyd[:16].contiguous())
    _, gwb = bwd_b(dyd[16:].contiguous())
    dev.synchronize()
    assert oracle.rel_frobenius(gwa + gwb, gw.double()) <= 1e-5


@pytest.mark.parametrize("lowering", [pytest.param((0, 0), id="auto"), pytest.param((2, 0), id="fold"),
                                      pytest.param((2, 1), id="fold-per-image"), pytest.param((1, 0), id="gather")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_grad_img_lowerings_agree_with_oracle(cuda_dev, oracle, dtype, lowering):
    """The data gradient by the planner's choice, by filters^T x grad_out + fold (all images at once, and one image
    per pass) and by the reference's gather + GEMM, every geometry of CASES, accumulating into a non-zero grad_img."""
    mode, group = lowering
    assert cuda_dev.lib.b200_set_conv_lowering(mode, group) == 0
    try:
        for case, cfg in enumerate(CASES):
            kw = {k: cfg[k] for k in ("stride", "padding", "dilation", "groups")}
            g = gen(90 + case)
            x = (torch.randn(*cfg["x"], generator=g, dtype=torch.float64) * 0.5).to(dtype)
            w = (torch.randn(*cfg["w"], generator=g, dtype=torch.float64) * 0.2).to(dtype)
            want, obwd = OracleBackend(oracle, dtype).conv2d(x, w, **kw)
            go = torch.randn(*want.shape, generator=g, dtype=torch.float64).to(dtype)
            wgx, wgw = obwd(go)
            xd, wd = x.to(cuda_dev.device), w.to(cuda_dev.device)
            op = cuda_dev.conv2d_op(xd, wd, **kw)
            gx, gw = torch.ones_like(xd), torch.zeros_like(wd)
            cuda_dev.conv2d_backward(op, xd, gx, wd, gw, go.to(cuda_dev.device))
            assert oracle.rel_frobenius(gx, wgx.to(torch.float64) + 1.0) <= FROB_TOL[dtype], (case, lowering)
            assert oracle.rel_frobenius(gw, wgw) <= FROB_TOL[dtype], (case, lowering)
    finally:
        cuda_dev.lib.b200_set_conv_lowering(0, 0)
    assert cuda_dev.lib.b200_set_conv_lowering(3, 0) == dfdx_b200._lib.ERR_UNSUPPORTED


# Geometries the implicit-GEMM lowering serves (f32, unit stride, tensor-core sized): padding 0 / 1 / 2, dilation,
# groups, 1x1 and 5x5 filters, channel counts that need zero padding (24 -> 32), output rows that do not fill a
# tile (20 pixels per row: 12 rows = 240 positions per tile, the last tile of an image ragged), more than one tile
# of output channels with a ragged last one (200), data gradients with 64 and 128 channels per group.
IMPLICIT_CASES = [
    dict(x=(2, 16, 24, 24), w=(32, 16, 3, 3), padding=1, dilation=1, groups=1, dgrad=False),
    dict(x=(2, 64, 14, 20), w=(48, 64, 3, 3), padding=1, dilation=1, groups=1, dgrad=True),
    dict(x=(3, 24, 12, 12), w=(40, 24, 5, 5), padding=2, dilation=1, groups=1, dgrad=False),
    dict(x=(2, 32, 16, 16), w=(64, 32, 3, 3), padding=2, dilation=2, groups=1, dgrad=False),
    dict(x=(2, 64, 12, 12), w=(64, 32, 3, 3), padding=1, dilation=1, groups=2, dgrad=False),
    dict(x=(2, 128, 12, 12), w=(128, 64, 3, 3), padding=1, dilation=1, groups=2, dgrad=True),
    dict(x=(2, 64, 16, 16), w=(128, 64, 1, 1), padding=0, dilation=1, groups=1, dgrad=True),
    dict(x=(2, 16, 16, 16), w=(200, 16, 3, 3), padding=1, dilation=1, groups=1, dgrad=False),
    dict(x=(2, 128, 10, 12), w=(24, 128, 3, 3), padding=1, dilation=1, groups=1, dgrad=True),
    dict(x=(6, 64, 9, 10), w=(32, 64, 3, 3), padding=0, dilation=1, groups=1, dgrad=False),  # 7 x 8 outputs: one 56-wide tile
]


@pytest.mark.parametrize("case", range(len(IMPLICIT_CASES)))
def test_implicit_gemm_lowering(cuda_dev, oracle, case):
    """Forward, filter gradient and data gradient through the implicit GEMM (no patch buffer): against the oracle, and
    against the materialising lowering of the same library; the launch counts show which lowering ran."""
    dev, lib = cuda_dev, cuda_dev.lib
    cfg = IMPLICIT_CASES[case]
    kw = dict(stride=1, padding=cfg["padding"], dilation=cfg["dilation"], groups=cfg["groups"])
    g = gen(300 + case)
    x = (torch.randn(*cfg["x"], generator=g, dtype=torch.float64) * 0.5).float()
    w = (torch.randn(*cfg["w"], generator=g, dtype=torch.float64) * 0.2).float()
    want, obwd = OracleBackend(oracle, torch.float32).conv2d(x, w, **kw)
    go = torch.randn(*want.shape, generator=g, dtype=torch.float64).float()
    wgx, wgw = obwd(go)
    xd, wd, god = x.to(dev.device), w.to(dev.device), go.to(dev.device)
    op = dev.conv2d_op(xd, wd, **kw)
    res = {}
    for mode in (0, 2):
        assert lib.b200_set_conv_lowering(mode, 0) == 0
        try:
            y = torch.full(want.shape, float("nan"), device=dev.device)
            l0, t0, i0 = lib.b200_launch_count(), lib.b200_tensor_launch_count(), lib.b200_conv_implicit_count()
            dev.conv2d_forward(op, xd, wd, y)
            fwd = (lib.b200_launch_count() - l0, lib.b200_tensor_launch_count() - t0, lib.b200_conv_implicit_count() - i0)
            gx, gw = torch.ones_like(xd), torch.full_like(wd, 0.5)
            l0, i0 = lib.b200_launch_count(), lib.b200_conv_implicit_count()
            dev.conv2d_backward(op, xd, gx, wd, gw, god)
            bwd = (lib.b200_launch_count() - l0, lib.b200_conv_implicit_count() - i0)
            dev.synchronize()
        finally:
            lib.b200_set_conv_lowering(0, 0)
        res[mode] = (y, gx, gw)
        assert oracle.rel_frobenius(y, want) <= 1e-5, (case, mode)
        assert oracle.rel_frobenius(gx, wgx.double() + 1.0) <= 1e-5, (case, mode)
        assert oracle.rel_frobenius(gw, wgw.double() + 0.5) <= 1e-5, (case, mode)
        groups = cfg["groups"]
        if mode == 0:
            # implicit forward: one launch for the layout change and the filter rows, one tensor-core launch
            assert fwd == (2, 1, 1), fwd
            # filter gradient: layout change, one launch per group, add; data gradient: 2 launches when implicit, else
            # one GEMM + one fold
            assert bwd == (2 + groups + 2, 2 if cfg["dgrad"] else 1), bwd
        else:
            assert fwd == (2, 1, 0), fwd                    # unfold + GEMM
            assert bwd[1] == 0, bwd
    for a, b in zip(res[0], res[2]):
        assert oracle.rel_frobenius(a, b.double()) <= 2e-5
