"""The encoder harness of configuration 5: its matmuls (forward and backward, through the C ABI) against
torch's own f32 autograd on the same f16-rounded parameters and inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True, "attention"], ids=["unfused", "fused-epilogues", "fused-attention"])
def test_encoder_block_matches_torch_autograd(cuda_dev, fused):
    from dfdx_b200 import encoder as enc
    dev = cuda_dev
    gen = torch.Generator().manual_seed(1)
    blk = enc.EncoderBlock(dev, 128, 4, 256, gen, fused=fused)
    x = torch.randn(3, 40, 128, generator=gen).half().to(dev.device).requires_grad_(True)
    t = torch.randn(3, 40, 128, generator=gen).to(dev.device)
    before = dev.lib.b200_launch_count()
    loss = torch.nn.functional.mse_loss(blk(x).float(), t)
    loss.backward()
    # 6 Linear + 2 attention matmuls, forward + 2 grads each; fused attention: 1 forward + 3 backward launches instead of 6
    assert dev.lib.b200_launch_count() - before >= (3 * 6 + 4 if fused == "attention" else 3 * 8)
    got = {n: p.grad.clone() for n, p in blk.named_parameters()}
    gx = x.grad.float().clone()

    # reference: same math with torch.matmul in f32 on the f16-rounded values
    real = enc.matmul
    enc.matmul = lambda d, a, b: torch.matmul(a.float(), b.float()).half()
    for mod in blk.modules():                                      # the reference pass runs the unfused op sequence
        if hasattr(mod, "fused"):
            mod.fused = False
    try:
        for p in blk.parameters():
            p.grad = None
        x2 = x.detach().clone().requires_grad_(True)
        loss2 = torch.nn.functional.mse_loss(blk(x2).float(), t)
        loss2.backward()
    finally:
        enc.matmul = real
    assert abs(loss.item() - loss2.item()) <= 2e-3 * abs(loss2.item())
    biggest = max(float(p.grad.norm()) for p in blk.parameters())
    for n, p in blk.named_parameters():
        ref = p.grad
        # gradients that are mathematically zero (the key bias: softmax is shift-invariant) are pure rounding
        # noise, so the error is measured against the larger of the reference norm and 1e-2 of the largest one
        err = (got[n] - ref).norm() / max(float(ref.norm()), 1e-2 * biggest)
        assert err <= 2e-2, f"{n}: relative error {float(err):.3e}"
    err = (gx - x2.grad.float()).norm() / x2.grad.float().norm()
    assert err <= 2e-2


def test_trainer_graph_replay_matches_eager(cuda_dev):
    """A captured step replays to the same loss trajectory as eager steps from the same initial state."""
    from dfdx_b200.encoder import Trainer
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(4, 32, 64, generator=gen).half().to(cuda_dev.device)
    t = torch.randn(4, 32, 64, generator=gen).half().to(cuda_dev.device)
    kw = dict(layers=2, model=64, heads=4, ff=128, seed=3)
    eager = Trainer(cuda_dev, 1, **kw)
    want = [eager.step(x, t).item() for _ in range(7)]
    graphed = Trainer(cuda_dev, 1, **kw)
    assert graphed.capture(x, t), getattr(graphed, "capture_error", "")
    got = [graphed.step(x, t).item() for _ in range(4)]            # capture ran 3 warm-up steps + 1 recorded step
    assert want[6] < want[0]                                        # it trains
    for g_, w_ in zip(got, want[4:7] + [None]):
        if w_ is not None:
            assert abs(g_ - w_) <= 2e-2 * abs(w_)


def test_trainer_direct_gradients_match_autograd_route(cuda_dev):
    """Gradients written straight into the trainer's flat buffers equal the ones torch's autograd collects
    (cast, add per parameter) for the same step; bias / LayerNorm gradients differ by the f16 rounding the
    autograd route puts on the f32 column sums, and everything upstream of an attention block by the rounding of
    the two f16 adds with which autograd sums the q, k and v projections' data gradients (the direct route's single
    (model -> 3 * model) projection sums them in f32 inside one GEMM)."""
    from dfdx_b200.encoder import Trainer
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(4, 32, 64, generator=gen).half().to(cuda_dev.device)
    t = torch.randn(4, 32, 64, generator=gen).half().to(cuda_dev.device)
    kw = dict(layers=2, model=64, heads=4, ff=128, seed=3, fused="attention")
    a, b = Trainer(cuda_dev, 1, direct=True, **kw), Trainer(cuda_dev, 1, direct=False, **kw)
    assert a.direct and not b.direct
    assert torch.equal(a.flat_param, b.flat_param)
    la, lb = a._step(x, t), b._step(x, t)
    assert abs(la.item() - lb.item()) <= 1e-6 * abs(lb.item())
    for pa, pb, (name, _) in zip(a.params, b.params, [(n, 0) for n in range(10 ** 6)]):
        ref = pb.grad.float()
        err = (pa.grad.float() - ref).norm() / max(float(ref.norm()), 1e-2 * float(b.flat_grad.norm()))
        assert err <= 5e-3, f"parameter {name}: {float(err):.3e}"
    # the step trained both the same way
    assert (a.flat_param - b.flat_param).abs().max() <= 2.1e-3    # one Adam step moves a weight by at most lr


def test_fused_qkv_attention_matches_separate_projections(cuda_dev):
    """Attention on the strided q, k, v views of one (b, s, 3 * model) projection output, with the three gradients
    written into the views of one buffer, equals attention on three separate tensors: same kernels, other strides."""
    from dfdx_b200 import encoder as enc
    dev = cuda_dev
    b, s, h, d = 2, 64, 4, 16
    m = h * d
    gen = torch.Generator().manual_seed(11)
    qkv = torch.randn(b, s, 3 * m, generator=gen).half().to(dev.device).requires_grad_()
    go = torch.randn(b, h, s, d, generator=gen).half().to(dev.device)
    alpha = 1.0 / d ** 0.5
    out = enc._FusedAttentionQKV.apply(dev, qkv, h, alpha)
    out.backward(go)
    parts = [qkv.detach()[..., i * m:(i + 1) * m].reshape(b, s, h, d).clone().requires_grad_() for i in range(3)]
    q, k, v = parts[0].permute(0, 2, 1, 3), parts[1].permute(0, 2, 3, 1), parts[2].permute(0, 2, 1, 3)
    ref = enc._FusedAttention.apply(dev, q, k, v, alpha)
    ref.backward(go)
    assert torch.equal(out, ref)
    for i, p in enumerate(parts):
        assert torch.equal(qkv.grad[..., i * m:(i + 1) * m].reshape(b, s, h, d), p.grad), "qkv"[i]
