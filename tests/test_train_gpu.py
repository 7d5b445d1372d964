"""The training-step harness: fused Adam kernel against a plain fp32 Adam, and
a few steps of the GTrXL-style value network driving the loss down."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_adam_matches_reference_update():
    from memorax_b200 import ops
    g = torch.Generator().manual_seed(0)
    n = 8 * 1000
    p0 = torch.randn(n, generator=g).bfloat16()
    p, m, v = p0.clone().cuda(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pr, mr, vr = p0.float(), torch.zeros(n), torch.zeros(n)
    lr, b1, b2, eps, world = 1e-2, 0.9, 0.999, 1e-8, 4
    for step in range(1, 6):
        grad = (torch.randn(n, generator=g) * world).bfloat16()
        ops.adam_step(p, grad.cuda(), m, v, step, lr, (b1, b2), eps, grad_scale=1.0 / world)
        gr = grad.float() / world
        mr = b1 * mr + (1 - b1) * gr
        vr = b2 * vr + (1 - b2) * gr * gr
        pr = (pr - lr * (mr / (1 - b1 ** step)) / ((vr / (1 - b2 ** step)).sqrt() + eps)).bfloat16().float()
    # betas cross the C ABI as fp32: 1 - 0.999f differs from 0.001 by 1.3e-5 relative
    assert torch.allclose(m.cpu(), mr, rtol=1e-4, atol=1e-7) and torch.allclose(v.cpu(), vr, rtol=1e-4, atol=1e-9)
    assert float((p.float().cpu() - pr).abs().max()) <= 2e-2   # bf16 parameter rounding (one ulp at |p| < 4)


def test_value_network_trains():
    from memorax_b200.blocks import FlatAdamTrainer, GTrXLStyleValueNet
    torch.manual_seed(0)
    model = GTrXLStyleValueNet(obs_dim=16, d_model=128, num_heads=1, head_dim=128, layers=2).to("cuda", torch.bfloat16)
    trainer = FlatAdamTrainer(model, lr=3e-3)
    g = torch.Generator().manual_seed(1)
    obs = torch.randn(8, 96, 16, generator=g).bfloat16().cuda()
    done = (torch.rand(8, 96, generator=g) < 0.02).cuda()
    target = obs.float().mean(-1) * 2.0
    losses = [float(trainer.step(obs, done, target)) for _ in range(30)]
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < 0.7 * losses[0], losses
    assert all(p.data_ptr() >= trainer.flat.data_ptr() for p in model.parameters())
