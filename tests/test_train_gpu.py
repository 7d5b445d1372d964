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


def test_fused_adam_fp32_master_moves_parameters_at_small_learning_rates():
    """lr = 3e-4 (the reference's optax.adam default scale) on parameters of magnitude 1: one step is a
    twentieth of a bf16 ulp, so only an fp32 master copy accumulates it.  The master follows plain fp32 Adam,
    the bf16 working copy is its rounding, and after enough steps the bf16 values have moved."""
    from memorax_b200 import ops
    g = torch.Generator().manual_seed(3)
    n = 8 * 512
    p0 = torch.ones(n).bfloat16()
    p0[::2] = -0.75
    p, master = p0.clone().cuda(), p0.float().cuda()
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pr, mr, vr = p0.double(), torch.zeros(n, dtype=torch.float64), torch.zeros(n, dtype=torch.float64)
    lr, b1, b2, eps = 3e-4, 0.9, 0.999, 1e-8
    direction = torch.where(torch.arange(n) % 3 == 0, -1.0, 1.0)
    for step in range(1, 41):
        grad = (direction * (0.5 + torch.rand(n, generator=g))).bfloat16()
        ops.adam_step(p, grad.cuda(), m, v, step, lr, (b1, b2), eps, master=master)
        gr = grad.double()
        mr = b1 * mr + (1 - b1) * gr
        vr = b2 * vr + (1 - b2) * gr * gr
        pr = pr - lr * (mr / (1 - b1 ** step)) / ((vr / (1 - b2 ** step)).sqrt() + eps)
    assert float((master.cpu().double() - pr).abs().max()) <= 2e-5          # fp32 accumulation of 40 steps
    assert torch.equal(p.cpu(), master.cpu().bfloat16())                      # working copy = rounded master
    moved = (p.cpu().float() != p0.float())
    assert float(moved.float().mean()) > 0.9, "bf16 parameters of magnitude 1 must move after 40 steps of 3e-4"
    # without the master copy the same 40 steps leave every such parameter where it was
    q = p0.clone().cuda()
    m.zero_(); v.zero_()
    g = torch.Generator().manual_seed(3)
    for step in range(1, 41):
        grad = (direction * (0.5 + torch.rand(n, generator=g))).bfloat16()
        ops.adam_step(q, grad.cuda(), m, v, step, lr, (b1, b2), eps)
    assert torch.equal(q.cpu(), p0)


def test_bounded_wait_selftest_reports_and_context_survives():
    """The failure path every tensor-core kernel shares: a bounded mbarrier wait that nothing completes
    gives up after its poll limit, sets the status word and returns; the context stays usable."""
    from memorax_b200 import _lib, ops
    assert ops.selftest_bounded_wait(polls=2) == 1
    # the device still works, and the regular status word of the wrappers is untouched
    x = torch.arange(8, device="cuda").float()
    assert float(x.sum()) == 28.0
    ops.check_status()
    assert _lib.lib.mxk_selftest_bounded_wait(None, 2, None) == -1
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert _lib.lib.mxk_selftest_bounded_wait(word.data_ptr(), 1000, None) == -2


def test_status_word_reaches_the_autograd_functions():
    """LinAttn / GatedDelta hand the kernels the per-device status word (never NULL), and check_status()
    raises once it is set."""
    from memorax_b200 import _lib, ops
    word = ops._status_word(torch.device("cuda", torch.cuda.current_device()))
    g = torch.Generator().manual_seed(0)
    q, k, v = ((torch.randn(1, 64, 1, 64, generator=g) / 8).bfloat16().cuda().requires_grad_() for _ in range(3))
    o, _, _ = ops.LinAttn.apply(q, k, v, None, None, None, 1e-6, True)
    o.float().sum().backward()
    ops.check_status()
    word.fill_(1)
    with pytest.raises(_lib.MxkError):
        ops.check_status()
    ops.check_status()   # cleared by the failed check


def _cpu_restatement(model, obs, done, target):
    """fp32 CPU forward of GTrXLStyleValueNet with the model's own parameters and the oracle's sequential
    delta rule as the mixer (the composition of blocks/residual.py:33-63, blocks/normalization.py:10-35,
    blocks/ffn.py:11-50 around the cell); returns the loss, with gradients on the returned leaves."""
    from oracle import memoroid_oracle as mo
    F = torch.nn.functional
    P = {n: p.detach().float().cpu().requires_grad_() for n, p in model.named_parameters()}
    lin = lambda x, name: F.linear(x, P[name + ".weight"], P.get(name + ".bias"))
    h = lin(obs.float(), "embed")
    B, T, _ = h.shape
    nblocks = len(model.torso.blocks)
    for i in range(0, nblocks, 2):
        cell = model.torso.blocks[i].module.module.cell
        H, hd = cell.num_heads, cell.head_dim
        pre = f"torso.blocks.{i}"
        y = F.layer_norm(h, h.shape[-1:], P[pre + ".module.norm.weight"], P[pre + ".module.norm.bias"])
        c = pre + ".module.module.cell"
        hv = lambda t: t.view(B, T, H, hd)
        q, k = F.normalize(hv(lin(y, c + ".query")), dim=-1), F.normalize(hv(lin(y, c + ".key")), dim=-1)
        b_logit, a_logit = lin(y, c + ".gate").chunk(2, -1)
        o, _ = mo.gdelta_seq(q, k, hv(lin(y, c + ".value")), torch.exp(-F.softplus(a_logit)), torch.sigmoid(b_logit),
                             torch.zeros(B, H, hd, hd), done.float())
        o = F.rms_norm(o.reshape(B, T, -1), (H * hd,), P[c + ".norm.weight"], cell.norm.eps)
        h = h + torch.sigmoid(lin(h, pre + ".gate")) * lin(o, c + ".output_projection")
        pre = f"torso.blocks.{i + 1}"
        y = F.layer_norm(h, h.shape[-1:], P[pre + ".module.norm.weight"], P[pre + ".module.norm.bias"])
        y = lin(F.gelu(lin(y, pre + ".module.module.up"), approximate="tanh"), pre + ".module.module.down")
        h = h + torch.sigmoid(lin(h, pre + ".gate")) * y
    loss = 0.5 * (lin(h, "head").squeeze(-1) - target).square().mean()
    return loss, P


def test_training_step_loss_and_gradient_match_the_fp32_restatement():
    """One training step of the value network (8 heads of 64, as the training-step configuration): the loss and
    the flat bf16 gradient the kernels produce against fp32 CPU autograd through the oracle's delta rule."""
    from memorax_b200.blocks import FlatAdamTrainer, GTrXLStyleValueNet
    torch.manual_seed(0)
    model = GTrXLStyleValueNet(obs_dim=16, d_model=128, num_heads=2, head_dim=64, layers=2).to("cuda", torch.bfloat16)
    trainer = FlatAdamTrainer(model, lr=0.0)     # lr = 0: the step leaves the parameters where they are
    g = torch.Generator().manual_seed(4)
    obs = torch.randn(2, 80, 16, generator=g).bfloat16()
    done = torch.rand(2, 80, generator=g) < 0.03
    target = torch.randn(2, 80, generator=g)
    loss = float(trainer.step(obs.cuda(), done.cuda(), target.cuda()))
    loss_ref, P = _cpu_restatement(model, obs, done, target)
    loss_ref.backward()
    assert abs(loss - float(loss_ref)) <= 2e-2 * max(1.0, abs(float(loss_ref))), (loss, float(loss_ref))
    flat_ref = torch.cat([P[n].grad.reshape(-1) for n, _ in model.named_parameters()])
    flat = trainer.flat_grad[:flat_ref.numel()].float().cpu()
    # bf16 activations through 4 blocks: compare direction and scale of the whole gradient, and every
    # element to 5 % of the gradient's max-abs
    cos = float(torch.dot(flat, flat_ref) / (flat.norm() * flat_ref.norm()))
    assert cos >= 0.995, cos
    assert float((flat - flat_ref).abs().max()) <= 5e-2 * float(flat_ref.abs().max())


def test_value_network_trains():
    from memorax_b200.blocks import FlatAdamTrainer, GTrXLStyleValueNet
    torch.manual_seed(0)
    model = GTrXLStyleValueNet(obs_dim=16, d_model=128, num_heads=2, head_dim=64, layers=2).to("cuda", torch.bfloat16)
    trainer = FlatAdamTrainer(model, lr=3e-3)
    g = torch.Generator().manual_seed(1)
    obs = torch.randn(8, 96, 16, generator=g).bfloat16().cuda()
    done = (torch.rand(8, 96, generator=g) < 0.02).cuda()
    target = obs.float().mean(-1) * 2.0
    losses = [float(trainer.step(obs, done, target)) for _ in range(30)]
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < 0.7 * losses[0], losses
    assert all(p.data_ptr() >= trainer.flat.data_ptr() for p in model.parameters())
