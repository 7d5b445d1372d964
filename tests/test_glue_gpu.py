"""The fused row-wise glue of the training-step harness (LayerNorm / RMSNorm, gated residual, per-head L2
normalisation; blocks/normalization.py:10-35, blocks/residual.py:53-59) against PyTorch fp32 on the same bf16
inputs, forward and backward, through the autograd wrappers.  Outputs are bf16: tolerance 2e-2 max-abs on O(1)
tensors (one bf16 ulp at 2 is 1.6e-2), parameter gradients 1e-2 of their max-abs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
F = torch.nn.functional


def _cmp(got, ref, tol, what):
    err = float((got.float() - ref.float()).abs().max())
    assert err <= tol * max(1.0, float(ref.float().abs().max())), f"{what}: {err:.4g}"


@pytest.mark.parametrize("rows,dim", [(7, 256), (1000, 512), (4096, 1024)])
@pytest.mark.parametrize("rms", [False, True])
def test_fused_norm_matches_torch(rows, dim, rms):
    from memorax_b200 import ops
    g = torch.Generator().manual_seed(rows + dim)
    x = (torch.randn(rows, dim, generator=g) * 1.5 + 0.3).bfloat16().cuda()
    w = (1.0 + 0.2 * torch.randn(dim, generator=g)).bfloat16().cuda()
    b = (0.1 * torch.randn(dim, generator=g)).bfloat16().cuda()
    dy = torch.randn(rows, dim, generator=g).bfloat16().cuda()
    xr, wr, br = (t.float().requires_grad_() for t in (x, w, b))
    ref = F.rms_norm(xr, (dim,), wr, 1e-6) if rms else F.layer_norm(xr, (dim,), wr, br, 1e-5)
    ref.backward(dy.float())
    xl, wl, bl = (t.clone().requires_grad_() for t in (x, w, b))
    y = ops.rms_norm(xl, wl, 1e-6) if rms else ops.layer_norm(xl, wl, bl, 1e-5)
    assert y.dtype == torch.bfloat16
    y.backward(dy)
    _cmp(y, ref, 2e-2, "y")
    _cmp(xl.grad, xr.grad, 2e-2, "dx")
    _cmp(wl.grad, wr.grad, 1e-2, "dgamma")
    if not rms:
        _cmp(bl.grad, br.grad, 1e-2, "dbeta")


def test_gated_residual_matches_torch():
    from memorax_b200 import ops
    g = torch.Generator().manual_seed(5)
    x, gate, o, dy = (torch.randn(33, 17, 512, generator=g).bfloat16().cuda() for _ in range(4))
    refs = [t.float().requires_grad_() for t in (x, gate, o)]
    ref = refs[0] + torch.sigmoid(refs[1]) * refs[2]
    ref.backward(dy.float())
    leaves = [t.clone().requires_grad_() for t in (x, gate, o)]
    y = ops.gated_residual(*leaves)
    y.backward(dy)
    _cmp(y, ref, 2e-2, "y")
    for got, r, name in zip(leaves, refs, ("dx", "dg", "do")):
        _cmp(got.grad, r.grad, 2e-2, name)


@pytest.mark.parametrize("head_dim", [64, 128])
def test_l2norm_heads_matches_torch(head_dim):
    from memorax_b200 import ops
    g = torch.Generator().manual_seed(head_dim)
    x = torch.randn(5, 40, 4 * head_dim, generator=g).bfloat16().cuda()
    dy = torch.randn(5, 40, 4, head_dim, generator=g).bfloat16().cuda()
    xr = x.float().requires_grad_()
    ref = F.normalize(xr.view(5, 40, 4, head_dim), dim=-1)
    ref.backward(dy.float())
    xl = x.clone().requires_grad_()
    y = ops.l2norm_heads(xl, head_dim)
    assert y.shape == (5, 40, 4, head_dim) and y.dtype == torch.bfloat16
    y.backward(dy)
    _cmp(y, ref, 1e-2, "y")
    _cmp(xl.grad, xr.grad, 2e-2, "dx")
    # zero vectors stay zero (norm clamped at eps), no NaN
    z = ops.l2norm_heads(torch.zeros(2, 3, head_dim, dtype=torch.bfloat16, device="cuda"), head_dim)
    assert float(z.abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(1, 8), (37, 16), (1000, 512), (16384, 2048), (4099, 520)])
def test_colsum_and_dense_bias_gradient(shape):
    """Column sums (bias gradient of a Dense layer) against an fp64 sum of the same bf16 values; bit-reproducible."""
    from memorax_b200 import ops
    rows, cols = shape
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    got = ops.colsum(x)
    ref = x.double().sum(0)
    tol = 2 ** -8 * float(ref.abs().max()) + 1e-6      # one bf16 rounding of the result
    assert float((got.double() - ref).abs().max()) <= tol
    assert torch.equal(got, ops.colsum(x))
    # through the autograd function: all three gradients against torch's own Linear
    if cols <= 520:
        lin = torch.nn.Linear(24, cols, device="cuda", dtype=torch.bfloat16)
        inp = torch.randn(3, max(rows // 3, 1), 24, device="cuda", generator=g).bfloat16().requires_grad_()
        ct = torch.randn(3, max(rows // 3, 1), cols, device="cuda", generator=g).bfloat16()
        want = torch.autograd.grad(lin(inp), [inp, lin.weight, lin.bias], ct)
        have = torch.autograd.grad(ops.dense(inp, lin.weight, lin.bias), [inp, lin.weight, lin.bias], ct)
        assert torch.equal(have[0], want[0]) and torch.equal(have[1], want[1])
        ref_b = ct.double().sum((0, 1))
        assert float((have[2].double() - ref_b).abs().max()) <= 2 ** -8 * float(ref_b.abs().max()) + 1e-6


@pytest.mark.parametrize("n", [8, 4096, 1000 * 520])
def test_gelu_tanh_form(n):
    """Fused GELU (tanh form, flax's default) and its derivative against fp64 on the same bf16 inputs: one bf16
    rounding of the result plus the approximate tanh."""
    from memorax_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(n)
    x = (torch.randn(n, device="cuda", generator=g) * 3).bfloat16().requires_grad_()
    dy = torch.randn(n, device="cuda", generator=g).bfloat16()
    y = ops.gelu(x)
    (dx,) = torch.autograd.grad(y, x, dy)
    xr = x.detach().double().requires_grad_()
    yr = torch.nn.functional.gelu(xr, approximate="tanh")
    (dxr,) = torch.autograd.grad(yr, xr, dy.double())
    assert float((y.double() - yr).abs().max()) <= 2 ** -8 * float(yr.abs().max()) + 2e-3
    assert float((dx.double() - dxr).abs().max()) <= 2 ** -8 * float(dxr.abs().max()) + 4e-3
