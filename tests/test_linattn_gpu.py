"""GPU parity of chunked linear attention against the fp64 CPU oracle, through
the C-ABI.  Inputs are bf16; tolerance 2e-2 max-abs on outputs and gradients
(state compared relative to its max-abs)."""
import numpy as np
import pytest
import torch

from oracle import memoroid_oracle as mo

pytestmark = pytest.mark.gpu
ATOL = 2e-2


def make_case(seed, bsz, steps, heads, dim, p_done, zero_state=False):
    gen = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=gen)
    q = (mk(bsz, steps, heads, dim) / 8).bfloat16()
    k = (mk(bsz, steps, heads, dim) / 8).bfloat16()
    v = (mk(bsz, steps, heads, dim) / 8).bfloat16()
    s0 = torch.zeros(bsz, heads, dim, dim) if zero_state else mk(bsz, heads, dim, dim) * 0.1
    z0 = torch.zeros(bsz, heads, dim) if zero_state else mk(bsz, heads, dim).abs() * 0.1
    done = torch.rand(bsz, steps, generator=gen) < p_done
    if steps > 3:
        done[0, 0] = True
        done[-1, 1:3] = True
    return q, k, v, s0, z0, done


def max_abs(a, b):
    return float((a.detach().double().cpu() - b.detach().double().cpu()).abs().max())


@pytest.mark.parametrize("shape,p_done", [((2, 64, 2, 64), 0.0), ((2, 64, 2, 64), 0.05), ((3, 256, 4, 64), 0.01),
                                          ((2, 1, 1, 64), 0.0), ((2, 7, 3, 64), 0.3), ((2, 65, 2, 64), 0.05),
                                          ((1, 200, 2, 64), 0.02), ((2, 128, 1, 64), 1.0),
                                          ((1, 1100, 1, 64), 0.003),   # 18 chunks
                                          # head dims below the 64-column tile (columns past d are zero-filled)
                                          ((2, 130, 2, 32), 0.03), ((2, 70, 3, 16), 0.05), ((3, 64, 2, 8), 0.0),
                                          ((1, 200, 2, 48), 0.02)])
def test_linattn_fwd(shape, p_done):
    from memorax_b200 import ops
    q, k, v, s0, z0, done = make_case(sum(shape), *shape, p_done)
    o_ref, s_ref, z_ref = mo.linattn_seq(q.double(), k.double(), v.double(), s0.double(), z0.double(), done.double())
    o, s_last, z_last, _ = ops.linattn_fwd(q.cuda(), k.cuda(), v.cuda(), s0.cuda(), z0.cuda(), done.cuda(), check=True)
    assert max_abs(o.float(), o_ref) <= ATOL
    assert max_abs(s_last, s_ref) <= 1e-2 * max(1.0, float(s_ref.abs().max()))
    assert max_abs(z_last, z_ref) <= 1e-2 * max(1.0, float(z_ref.abs().max()))


def test_linattn_golden_vectors(golden):
    """Reference-source vectors (head_dim 4 there) embedded in a 64-wide head:
    zero-padded feature columns contribute phi(0)=1 to q.k sums, so the feature
    map is applied on the host and padded with zeros afterwards."""
    from memorax_b200 import ops
    g = golden
    bsz, steps, heads, hd = g["la_q"].shape
    pad = lambda x: torch.nn.functional.pad(torch.from_numpy(x).float(), (0, 64 - hd))
    fq, fk = mo.elu_plus_one(g["la_q"]), mo.elu_plus_one(g["la_k"])
    s0 = torch.zeros(bsz, heads, 64, 64)
    s0[:, :, :hd, :hd] = torch.from_numpy(g["la_c_S"][:, 0]).float()
    z0 = pad(g["la_c_z"][:, 0])
    done = torch.from_numpy(g["la_done"]).cuda()
    o, s_last, z_last, _ = ops.linattn_fwd(pad(fq).cuda(), pad(fk).cuda(), pad(g["la_v"]).cuda(), s0.cuda(), z0.cuda(),
                                           done, feature_map=False, check=True)
    assert max_abs(o[..., :hd].float(), torch.from_numpy(g["la_y"])) <= ATOL
    s_ref = torch.from_numpy(g["la_n_S"][:, 0])
    assert max_abs(s_last[:, :, :hd, :hd], s_ref) <= 1e-2 * float(s_ref.abs().max())
    z_ref = torch.from_numpy(g["la_n_z"][:, 0])
    assert max_abs(z_last[..., :hd], z_ref) <= 1e-2 * float(z_ref.abs().max())


def test_linattn_golden_vectors_at_head_dim_8(golden):
    """The reference-source vectors (head_dim 4) embedded in the smallest native head (8 columns): as in the
    64-wide replay the host applies the feature map and pads with zeros (a padded raw column would contribute
    phi(0) = 1), but the call goes through the d = 8 path of the kernels (tensor maps over 8-column tensors,
    zero-filled tiles, bounded state I/O)."""
    from memorax_b200 import ops
    g = golden
    bsz, steps, heads, hd = g["la_q"].shape
    pad = lambda x: torch.nn.functional.pad(torch.from_numpy(x).float(), (0, 8 - hd))
    fq, fk = mo.elu_plus_one(g["la_q"]), mo.elu_plus_one(g["la_k"])
    s0 = torch.zeros(bsz, heads, 8, 8)
    s0[:, :, :hd, :hd] = torch.from_numpy(g["la_c_S"][:, 0]).float()
    z0 = pad(g["la_c_z"][:, 0])
    done = torch.from_numpy(g["la_done"]).cuda()
    o, s_last, z_last, _ = ops.linattn_fwd(pad(fq).cuda(), pad(fk).cuda(), pad(g["la_v"]).cuda(), s0.cuda(), z0.cuda(),
                                           done, feature_map=False, check=True)
    assert max_abs(o[..., :hd].float(), torch.from_numpy(g["la_y"])) <= ATOL
    s_ref = torch.from_numpy(g["la_n_S"][:, 0])
    assert max_abs(s_last[:, :, :hd, :hd], s_ref) <= 1e-2 * float(s_ref.abs().max())
    z_ref = torch.from_numpy(g["la_n_z"][:, 0])
    assert max_abs(z_last[..., :hd], z_ref) <= 1e-2 * float(z_ref.abs().max())


def test_linattn_split_sequence_matches_single_call():
    from memorax_b200 import ops
    q, k, v, s0, z0, done = make_case(3, 2, 192, 2, 64, 0.02)
    cu = lambda t: t.cuda()
    o, s_last, z_last, _ = ops.linattn_fwd(cu(q), cu(k), cu(v), cu(s0), cu(z0), cu(done))
    o1, s1, z1, _ = ops.linattn_fwd(cu(q[:, :128]), cu(k[:, :128]), cu(v[:, :128]), cu(s0), cu(z0), cu(done[:, :128]))
    o2, s2, z2, _ = ops.linattn_fwd(cu(q[:, 128:]), cu(k[:, 128:]), cu(v[:, 128:]), s1, z1, cu(done[:, 128:]))
    assert torch.equal(torch.cat([o1, o2], 1), o)   # chunk-aligned split: identical arithmetic
    assert torch.equal(s2, s_last) and torch.equal(z2, z_last)


@pytest.mark.parametrize("shape,p_done", [((2, 64, 2, 64), 0.0), ((2, 64, 2, 64), 0.05), ((2, 256, 4, 64), 0.01),
                                          ((2, 1, 1, 64), 0.0), ((2, 7, 3, 64), 0.3), ((2, 65, 2, 64), 0.05),
                                          ((1, 200, 2, 64), 0.02), ((2, 128, 1, 64), 1.0),
                                          ((1, 1100, 1, 64), 0.003),   # 18 chunks
                                          ((2, 130, 2, 32), 0.03), ((2, 70, 3, 16), 0.05), ((3, 64, 2, 8), 0.0),
                                          ((1, 200, 2, 48), 0.02)])
def test_linattn_bwd(shape, p_done):
    from memorax_b200 import ops
    q, k, v, s0, z0, done = make_case(sum(shape) + 1, *shape, p_done)
    gen = torch.Generator().manual_seed(99)
    d_o = torch.randn(*shape, generator=gen).bfloat16()
    ds_last = torch.randn(*s0.shape, generator=gen) * 0.1
    dz_last = torch.randn(*z0.shape, generator=gen) * 0.1
    leaves = [t.double().requires_grad_() for t in (q, k, v, s0, z0)]
    o_ref, s_ref, z_ref = mo.linattn_seq(*leaves, done.double())
    ((o_ref * d_o.double()).sum() + (s_ref * ds_last.double()).sum() + (z_ref * dz_last.double()).sum()).backward()
    cu = lambda t: t.cuda()
    _, _, _, states = ops.linattn_fwd(cu(q), cu(k), cu(v), cu(s0), cu(z0), cu(done), save_states=True, check=True)
    outs = ops.linattn_bwd(cu(q), cu(k), cu(v), cu(d_o), states, cu(done), cu(ds_last), cu(dz_last), check=True)
    for got, leaf, name in zip(outs, leaves, ["dq", "dk", "dv", "ds0", "dz0"]):
        ref = leaf.grad
        tol = ATOL if name in ("dq", "dk", "dv") else 1e-2 * max(1.0, float(ref.abs().max()))
        err = max_abs(got.float(), ref)
        assert err <= tol, f"{name}: {err:.4f} > {tol:.4f} (ref max {float(ref.abs().max()):.3f})"


def test_linattn_autograd_function():
    from memorax_b200 import ops
    q, k, v, s0, z0, done = make_case(5, 2, 96, 2, 64, 0.03)
    w = torch.randn(2, 96, 2, 64, generator=torch.Generator().manual_seed(1))
    leaves = [t.double().requires_grad_() for t in (q, k, v, s0, z0)]
    o_ref, _, _ = mo.linattn_seq(*leaves, done.double())
    (o_ref * w.double()).sum().backward()
    dev = [t.cuda().requires_grad_() for t in (q, k, v, s0, z0)]
    o, _, _ = ops.LinAttn.apply(*dev, done.cuda(), 1e-6, True)
    (o.float() * w.cuda()).sum().backward()
    for got, leaf in zip(dev, leaves):
        tol = ATOL if got.dtype == torch.bfloat16 else 1e-2 * max(1.0, float(leaf.grad.abs().max()))
        assert max_abs(got.grad.float(), leaf.grad) <= tol
