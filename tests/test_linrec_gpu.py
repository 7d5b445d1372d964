"""GPU parity of the diagonal recurrences (real, complex, log-space) against
the fp64 CPU oracle, through the C-ABI.  Tolerance: 1e-5 of the max-abs value
of each tensor (fp32 recurrences)."""
import numpy as np
import pytest
import torch

from oracle import memoroid_oracle as mo

pytestmark = pytest.mark.gpu
REL = 1e-5


def close(got, want, rel=REL, what=""):
    got = got.detach().cpu()
    want = want.detach().cpu().to(got.dtype)
    assert torch.isfinite(torch.view_as_real(got) if got.is_complex() else got).all(), what
    scale = max(float(want.abs().max()), 1e-30)
    err = float((got - want).abs().max()) / scale
    assert err <= rel, f"{what}: rel err {err:.3e} > {rel}"


def make_done(gen, bsz, steps, p):
    done = (torch.rand(bsz, steps, generator=gen) < p)
    if steps > 2:
        done[0, 0] = True
        done[-1, 1:3] = True
    return done


def rnd(gen, *shape, cplx=False):
    x = torch.randn(*shape, generator=gen, dtype=torch.float64)
    if cplx:
        x = torch.complex(x, torch.randn(*shape, generator=gen, dtype=torch.float64))
    return x


# the last three reach the one-thread-per-channel kernels on grids of at most three blocks per SM (deeper unroll,
# T not a multiple of it): narrow packs with T beyond the time-split range, and 16-byte packs
SHAPES = [(2, 1, 4), (3, 7, 5), (4, 33, 64), (64, 128, 256), (2, 130, 1024), (2, 300, 96), (40, 43, 8192),
          (20, 43, 8192)]


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("tinv", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_linrec_fwd_bwd(shape, tinv, cplx):
    from memorax_b200 import ops
    bsz, steps, dim = shape
    gen = torch.Generator().manual_seed(1234 + steps + dim)
    a = rnd(gen, *((dim,) if tinv else shape), cplx=cplx)
    a = a / (1.0 + a.abs()) * 1.2  # |a| < 1.2, mostly contracting
    b = rnd(gen, *shape, cplx=cplx)
    h0, a0 = rnd(gen, bsz, dim, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)
    done = make_done(gen, bsz, steps, 0.05)
    gh, gh_last = rnd(gen, *shape, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)

    ar, br, h0r = a.clone().requires_grad_(), b.clone().requires_grad_(), h0.clone().requires_grad_()
    h_ref, a_last_ref = mo.linrec_seq(ar, br, h0r, done.double(), a0)
    # real loss whose JAX cotangents are exactly (gh, gh_last): L = Re sum(ct * out)
    loss = (gh * h_ref).sum() + (gh_last * h_ref[:, -1]).sum()
    loss = loss.real if cplx else loss
    loss.backward()

    dt = torch.complex64 if cplx else torch.float32
    dev = "cuda"
    h, a_last = ops.linrec_fwd(a.to(dt).to(dev), b.to(dt).to(dev), h0.to(dt).to(dev), a0.to(dt).to(dev), done.to(dev))
    close(h, h_ref, what="h")
    close(a_last, a_last_ref, what="a_last")

    gb, ga, gh0 = ops.linrec_bwd(a.to(dt).to(dev), h, h0.to(dt).to(dev), done.to(dev), gh.to(dt).to(dev),
                                 gh_last.to(dt).to(dev))
    rel = REL * (10 if tinv else 1)  # the (D,) reduction sums B*T terms in fp32
    close(gb, mo.jax_cotangent(br.grad), what="gb")
    close(ga, mo.jax_cotangent(ar.grad), rel=rel, what="ga")
    close(gh0, mo.jax_cotangent(h0r.grad), what="gh0")


@pytest.mark.parametrize("cplx", [False, True])
def test_linrec_autograd_function_matches_torch_convention(cplx):
    from memorax_b200 import ops
    bsz, steps, dim = 3, 19, 8
    gen = torch.Generator().manual_seed(5)
    a = rnd(gen, dim, cplx=cplx) * 0.5
    b, h0 = rnd(gen, bsz, steps, dim, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)
    done = make_done(gen, bsz, steps, 0.1)
    w = rnd(gen, bsz, steps, dim, cplx=cplx)

    def run(a_, b_, h0_, fn):
        a_, b_, h0_ = a_.requires_grad_(), b_.requires_grad_(), h0_.requires_grad_()
        h = fn(a_, b_, h0_)
        loss = (h * w.to(h.device).to(h.dtype)).sum()
        (loss.real if cplx else loss).backward()
        return h, a_.grad, b_.grad, h0_.grad

    ref = run(a.clone(), b.clone(), h0.clone(), lambda a_, b_, h0_: mo.linrec_seq(a_, b_, h0_, done.double())[0])
    dt = torch.complex64 if cplx else torch.float32
    got = run(a.to(dt).cuda(), b.to(dt).cuda(), h0.to(dt).cuda(),
              lambda a_, b_, h0_: ops.LinRec.apply(a_, b_, h0_, None, done.cuda())[0])
    for g, r, name in zip(got, ref, ["h", "ga", "gb", "gh0"]):
        close(g, r, rel=1e-4 if name == "ga" else REL, what=name)


def test_linrec_optional_arguments_and_no_done():
    from memorax_b200 import ops
    gen = torch.Generator().manual_seed(9)
    a, b = torch.rand(2, 6, 8, generator=gen, dtype=torch.float64), rnd(gen, 2, 6, 8)
    h_ref, acc_ref = mo.linrec_seq(a, b, torch.zeros(2, 8, dtype=torch.float64), torch.zeros(2, 6, dtype=torch.float64))
    h, acc = ops.linrec_fwd(a.float().cuda(), b.float().cuda())
    close(h, h_ref)
    close(acc, acc_ref)


def test_linrec_split_sequence_is_bit_identical():
    """One call over T == two calls threading the carry (memoroid.py:89)."""
    from memorax_b200 import ops
    gen = torch.Generator().manual_seed(11)
    # wide enough for the streaming kernel (the time-split kernel for small B*D chains affine
    # maps across segments and agrees to rounding, not bit for bit)
    a, b = torch.rand(40, 40, 8192, generator=gen).cuda(), torch.randn(40, 40, 8192, generator=gen).cuda()
    done = make_done(gen, 40, 40, 0.1).cuda()
    h, acc = ops.linrec_fwd(a, b, None, None, done)
    h1, acc1 = ops.linrec_fwd(a[:, :13].contiguous(), b[:, :13].contiguous(), None, None, done[:, :13])
    h2, acc2 = ops.linrec_fwd(a[:, 13:].contiguous(), b[:, 13:].contiguous(), h1[:, -1].contiguous(), acc1, done[:, 13:])
    assert torch.equal(torch.cat([h1, h2], 1), h)
    assert torch.equal(acc2, acc)


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("steps", [32, 33, 40, 128, 255, 256])
@pytest.mark.parametrize("tinv", [False, True])
def test_linrec_time_split_kernels(steps, tinv, cplx):
    """Small B*D with moderate T takes the time-split forward and backward kernels (real and complex)."""
    from memorax_b200 import ops
    gen = torch.Generator().manual_seed(steps)
    bsz, dim = 5, 48
    a = rnd(gen, *((dim,) if tinv else (bsz, steps, dim)), cplx=cplx)
    a = a / (1.0 + a.abs()) * 1.1
    b, h0, a0 = rnd(gen, bsz, steps, dim, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)
    gh, gh_last = rnd(gen, bsz, steps, dim, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)
    done = make_done(gen, bsz, steps, 0.08)
    ar, br, h0r = a.clone().requires_grad_(), b.clone().requires_grad_(), h0.clone().requires_grad_()
    h_ref, acc_ref = mo.linrec_seq(ar, br, h0r, done.double(), a0)
    loss = (gh * h_ref).sum() + (gh_last * h_ref[:, -1]).sum()
    (loss.real if cplx else loss).backward()
    dt = torch.complex64 if cplx else torch.float32
    cu = lambda t: t.to(dt).cuda()
    h, acc = ops.linrec_fwd(cu(a), cu(b), cu(h0), cu(a0), done.cuda())
    close(h, h_ref, what="h")
    close(acc, acc_ref, what="a_last")
    gb, ga, gh0 = ops.linrec_bwd(cu(a), h, cu(h0), done.cuda(), cu(gh), cu(gh_last))
    close(gb, mo.jax_cotangent(br.grad), what="gb")
    close(ga, mo.jax_cotangent(ar.grad), rel=REL * (10 if tinv else 1), what="ga")
    close(gh0, mo.jax_cotangent(h0r.grad), what="gh0")
    # no carried state, no decay gradient wanted, no resets
    h2, _ = ops.linrec_fwd(cu(a), cu(b), None, None, None)
    h2_ref, _ = mo.linrec_seq(a, b, torch.zeros_like(h0), torch.zeros(bsz, steps, dtype=torch.float64), None)
    close(h2, h2_ref, what="h without carry")


def test_linrec_rejects_bad_arguments():
    from memorax_b200 import _lib
    st = _lib.lib.mxk_linrec_f32_fwd(None, 0, None, None, None, None, None, None, 1, 1, 1, None)
    assert st == -1 and "NULL" in _lib.status_string(st)
    x = torch.zeros(64, device="cuda")
    p = x.data_ptr()
    assert _lib.lib.mxk_linrec_f32_fwd(p, 0, p, None, None, None, p, None, 0, 4, 4, None) == -2
    assert _lib.lib.mxk_linrec_f32_fwd(p + 2, 0, p, None, None, None, p, None, 1, 4, 4, None) == -3
    # time-invariant decay gradient without a workspace
    assert _lib.lib.mxk_linrec_f32_bwd(p, 1, p, None, None, p, None, p, p, None, None, 0, 1, 4, 4, None) == -5


@pytest.mark.parametrize("shape", [(2, 1, 4), (3, 9, 6), (8, 65, 256), (64, 40, 1024)])
@pytest.mark.parametrize("neg_inf_carry", [True, False])
def test_loglinrec_fwd_bwd(shape, neg_inf_carry):
    from memorax_b200 import ops
    bsz, steps, dim = shape
    gen = torch.Generator().manual_seed(77 + steps)
    ls = rnd(gen, *shape) * 2
    d = -torch.nn.functional.softplus(rnd(gen, *shape) * 2)
    x0 = torch.full((bsz, dim), -float("inf"), dtype=torch.float64) if neg_inf_carry else rnd(gen, bsz, dim)
    a0 = -rnd(gen, bsz, dim).abs()
    done = make_done(gen, bsz, steps, 0.05)
    gx, gy, gx_last = rnd(gen, *shape), rnd(gen, *shape), rnd(gen, bsz, dim)

    lsr, dr = ls.clone().requires_grad_(), d.clone().requires_grad_()
    x0r = x0.clone().requires_grad_(not neg_inf_carry)
    x_ref, a_ref = mo.mingru_seq(lsr, dr, x0r, done.double(), a0)
    ((gx * x_ref).sum() + (gy * x_ref.exp()).sum() + (gx_last * x_ref[:, -1]).sum()).backward()

    cu = lambda t: t.float().cuda()
    x, y, a_last = ops.loglinrec_fwd(cu(ls), cu(d), cu(x0), cu(a0), done.cuda())
    assert not torch.isnan(x).any()
    close(x, x_ref, what="x")
    close(y, x_ref.exp(), what="y")
    close(a_last, a_ref, what="a_last")
    gls, gd, gx0 = ops.loglinrec_bwd(cu(d), x, cu(x0), done.cuda(), cu(gx), cu(gy), cu(gx_last))
    assert not (torch.isnan(gls).any() or torch.isnan(gd).any() or torch.isnan(gx0).any())
    close(gls, lsr.grad, rel=1e-4, what="gls")
    close(gd, dr.grad, rel=1e-4, what="gd")
    if not neg_inf_carry:
        close(gx0, x0r.grad, rel=1e-4, what="gx0")


def test_golden_vectors_through_cuda(golden):
    """The vectors produced by the reference's own source, replayed on the GPU."""
    from memorax_b200 import ops
    g = golden
    c64 = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(torch.complex64).cuda()
    f32 = lambda x: torch.from_numpy(np.ascontiguousarray(x)).float().cuda()
    done = torch.from_numpy(g["lru_done"]).cuda()
    h, a_last = ops.linrec_fwd(c64(g["lru_z_decay"]), c64(g["lru_z_state"]), c64(g["lru_c_state"][:, 0]),
                               c64(g["lru_c_decay"][:, 0]), done)
    close(h, torch.from_numpy(g["lru_h_state"]), what="lru h")
    close(a_last, torch.from_numpy(g["lru_n_decay"][:, 0]), what="lru decay")
    x, y, a_last = ops.loglinrec_fwd(f32(g["gru_z_state"]), f32(g["gru_z_decay"]), None, None,
                                     torch.from_numpy(g["gru_done"]).cuda())
    close(x, torch.from_numpy(g["gru_h_state"]), what="gru x")
    close(y, torch.from_numpy(g["gru_y"]), what="gru y")
    close(a_last, torch.from_numpy(g["gru_n_decay"][:, 0]), what="gru decay")
    bsz, steps, hid, psz = g["rt_jac"].shape
    a = np.repeat(g["rt_decay"], psz, axis=-1)
    h, _ = ops.linrec_fwd(f32(a), f32(g["rt_jac"].reshape(bsz, steps, -1)), f32(g["rt_sens"].reshape(bsz, -1)), None,
                          torch.from_numpy(g["rt_done"]).cuda(), want_decay=False)
    close(h[:, -1], torch.from_numpy(g["rt_next"].reshape(bsz, -1)), what="rtrl")


@pytest.mark.parametrize("shape,groups", [((3, 9, 256), 2), ((2, 37, 1024), 4), ((4, 130, 2048), 8), ((2, 5, 128), 1)])
def test_linrec_grouped_decay_fwd_bwd(shape, groups):
    """One decay per group of channels (MambaCell's per-head decay, mamba.py:109-122) against the oracle run on
    the expanded decay: states, the carry's decay leaf per group, and the cotangents with the decay gradient
    reduced over each group."""
    from memorax_b200 import ops
    bsz, steps, dim = shape
    per = dim // groups
    gen = torch.Generator().manual_seed(dim + steps)
    a = torch.rand(bsz, steps, groups, generator=gen, dtype=torch.float64) * 0.6 + 0.4
    b, h0 = rnd(gen, bsz, steps, dim), rnd(gen, bsz, dim)
    a0 = torch.rand(bsz, groups, generator=gen, dtype=torch.float64)
    gh, gh_last = rnd(gen, bsz, steps, dim), rnd(gen, bsz, dim)
    done = make_done(gen, bsz, steps, 0.08)
    ar, br, h0r = a.clone().requires_grad_(), b.clone().requires_grad_(), h0.clone().requires_grad_()
    h_ref, acc_ref = mo.linrec_seq(ar.repeat_interleave(per, dim=-1), br, h0r, done.double(), a0.repeat_interleave(per, dim=-1))
    ((h_ref * gh).sum() + (h_ref[:, -1] * gh_last).sum()).backward()
    cu = lambda t: t.float().cuda()
    assert ops.grouped_decay_supported(dim, groups)
    h, a_last = ops.linrec_grouped_fwd(cu(a), cu(b), cu(h0), cu(a0), done.cuda())
    close(h, h_ref, what="h")
    close(a_last, acc_ref[:, ::per], what="a_last")
    gb, ga, gh0 = ops.linrec_grouped_bwd(cu(a), h, cu(h0), done.cuda(), cu(gh), cu(gh_last))
    close(gb, br.grad, what="gb")
    close(ga, ar.grad, rel=1e-4, what="ga")     # a sum over `per` channels
    close(gh0, h0r.grad, what="gh0")
    # default carry and the autograd Function
    leaves = [cu(a).requires_grad_(), cu(b).requires_grad_()]
    h2, _ = ops.LinRecGrouped.apply(leaves[0], leaves[1], None, None, done.cuda())
    h_ref2, _ = mo.linrec_seq(ar.detach().repeat_interleave(per, dim=-1), b, torch.zeros(bsz, dim, dtype=torch.float64), done.double())
    close(h2, h_ref2, what="h default carry")
    (h2 * cu(gh)).sum().backward()
    assert leaves[0].grad.shape == (bsz, steps, groups)


def test_linrec_grouped_rejects_narrow_groups():
    from memorax_b200 import _lib
    x = torch.zeros(64 * 96, device="cuda")
    p = x.data_ptr()
    assert _lib.lib.mxk_linrec_f32_grouped_fwd(p, p, None, None, None, p, None, 1, 1, 96, 2, None) == -4
    assert _lib.lib.mxk_linrec_f32_grouped_fwd(p, p, None, None, None, p, None, 1, 1, 100, 3, None) == -2


@pytest.mark.parametrize("shape", [(3, 9, 6), (8, 65, 256), (64, 40, 1024)])
def test_mingru_fused_gate_math(shape):
    """MinGRU's gate math (min_gru.py:52-61) inside the scan kernels: the Dense pre-activations z, h~ in, log
    states / read-out out, cotangents of z and h~ back -- against fp64 autograd through the same formulas and
    the oracle's sequential scan."""
    from memorax_b200 import ops
    bsz, steps, dim = shape
    gen = torch.Generator().manual_seed(31 + steps)
    z, ht = rnd(gen, *shape) * 2.5, rnd(gen, *shape) * 2.0
    x0, a0 = rnd(gen, bsz, dim), -rnd(gen, bsz, dim).abs()
    done = make_done(gen, bsz, steps, 0.05)
    gx, gy = rnd(gen, *shape), rnd(gen, *shape)
    zr, hr, x0r = z.clone().requires_grad_(), ht.clone().requires_grad_(), x0.clone().requires_grad_()
    sp = torch.nn.functional.softplus
    log_state = -sp(-zr) + torch.where(hr >= 0, torch.log(torch.relu(hr) + 0.5), -sp(-hr))
    x_ref, a_ref = mo.mingru_seq(log_state, -sp(zr), x0r, done.double(), a0)
    ((gx * x_ref).sum() + (gy * x_ref.exp()).sum()).backward()
    cu = lambda t: t.float().cuda()
    leaves = [cu(z).requires_grad_(), cu(ht).requires_grad_(), cu(x0).requires_grad_()]
    x, y, a_last = ops.MinGRUFused.apply(*leaves, cu(a0), done.cuda())
    close(x, x_ref, what="x")
    close(y, x_ref.exp(), what="y")
    close(a_last, a_ref, what="a_last")
    ((x * cu(gx)).sum() + (y * cu(gy)).sum()).backward()
    close(leaves[0].grad, zr.grad, rel=1e-4, what="gz")
    close(leaves[1].grad, hr.grad, rel=1e-4, what="gh")
    close(leaves[2].grad, x0r.grad, rel=1e-4, what="gx0")
    # default (-inf) carry: finite everywhere
    x2, y2, _ = ops.MinGRUFused.apply(cu(z), cu(ht), None, None, done.cuda())
    assert torch.isfinite(y2).all() and not torch.isnan(x2).any()


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("tinv", [False, True])
@pytest.mark.parametrize("shape", [(2, 1, 4), (3, 7, 5), (5, 70, 48), (40, 43, 8192)])
def test_linrec_last_state_only(shape, tinv, cplx):
    """The last-state-only entry points (what the RTRL propagation returns, memoroid.py:114-141) against the
    fp64 oracle's final state, with resets, a carried state and T not a multiple of the unroll depth."""
    from memorax_b200 import ops
    bsz, steps, dim = shape
    gen = torch.Generator().manual_seed(77 + steps + dim)
    a = rnd(gen, *((dim,) if tinv else shape), cplx=cplx)
    a = a / (1.0 + a.abs()) * 1.1
    b, h0 = rnd(gen, *shape, cplx=cplx), rnd(gen, bsz, dim, cplx=cplx)
    done = make_done(gen, bsz, steps, 0.05)
    h_ref, _ = mo.linrec_seq(a, b, h0, done.double())
    dt = torch.complex64 if cplx else torch.float32
    last = ops.linrec_last(a.to(dt).cuda(), b.to(dt).cuda(), h0.to(dt).cuda(), done.cuda())
    close(last, h_ref[:, -1], what="h_T")
    last0 = ops.linrec_last(a.to(dt).cuda(), b.to(dt).cuda(), None, None)
    h_ref0, _ = mo.linrec_seq(a, b, torch.zeros_like(h0), torch.zeros(bsz, steps, dtype=torch.float64))
    close(last0, h_ref0[:, -1], what="h_T without carry and resets")


def test_linrec_grouped_last_state_only():
    from memorax_b200 import ops
    gen = torch.Generator().manual_seed(5)
    bsz, steps, groups, group = 6, 37, 3, 256
    a = torch.rand(bsz, steps, groups, generator=gen, dtype=torch.float64)
    b, h0 = rnd(gen, bsz, steps, groups * group), rnd(gen, bsz, groups * group)
    done = make_done(gen, bsz, steps, 0.08)
    h_ref, _ = mo.linrec_seq(a.repeat_interleave(group, dim=-1), b, h0, done.double())
    last = ops.linrec_grouped_last(a.float().cuda(), b.float().cuda(), h0.float().cuda(), done.cuda())
    close(last, h_ref[:, -1], what="h_T")
    full, _ = ops.linrec_grouped_fwd(a.float().cuda(), b.float().cuda(), h0.float().cuda(), None, done.cuda(), want_decay=False)
    assert torch.equal(last, full[:, -1])
