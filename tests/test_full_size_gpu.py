"""Size-independent properties at the benchmark configurations' FULL sizes, where the
CPU oracle is too slow to serve as the checker: splitting a sequence and threading the
carry (memoroid.py:60-91 returns the last element of the scan as the next carry),
permuting the batch, a reset at a chunk boundary, exact linearity.  All comparisons
are bit-exact: the kernels do the same arithmetic on the same values in the same order."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _linattn_inputs(seed, B=256, T=256, H=4, D=64, p_done=0.01):
    g = _gen(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)
    q, k, v = ((mk(B, T, H, D) / 8).bfloat16() for _ in range(3))
    d_o = mk(B, T, H, D).bfloat16()
    s0, z0 = mk(B, H, D, D) * 0.1, mk(B, H, D).abs() * 0.1
    done = (torch.rand(B, T, device="cuda", generator=g) < p_done).to(torch.uint8)
    return q, k, v, d_o, s0, z0, done


def test_c2_linear_attention_split_and_permutation():
    from memorax_b200 import ops
    q, k, v, d_o, s0, z0, done = _linattn_inputs(21)
    h = q.shape[1] // 2
    o, s_last, z_last, st = ops.linattn_fwd(q, k, v, s0, z0, done, save_states=True, check=True)
    # forward: one call == two calls threading the carry
    o1, s1, z1, st1 = ops.linattn_fwd(q[:, :h], k[:, :h], v[:, :h], s0, z0, done[:, :h], save_states=True)
    o2, s2, z2, st2 = ops.linattn_fwd(q[:, h:], k[:, h:], v[:, h:], s1, z1, done[:, h:], save_states=True)
    assert torch.equal(torch.cat([o1, o2], 1), o)
    assert torch.equal(s2, s_last) and torch.equal(z2, z_last)
    # backward: the state cotangent threads the other way
    dq, dk, dv, ds0, dz0 = ops.linattn_bwd(q, k, v, d_o, st, done, check=True)
    dq2, dk2, dv2, ds_mid, dz_mid = ops.linattn_bwd(q[:, h:], k[:, h:], v[:, h:], d_o[:, h:], st2, done[:, h:])
    dq1, dk1, dv1, ds0_s, dz0_s = ops.linattn_bwd(q[:, :h], k[:, :h], v[:, :h], d_o[:, :h], st1, done[:, :h],
                                                  ds_mid, dz_mid)
    for whole, a, b in ((dq, dq1, dq2), (dk, dk1, dk2), (dv, dv1, dv2)):
        assert torch.equal(torch.cat([a, b], 1), whole)
    assert torch.equal(ds0_s, ds0) and torch.equal(dz0_s, dz0)
    # sequences are independent: permuting the batch permutes the results
    perm = torch.randperm(q.shape[0], device="cuda", generator=_gen(22))
    op, sp, zp, _ = ops.linattn_fwd(q[perm], k[perm], v[perm], s0[perm], z0[perm], done[perm])
    assert torch.equal(op, o[perm]) and torch.equal(sp, s_last[perm]) and torch.equal(zp, z_last[perm])


def test_c2_reset_at_a_chunk_boundary_starts_a_fresh_sequence():
    from memorax_b200 import ops
    q, k, v, _, s0, z0, done = _linattn_inputs(23)
    h = q.shape[1] // 2
    done = done.clone()
    done[:, h] = 1          # the state before step h is discarded (memoroid.py:66-88)
    o, s_last, z_last, _ = ops.linattn_fwd(q, k, v, s0, z0, done, check=True)
    o2, s2, z2, _ = ops.linattn_fwd(q[:, h:], k[:, h:], v[:, h:], None, None, done[:, h:])
    assert torch.equal(o[:, h:], o2) and torch.equal(s_last, s2) and torch.equal(z_last, z2)


def test_c3_gated_delta_rule_split_and_permutation():
    from memorax_b200 import ops
    g = _gen(31)
    B, T, H, D = 128, 512, 8, 128
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)
    nrm = lambda x: x / x.norm(dim=-1, keepdim=True)
    q, k = nrm(mk(B, T, H, D)).bfloat16(), nrm(mk(B, T, H, D)).bfloat16()
    v, d_o = mk(B, T, H, D).bfloat16(), mk(B, T, H, D).bfloat16()
    beta = torch.sigmoid(mk(B, T, H))
    alpha = torch.exp(-torch.nn.functional.softplus(mk(B, T, H)))
    done = (torch.rand(B, T, device="cuda", generator=g) < 0.005).to(torch.uint8)
    h = T // 2
    o, s_last, st = ops.gdelta_fwd(q, k, v, alpha, beta, None, done, save_states=True, check=True)
    o1, s1, st1 = ops.gdelta_fwd(q[:, :h], k[:, :h], v[:, :h], alpha[:, :h], beta[:, :h], None, done[:, :h],
                                 save_states=True)
    o2, s2, st2 = ops.gdelta_fwd(q[:, h:], k[:, h:], v[:, h:], alpha[:, h:], beta[:, h:], s1, done[:, h:],
                                 save_states=True)
    assert torch.equal(torch.cat([o1, o2], 1), o) and torch.equal(s2, s_last)
    outs = ops.gdelta_bwd(q, k, v, alpha, beta, d_o, st, done, check=True)
    outs2 = ops.gdelta_bwd(q[:, h:], k[:, h:], v[:, h:], alpha[:, h:], beta[:, h:], d_o[:, h:], st2, done[:, h:])
    outs1 = ops.gdelta_bwd(q[:, :h], k[:, :h], v[:, :h], alpha[:, :h], beta[:, :h], d_o[:, :h], st1, done[:, :h],
                           outs2[5])
    for i in range(5):   # dq, dk, dv, dalpha, dbeta
        assert torch.equal(torch.cat([outs1[i], outs2[i]], 1), outs[i]), i
    assert torch.equal(outs1[5], outs[5])
    perm = torch.randperm(B, device="cuda", generator=_gen(32))
    op, sp, _ = ops.gdelta_fwd(q[perm], k[perm], v[perm], alpha[perm], beta[perm], None, done[perm])
    assert torch.equal(op, o[perm]) and torch.equal(sp, s_last[perm])


def test_c4_complex_lru_split_and_linearity():
    from memorax_b200 import ops
    g = _gen(41)
    B, T, D = 1024, 1024, 512
    mag = 0.9 + 0.099 * torch.rand(D, device="cuda", generator=g)
    lam = torch.polar(mag, 6.2831853 * torch.rand(D, device="cuda", generator=g))
    bu = torch.view_as_complex(torch.randn(B, T, D, 2, device="cuda", generator=g))
    done = (torch.rand(B, T, device="cuda", generator=g) < 0.002).to(torch.uint8)
    h, _ = ops.linrec_fwd(lam, bu, None, None, done, want_decay=False)
    cut = 384
    h1, _ = ops.linrec_fwd(lam, bu[:, :cut], None, None, done[:, :cut], want_decay=False)
    h2, _ = ops.linrec_fwd(lam, bu[:, cut:], h1[:, -1].contiguous(), None, done[:, cut:], want_decay=False)
    assert torch.equal(h[:, :cut], h1) and torch.equal(h[:, cut:], h2)
    del h1, h2
    # the recurrence is linear in its input: a power-of-two scale is exact in floating point
    hs, _ = ops.linrec_fwd(lam, bu * 4, None, None, done, want_decay=False)
    assert torch.equal(hs, h * 4)
