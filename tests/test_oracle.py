"""CPU checks of the oracle itself: against the golden vectors produced by the
reference's own source, and layer 2 (sequential closed forms) against layer 1
(the reference's prefix-scan formulation)."""
import numpy as np
import pytest
import torch

from oracle import memoroid_oracle as mo

T64 = lambda x: torch.from_numpy(np.ascontiguousarray(x))
TOL = dict(rtol=1e-11, atol=1e-11)


# ---------------------------------------------------------------- golden pins
def test_golden_lru_scan_and_read(golden):
    g = golden
    h, a_last = mo.linrec_seq(T64(g["lru_z_decay"]), T64(g["lru_z_state"]), T64(g["lru_c_state"][:, 0]),
                              T64(g["lru_done"]), T64(g["lru_c_decay"][:, 0]))
    np.testing.assert_allclose(h.numpy(), g["lru_h_state"], **TOL)
    np.testing.assert_allclose(h[:, -1:].numpy(), g["lru_n_state"], **TOL)
    np.testing.assert_allclose(a_last[:, None].numpy(), g["lru_n_decay"], **TOL)
    # read-out of lru.py:97-102 on top of the scanned state
    y = np.einsum("fh,bth->btf", g["lru_C"], h.numpy()).real + g["lru_D"] * g["lru_x"]
    np.testing.assert_allclose(y, g["lru_y"], **TOL)


def test_golden_lru_time_invariant_decay_and_default_carry(golden):
    g = golden
    lam = T64(g["lru_z_decay"][0, 0])
    assert np.all(g["lru_z_decay"] == g["lru_z_decay"][0, 0])  # lru.py:86 broadcasts one lambda
    bsz, _, hid = g["lru_z_state"].shape
    h0 = torch.zeros(bsz, hid, dtype=torch.complex128)
    h, a_last = mo.linrec_seq(lam, T64(g["lru_z_state"]), h0, T64(g["lru_done"]))
    np.testing.assert_allclose(h[:, -1:].numpy(), g["lru_default_n_state"], **TOL)
    np.testing.assert_allclose(a_last[:, None].numpy(), g["lru_default_n_decay"], **TOL)


def test_golden_mingru(golden):
    g = golden
    bsz, _, feat = g["gru_z_state"].shape
    x0 = torch.full((bsz, feat), -float("inf"), dtype=torch.float64)
    x, a_last = mo.mingru_seq(T64(g["gru_z_state"]), T64(g["gru_z_decay"]), x0, T64(g["gru_done"]))
    assert not torch.isnan(x).any()
    np.testing.assert_allclose(x.numpy(), g["gru_h_state"], **TOL)
    np.testing.assert_allclose(torch.exp(x).numpy(), g["gru_y"], **TOL)
    np.testing.assert_allclose(a_last[:, None].numpy(), g["gru_n_decay"], **TOL)
    x, a_last = mo.mingru_seq(T64(g["gru_z_state"]), T64(g["gru_z_decay"]), T64(g["gru_c1_state"][:, 0]),
                              T64(g["gru_done"]), T64(g["gru_c1_decay"][:, 0]))
    np.testing.assert_allclose(x.numpy(), g["gru_h1_state"], **TOL)
    np.testing.assert_allclose(a_last[:, None].numpy(), g["gru_n1_decay"], **TOL)


@pytest.mark.parametrize("variant", ["", "neg_"])
def test_golden_linear_attention(golden, variant):
    g = golden
    z0 = g["la_c_z"] if variant == "" else g["la_neg_c_z"]
    o, s_last, z_last = mo.linattn_seq(T64(g["la_q"]), T64(g["la_k"]), T64(g["la_v"]), T64(g["la_c_S"][:, 0]),
                                       T64(z0[:, 0]), T64(g["la_done"]))
    np.testing.assert_allclose(o.numpy(), g["la_y"] if variant == "" else g["la_neg_y"], rtol=1e-9, atol=1e-9)
    if variant == "":
        np.testing.assert_allclose(s_last[:, None].numpy(), g["la_n_S"], **TOL)
        np.testing.assert_allclose(z_last[:, None].numpy(), g["la_n_z"], **TOL)
    o2, s2, z2 = mo.linattn_reference_form(T64(g["la_q"]), T64(g["la_k"]), T64(g["la_v"]), T64(g["la_c_S"][:, 0]),
                                           T64(z0[:, 0]), T64(g["la_done"]))
    np.testing.assert_allclose(o2.numpy(), o.numpy(), rtol=1e-8, atol=1e-8)
    np.testing.assert_allclose(s2.numpy(), s_last.numpy(), rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(z2.numpy(), z_last.numpy(), rtol=1e-9, atol=1e-9)


def test_golden_rtrl_multiplicative_reset(golden):
    g = golden
    bsz, steps, hid, psz = g["rt_jac"].shape
    a = np.repeat(g["rt_decay"], psz, axis=-1)
    h, _ = mo.linrec_seq(T64(a), T64(g["rt_jac"].reshape(bsz, steps, -1)), T64(g["rt_sens"].reshape(bsz, -1)),
                         T64(g["rt_done"]))
    np.testing.assert_allclose(h[:, -1].numpy().reshape(bsz, 1, hid, psz), g["rt_next"], **TOL)


def test_golden_lru_rtrl_segment(golden):
    """lru_rtrl_seq against the vectors produced by the reference's own Memoroid.local_jacobian with its
    LRUCell (phantom injection, scan, read-out, local Jacobians, sensitivity propagation)."""
    g = golden
    C = lambda a: torch.from_numpy(np.asarray(a))
    names = ["nu_log", "theta_log", "gamma_log", "B_real", "B_imag"]
    for tag in ("s", "s0"):
        sens = {n: (C(g["lj_s_" + n]) if tag == "s" else torch.zeros_like(C(g["lj_s_" + n]))) for n in names}
        h_last, y, nxt = mo.lru_rtrl_seq(C(g["lj_x"]), C(g["lj_done"]), C(g["lj_c_state"])[:, 0], C(g["lj_nu_log"]),
                                         C(g["lj_theta_log"]), C(g["lj_gamma_log"]), C(g["lj_B"]), C(g["lj_C"]),
                                         C(g["lj_D"]), sens)
        np.testing.assert_allclose(h_last.numpy(), g["lj_n_state"][:, 0], **TOL)
        np.testing.assert_allclose(y.numpy(), g["lj_y"], **TOL)
        for n in names:
            np.testing.assert_allclose(nxt[n].numpy(), g[("lj_ns_" if tag == "s" else "lj_ns0_") + n], **TOL)


@pytest.mark.parametrize("disc", ["zoh", "bilinear"])
def test_golden_s5_discretisation_scan_and_read(golden, disc):
    """s5_discretize + linrec_seq + the read-out against the vectors produced by the reference's own S5Cell
    (s5.py:97-143 with hippo.py:34-50) under Memoroid."""
    g = golden
    C = lambda a: torch.from_numpy(np.asarray(a))
    lam = torch.complex(C(g["s5_p_lambda_real"]), C(g["s5_p_lambda_imag"]))
    b_tilde, c_tilde = torch.view_as_complex(C(g["s5_p_B"])), torch.view_as_complex(C(g["s5_p_C"]))
    lambda_bar, b_bar = mo.s5_discretize(lam, b_tilde, torch.exp(C(g["s5_p_log_step"])[:, 0]), disc)
    np.testing.assert_allclose(lambda_bar.numpy(), g[f"s5_{disc}_lambda_bar"], **TOL)
    x = C(g["s5_x"])
    z = x.to(torch.complex128) @ b_bar.t()
    np.testing.assert_allclose(z.numpy(), g[f"s5_{disc}_z_state"], **TOL)
    h, a_last = mo.linrec_seq(lambda_bar, z, C(g["s5_c_state"])[:, 0], C(g["s5_done"]), C(g["s5_c_decay"])[:, 0])
    np.testing.assert_allclose(h[:, -1].numpy(), g[f"s5_{disc}_n_state"][:, 0], **TOL)
    np.testing.assert_allclose(a_last.numpy(), g[f"s5_{disc}_n_decay"][:, 0], **TOL)
    y = (h @ c_tilde.t()).real + C(g["s5_p_d"]) * x
    np.testing.assert_allclose(y.numpy(), g[f"s5_{disc}_y"], **TOL)


@pytest.mark.parametrize("n", [4, 16])
def test_golden_hippo_eigenvalues(golden, n):
    """The oracle's and the host mirror's HiPPO-DPLR eigenvalues against the reference's make_dplr_hippo."""
    ref = np.sort_complex(golden[f"hippo_lambda_{n}"])
    np.testing.assert_allclose(np.sort_complex(mo.dplr_hippo_lambda(n)), ref, rtol=1e-9, atol=1e-9)
    from memorax_b200.memoroid import make_dplr_hippo
    lam, v = make_dplr_hippo(n)
    np.testing.assert_allclose(np.sort_complex(lam.numpy()), ref, rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose((v.conj().t() @ v).numpy(), np.eye(n), atol=1e-9)      # unitary eigenbasis


# ------------------------------------------------- layer 1 == layer 2, any bracketing
def _done(rng, bsz, steps, p=0.2):
    d = (rng.random((bsz, steps)) < p).astype(np.float64)
    d[0, 0] = 1
    if steps > 3:
        d[-1, 1:3] = 1
    return d


def test_golden_mamba_selective_scan(golden):
    """mamba_seq against the vectors produced by the reference's own MambaCell.__call__,
    binary_operator and read (mamba.py:109-135) under Memoroid.scan_fn."""
    g = golden
    y, h_last, a_last = mo.mamba_seq(T64(g["mb_hidden"]), T64(g["mb_B"]), T64(g["mb_C"]), T64(g["mb_dt"]),
                                     -torch.exp(T64(g["mb_A_log"])), T64(g["mb_D"]), T64(g["mb_c_state"][:, 0]),
                                     T64(g["mb_done"]), T64(g["mb_c_decay"][:, 0, :, 0, 0]))
    assert float((y - T64(g["mb_y_pre_gate"])).abs().max()) < 1e-11
    assert float((h_last - T64(g["mb_n_state"][:, 0])).abs().max()) < 1e-11
    assert float((a_last - T64(g["mb_n_decay"][:, 0, :, 0, 0])).abs().max()) < 1e-11
    # the per-step elements the scan consumes are what the reference's __call__ emits
    z = torch.einsum("bthn,bthd->bthnd", T64(g["mb_B"]) * T64(g["mb_dt"])[..., None], T64(g["mb_hidden"]))
    assert float((z - T64(g["mb_z_state"])).abs().max()) < 1e-12


@pytest.mark.parametrize("steps", [1, 2, 7, 16, 33])
@pytest.mark.parametrize("cplx", [False, True])
def test_linear_operator_scan_equals_recurrence(steps, cplx):
    rng = np.random.default_rng(steps)
    bsz, dim = 3, 5
    mk = (lambda *s: rng.normal(size=s) + 1j * rng.normal(size=s)) if cplx else (lambda *s: rng.normal(size=s))
    a, b = mk(bsz, steps, dim) * 0.7, mk(bsz, steps, dim)
    h0, a0 = mk(bsz, 1, dim), mk(bsz, 1, dim)
    done = _done(rng, bsz, steps)
    for br in ("tree", "left"):
        (h, acc), (hn, an) = mo.memoroid_scan(mo.op_linear, (b, a), (h0, a0), done, br)
        h_seq, a_last = mo.linrec_seq(T64(a), T64(b), T64(h0[:, 0]), T64(done), T64(a0[:, 0]))
        np.testing.assert_allclose(h, h_seq.numpy(), rtol=1e-10, atol=1e-10)
        np.testing.assert_allclose(an[:, 0], a_last.numpy(), rtol=1e-10, atol=1e-10)
        np.testing.assert_allclose(hn, h[:, -1:], rtol=0, atol=0)


@pytest.mark.parametrize("steps", [1, 5, 32])
def test_log_operator_scan_equals_recurrence(steps):
    rng = np.random.default_rng(steps + 100)
    bsz, dim = 2, 4
    ls, d = rng.normal(size=(bsz, steps, dim)), -np.abs(rng.normal(size=(bsz, steps, dim)))
    x0 = np.full((bsz, 1, dim), -np.inf)
    d0 = np.zeros((bsz, 1, dim))
    done = _done(rng, bsz, steps)
    (x, _), (_, dn) = mo.memoroid_scan(mo.op_log_linear, (ls, d), (x0, d0), done)
    x_seq, d_last = mo.mingru_seq(T64(ls), T64(d), T64(x0[:, 0]), T64(done))
    np.testing.assert_allclose(x, x_seq.numpy(), rtol=1e-10, atol=1e-10)
    np.testing.assert_allclose(dn[:, 0], d_last.numpy(), rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("steps", [1, 6, 19])
def test_additive_operator_scan_equals_linear_attention(steps):
    rng = np.random.default_rng(steps + 200)
    bsz, heads, dk, dv = 2, 2, 3, 4
    q, k = rng.normal(size=(bsz, steps, heads, dk)), rng.normal(size=(bsz, steps, heads, dk))
    v = rng.normal(size=(bsz, steps, heads, dv))
    s0, z0 = rng.normal(size=(bsz, 1, heads, dv, dk)), np.abs(rng.normal(size=(bsz, 1, heads, dk)))
    done = _done(rng, bsz, steps)
    fk = mo.elu_plus_one(k)
    elems = (np.einsum("bthi,bthj->bthij", v, fk), fk)
    (s_all, z_all), (sn, zn) = mo.memoroid_scan(mo.op_additive, elems, (s0, z0), done)
    fq = mo.elu_plus_one(q)
    o = np.einsum("bthij,bthj->bthi", s_all, fq) / np.maximum(np.einsum("bthi,bthi->bth", fq, z_all), 1e-6)[..., None]
    o_seq, s_last, z_last = mo.linattn_seq(T64(q), T64(k), T64(v), T64(s0[:, 0]), T64(z0[:, 0]), T64(done))
    np.testing.assert_allclose(o, o_seq.numpy(), rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(sn[:, 0], s_last.numpy(), rtol=1e-10, atol=1e-10)
    np.testing.assert_allclose(zn[:, 0], z_last.numpy(), rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("steps", [1, 6, 19])
def test_gated_delta_monoid_equals_recurrence(steps):
    rng = np.random.default_rng(steps + 300)
    bsz, heads, dk, dv = 2, 2, 4, 3
    q = rng.normal(size=(bsz, steps, heads, dk))
    k = rng.normal(size=(bsz, steps, heads, dk))
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.normal(size=(bsz, steps, heads, dv))
    alpha = rng.uniform(0.5, 1.0, size=(bsz, steps, heads))
    beta = rng.uniform(0.1, 0.9, size=(bsz, steps, heads))
    s0 = rng.normal(size=(bsz, 1, heads, dv, dk))
    done = _done(rng, bsz, steps)
    eye = np.broadcast_to(np.eye(dk), (bsz, steps, heads, dk, dk))
    m = alpha[..., None, None] * (eye - beta[..., None, None] * k[..., :, None] * k[..., None, :])
    u = beta[..., None, None] * v[..., :, None] * k[..., None, :]
    carry = (np.broadcast_to(np.eye(dk), (bsz, 1, heads, dk, dk)).copy(), s0)
    # With the carry's map set to the identity the U leaf of the prefix is the state.
    (_, s_all), _ = mo.memoroid_scan(mo.op_gated_delta, (m, u), carry, done)
    # A reset replaces the whole element by (M_t, U_t), i.e. S_t = U_t: the
    # previous state is dropped, exactly the recurrence with S' = 0.
    o = np.einsum("bthvk,bthk->bthv", s_all, q)
    o_seq, s_last = mo.gdelta_seq(T64(q), T64(k), T64(v), T64(alpha), T64(beta), T64(s0[:, 0]), T64(done))
    np.testing.assert_allclose(o, o_seq.numpy(), rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(s_all[:, -1], s_last.numpy(), rtol=1e-9, atol=1e-9)


# ------------------------------------------------------------ structural properties
def test_carry_split_invariance_and_reset_equivalence():
    rng = np.random.default_rng(7)
    bsz, steps, dim = 2, 12, 3
    a = T64(rng.uniform(0.1, 0.9, size=(bsz, steps, dim)))
    b = T64(rng.normal(size=(bsz, steps, dim)))
    h0 = T64(rng.normal(size=(bsz, dim)))
    done = torch.zeros(bsz, steps, dtype=torch.float64)
    done[:, 5] = 1
    h, acc = mo.linrec_seq(a, b, h0, done)
    h1, acc1 = mo.linrec_seq(a[:, :4], b[:, :4], h0, done[:, :4])
    h2, acc2 = mo.linrec_seq(a[:, 4:], b[:, 4:], h1[:, -1], done[:, 4:], acc1)
    np.testing.assert_allclose(torch.cat([h1, h2], 1).numpy(), h.numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(acc2.numpy(), acc.numpy(), rtol=1e-12)
    # a reset at t=5 == an independent sequence starting at t=5 from a zero state
    h_tail, _ = mo.linrec_seq(a[:, 5:], b[:, 5:], torch.zeros_like(h0), torch.zeros(bsz, steps - 5, dtype=torch.float64))
    np.testing.assert_allclose(h[:, 5:].numpy(), h_tail.numpy(), rtol=1e-12, atol=1e-12)


def _mlstm_inputs(g):
    hd = g["ml_q"].shape[-1]
    log_f = -np.logaddexp(-g["ml_f_pre"], 0.0)          # -softplus(-f), mlstm.py:185
    return dict(q=T64(g["ml_q"]), k=T64(g["ml_k"] / np.sqrt(hd)), v=T64(g["ml_v"]), log_i=T64(g["ml_i_pre"]),
                log_f=T64(log_f), done=T64(g["ml_done"]))


def test_golden_mlstm(golden):
    """The reference's own mlstm.py vectors: elements, every prefix state, the next carry and the read-out,
    with a non-trivial carry and with initialize_carry's (m = -1e9)."""
    g = golden
    x = _mlstm_inputs(g)
    # elements as the cell builds them (mlstm.py:188-203)
    np.testing.assert_allclose(np.einsum("bthi,bthj->bthij", x["k"].numpy(), x["v"].numpy()), g["ml_z_C"], **TOL)
    np.testing.assert_allclose(x["log_f"].numpy()[..., None, None], g["ml_z_logf"], **TOL)
    np.testing.assert_allclose(x["log_i"].numpy()[..., None, None], g["ml_z_m"], **TOL)
    carry = (T64(g["ml_c_C"][:, 0]), T64(g["ml_c_n"][:, 0, :, :, 0]), T64(g["ml_c_m"][:, 0, :, 0, 0]))
    h, (c_t, f_t, n_t, m_t) = mo.mlstm_seq(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], *carry, x["done"],
                                           T64(g["ml_c_logf"][:, 0, :, 0, 0]))
    np.testing.assert_allclose(h.numpy(), g["ml_h_tilde"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(c_t.numpy(), g["ml_n_C"][:, 0], **TOL)
    np.testing.assert_allclose(n_t.numpy(), g["ml_n_n"][:, 0, :, :, 0], **TOL)
    np.testing.assert_allclose(m_t.numpy(), g["ml_n_m"][:, 0, :, 0, 0], **TOL)
    np.testing.assert_allclose(f_t.numpy(), g["ml_n_logf"][:, 0, :, 0, 0], **TOL)
    # default carry
    bsz, _, heads, hd = g["ml_q"].shape
    zeros = lambda *s: torch.zeros(*s, dtype=torch.float64)
    assert np.all(g["ml_default_c_m"] == -1e9)             # initialize_carry, mlstm.py:238
    h0, (c_t, _, n_t, m_t) = mo.mlstm_seq(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], zeros(bsz, heads, hd, hd),
                                          zeros(bsz, heads, hd), T64(g["ml_default_c_m"][:, 0, :, 0, 0]), x["done"])
    np.testing.assert_allclose(h0.numpy(), g["ml_default_h_tilde"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(c_t.numpy(), g["ml_default_n_C"][:, 0], **TOL)
    np.testing.assert_allclose(m_t.numpy(), g["ml_default_n_m"][:, 0, :, 0, 0], **TOL)


def test_mlstm_operator_scan_equals_sequential_form(golden):
    """Layer 1 (prefix scan under the reset wrapper with mlstm.py's operator, any bracketing) against the
    reference's per-step states and against layer 2."""
    g = golden
    z = (g["ml_z_C"], g["ml_z_logf"], g["ml_z_n"], g["ml_z_m"])
    carry = (g["ml_c_C"], g["ml_c_logf"], g["ml_c_n"], g["ml_c_m"])
    for bracketing in ("tree", "left"):
        h, nxt = mo.memoroid_scan(mo.op_mlstm, z, carry, g["ml_done"], bracketing)
        for got, name in zip(h, ("ml_h_C", "ml_h_logf", "ml_h_n", "ml_h_m")):
            np.testing.assert_allclose(got, g[name], rtol=1e-9, atol=1e-9)
        np.testing.assert_allclose(nxt[0], g["ml_n_C"], rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("steps,p_done", [(200, 0.02), (64, 0.0), (130, 0.3), (5, 0.0)])
def test_mlstm_chunked_form_equals_the_sequential_oracle_and_its_autograd(steps, p_done):
    """The chunked algebra of the tensor-core kernels (decay factors with the stabiliser as a gauge, explicit path
    through the running maximum) against mlstm_seq and torch autograd, in float64: values and all eight gradients,
    with a carried state, cotangents on the next carry and resets (also at a chunk boundary)."""
    gen = torch.Generator().manual_seed(steps)
    d = 8
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float64)
    q, k, v, dh = rn(steps, d), rn(steps, d) / d ** 0.5, rn(steps, d), rn(steps, d)
    li = rn(steps) * 1.5 + 2.0
    lf = -torch.nn.functional.softplus(-(rn(steps) * 2 + 1))
    done = (torch.rand(steps, generator=gen) < p_done).double()
    if steps > 70:
        done[64] = 1.0
        done[70] = 1.0
    c0, n0, m0 = rn(d, d) * 0.5, rn(d) * 0.5, torch.tensor(0.3, dtype=torch.float64)
    dcl, dnl, dml = rn(d, d) * 0.3, rn(d) * 0.3, torch.tensor(0.7, dtype=torch.float64)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, li, lf, c0, n0, m0)]
    Q, K, V, LI, LF, C0, N0, M0 = leaves
    h_ref, (c_t, _, n_t, m_t) = mo.mlstm_seq(Q[None, :, None], K[None, :, None], V[None, :, None], LI[None, :, None],
                                             LF[None, :, None], C0[None, None], N0[None, None], M0[None, None], done[None])
    ((h_ref[0, :, 0] * dh).sum() + (c_t[0, 0] * dcl).sum() + (n_t[0, 0] * dnl).sum() + m_t[0, 0] * dml).backward()
    h, (c_out, n_out, m_out), g = mo.mlstm_chunked_single(q, k, v, li, lf, done, c0, n0, m0, dh, dcl, dnl, dml)
    close = lambda a, b: float((a - b.detach()).abs().max()) <= 1e-9 * max(1.0, float(b.detach().abs().max()))
    assert close(h, h_ref[0, :, 0]) and close(c_out, c_t[0, 0]) and close(n_out, n_t[0, 0]) and close(m_out, m_t[0, 0])
    for name, leaf in zip(["q", "k", "v", "li", "lf", "c0", "n0", "m0"], leaves):
        assert close(g[name], leaf.grad), name
