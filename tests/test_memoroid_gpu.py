"""The host-side mirror of the reference interface: Memoroid(cell)(inputs, done,
initial_carry) -> (next_carry, y) with the reference's carry pytrees, carry
threading across calls (memoroid.py:89) and gradients through the CUDA ops."""
import numpy as np
import pytest
import torch

from oracle import memoroid_oracle as mo

pytestmark = pytest.mark.gpu


def _done(bsz, steps, p=0.05, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(bsz, steps, generator=g) < p).cuda()


def test_lru_module_matches_oracle_and_threads_carry():
    from memorax_b200.memoroid import LRUCell, Memoroid
    torch.manual_seed(0)
    cell = LRUCell(features=8, hidden_dim=32, r_min=0.5, r_max=0.99, max_phase=0.6).cuda()
    model = Memoroid(cell)
    x, done = torch.randn(3, 20, 8, device="cuda"), _done(3, 20)
    (h_last, a_last), y = model(x, done)
    assert h_last.shape == (3, 1, 32) and a_last.shape == (3, 1, 32) and h_last.dtype == torch.complex64
    assert y.shape == (3, 20, 8)
    # oracle on the same elements
    state, lam = cell(x)
    h_ref, a_ref = mo.linrec_seq(lam.detach().cpu().to(torch.complex128), state.detach().cpu().to(torch.complex128),
                                 torch.zeros(3, 32, dtype=torch.complex128), done.cpu().double())
    assert float((h_last[:, 0].detach().cpu() - h_ref[:, -1]).abs().max()) <= 1e-5 * float(h_ref.abs().max())
    assert float((a_last[:, 0].cpu() - a_ref).abs().max()) <= 1e-5
    # one call == two calls threading the carry
    c1, y1 = model(x[:, :9], done[:, :9])
    c2, y2 = model(x[:, 9:], done[:, 9:], c1)
    assert torch.allclose(torch.cat([y1, y2], 1), y, atol=1e-5)
    assert torch.allclose(c2[0], h_last, atol=1e-5)
    # gradients reach every parameter
    y.square().mean().backward()
    for name, prm in cell.named_parameters():
        assert prm.grad is not None and torch.isfinite(prm.grad).all(), name


def test_mingru_module_default_carry_is_neg_inf_and_finite():
    from memorax_b200.memoroid import MinGRUCell, Memoroid
    torch.manual_seed(1)
    model = Memoroid(MinGRUCell(features=64, in_features=16)).cuda()
    carry = model.initialize_carry(None, (4, 16))
    assert torch.isneginf(carry[0]).all() and carry[0].shape == (4, 1, 64)
    x, done = torch.randn(4, 33, 16, device="cuda"), _done(4, 33)
    (x_last, d_last), y = model(x, done)
    assert torch.isfinite(y).all() and y.shape == (4, 33, 64) and x_last.shape == (4, 1, 64)
    y.sum().backward()
    assert all(torch.isfinite(p.grad).all() for p in model.parameters())


def test_linear_attention_and_deltanet_modules_run_and_thread_carry():
    from memorax_b200.memoroid import DeltaNetCell, LinearAttentionCell, Memoroid
    torch.manual_seed(2)
    for cell in (LinearAttentionCell(features=32, head_dim=64, num_heads=2),
                 LinearAttentionCell(features=32, head_dim=16, num_heads=4),
                 DeltaNetCell(features=32, head_dim=128, num_heads=2)):
        model = Memoroid(cell).cuda()
        x, done = torch.randn(2, 128, 32, device="cuda"), _done(2, 128, 0.02)
        carry, y = model(x, done)
        assert y.shape == (2, 128, 32) and all(c.shape[1] == 1 for c in carry)
        c1, y1 = model(x[:, :64], done[:, :64])
        c2, y2 = model(x[:, 64:], done[:, 64:], c1)
        assert torch.allclose(torch.cat([y1, y2], 1), y, atol=2e-2)
        y.square().mean().backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize("disc", ["zoh", "bilinear"])
def test_s5_module_matches_oracle(disc):
    from memorax_b200.memoroid import Memoroid, S5Cell
    torch.manual_seed(3)
    cell = S5Cell(features=6, state_size=16, discretization=disc).cuda()
    model = Memoroid(cell)
    x, done = torch.randn(2, 40, 6, device="cuda"), _done(2, 40, 0.05, seed=4)
    (h_last, a_last), y = model(x, done)
    state, lam = cell(x)
    h_ref, a_ref = mo.linrec_seq(lam.detach().cpu().to(torch.complex128), state.detach().cpu().to(torch.complex128),
                                 torch.zeros(2, 16, dtype=torch.complex128), done.cpu().double())
    scale = float(h_ref.abs().max())
    assert float((h_last[:, 0].detach().cpu() - h_ref[:, -1]).abs().max()) <= 1e-5 * scale
    c = torch.view_as_complex(cell.C.detach().cpu().contiguous()).to(torch.complex128)
    y_ref = (h_ref @ c.t()).real + cell.d.detach().cpu().double() * x.cpu().double()
    assert float((y.detach().cpu().double() - y_ref).abs().max()) <= 1e-4 * max(1.0, float(y_ref.abs().max()))
    y.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in cell.parameters())


@pytest.mark.parametrize("disc", ["zoh", "bilinear"])
def test_s5_matches_the_reference_vectors(disc):
    """S5Cell under Memoroid (discretisation, elements, scan with a non-trivial carry, read-out) against the
    vectors produced by the reference's own s5.py / hippo.py."""
    import os
    from memorax_b200.memoroid import Memoroid, S5Cell
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "memoroid_golden.npz"))
    nstate, feat = g["s5_p_B"].shape[:2]
    cell = S5Cell(feat, nstate, discretization=disc).cuda()
    f32 = lambda a: torch.from_numpy(np.asarray(a)).float().cuda()
    with torch.no_grad():
        cell.lambda_real.copy_(f32(g["s5_p_lambda_real"])); cell.lambda_imag.copy_(f32(g["s5_p_lambda_imag"]))
        cell.B.copy_(f32(g["s5_p_B"])); cell.C.copy_(f32(g["s5_p_C"])); cell.d.copy_(f32(g["s5_p_d"]))
        cell.log_step.copy_(f32(g["s5_p_log_step"]))
    c64 = lambda a: torch.from_numpy(np.asarray(a)).to(torch.complex64).cuda()
    (n_state, n_decay), y = Memoroid(cell)(f32(g["s5_x"]), torch.from_numpy(g["s5_done"]).cuda() > 0,
                                           (c64(g["s5_c_state"]), c64(g["s5_c_decay"])))
    close = lambda got, ref, what: float((got.detach().cpu().to(torch.complex128) - torch.from_numpy(np.asarray(ref))).abs().max()) \
        <= 2e-5 * max(1.0, float(np.abs(ref).max())) or pytest.fail(what)
    close(n_state, g[f"s5_{disc}_n_state"], "next state")
    close(n_decay, g[f"s5_{disc}_n_decay"], "next decay")
    close(y, g[f"s5_{disc}_y"], "y")


def test_propagate_sensitivities_matches_the_reference_vectors():
    """Memoroid.propagate_sensitivities against the vectors produced by the reference's own
    ``_propagate_sensitivities`` source (tests/golden/make_golden.py)."""
    import os
    import numpy as np
    from memorax_b200.memoroid import Memoroid, LRUCell
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "memoroid_golden.npz"))
    model = Memoroid(LRUCell(4, 4))
    f32 = lambda a: torch.from_numpy(np.asarray(a)).float().cuda()
    nxt = model.propagate_sensitivities(f32(g["rt_decay"]), {"w": f32(g["rt_jac"])}, {"w": f32(g["rt_sens"])},
                                        torch.from_numpy(g["rt_done"]).cuda())
    ref = torch.from_numpy(g["rt_next"])
    assert nxt["w"].shape == ref.shape
    err = float((nxt["w"].double().cpu() - ref).abs().max())
    assert err <= 1e-5 * max(1.0, float(ref.abs().max())), err


def _lru_from_golden(g):
    from memorax_b200.memoroid import LRUCell
    feat, hid = g["lj_x"].shape[-1], g["lj_nu_log"].shape[0]
    cell = LRUCell(feat, hid).cuda()
    f32 = lambda a: torch.from_numpy(np.asarray(a)).float().cuda()
    with torch.no_grad():
        cell.nu_log.copy_(f32(g["lj_nu_log"])); cell.theta_log.copy_(f32(g["lj_theta_log"]))
        cell.gamma_log.copy_(f32(g["lj_gamma_log"]))
        cell.B_real.copy_(f32(g["lj_B"].real)); cell.B_imag.copy_(f32(g["lj_B"].imag))
        cell.C_real.copy_(f32(g["lj_C"].real)); cell.C_imag.copy_(f32(g["lj_C"].imag))
        cell.D.copy_(f32(g["lj_D"]))
    return cell


def test_local_jacobian_matches_the_reference_vectors():
    """Memoroid.local_jacobian with the LRU cell (phantom injection, scan, read-out, local Jacobians, propagated
    sensitivities) against the vectors produced by the reference's own memoroid.py / lru.py."""
    import os
    from memorax_b200.memoroid import Memoroid
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "memoroid_golden.npz"))
    model = Memoroid(_lru_from_golden(g))
    c64 = lambda a: torch.from_numpy(np.asarray(a)).to(torch.complex64).cuda()
    names = ["nu_log", "theta_log", "gamma_log", "B_real", "B_imag"]
    x = torch.from_numpy(g["lj_x"]).float().cuda()
    done = torch.from_numpy(g["lj_done"]).cuda() > 0
    carry = (c64(g["lj_c_state"]), c64(g["lj_c_decay"]))
    close = lambda got, ref, what: float((got.detach().cpu().to(torch.complex128) - torch.from_numpy(np.asarray(ref))).abs().max()) \
        <= 2e-5 * max(1.0, float(np.abs(ref).max())) or pytest.fail(what)
    for tag in ("ns", "ns0"):
        sens = {n: c64(g["lj_s_" + n]) if tag == "ns" else torch.zeros_like(c64(g["lj_s_" + n])) for n in names}
        (n_state, n_decay), y, nxt = model.local_jacobian(x, done, carry, sens)
        close(n_state, g["lj_n_state"], "next state")
        close(n_decay, g["lj_n_decay"], "next decay")
        close(y, g["lj_y"], "y")
        for n in names:
            assert nxt[n].shape == sens[n].shape
            close(nxt[n], g["lj_" + tag + "_" + n], n)
    zero = model.initialize_sensitivity(None, (x.shape[0], x.shape[-1]))
    assert sorted(zero) == sorted(names) and all(zero[n].shape == c64(g["lj_s_" + n]).shape for n in names)


def test_rtrl_sensitivities_are_the_state_derivatives():
    """From a parameter-independent start and zero sensitivity, two chained RTRL segments must give
    d state_T / d leaf for every leaf: compared with fp64 autograd through the sequential oracle (real and
    imaginary parts of the state differentiated separately; each hidden unit depends on its own rows only)."""
    from memorax_b200.memoroid import Memoroid, LRUCell
    torch.manual_seed(21)
    feat, hid, bsz, steps = 3, 4, 2, 12
    cell = LRUCell(feat, hid, r_min=0.5, r_max=0.95, max_phase=1.0).cuda()
    model = Memoroid(cell)
    x = torch.randn(bsz, steps, feat, device="cuda")
    done = torch.zeros(bsz, steps, dtype=torch.bool, device="cuda")
    done[1, 5] = True
    carry = cell.initialize_carry(None, (bsz, feat))
    carry = tuple(c.cuda() for c in carry)
    sens = model.initialize_sensitivity(None, (bsz, feat))
    with torch.no_grad():
        carry, _, sens = model.local_jacobian(x[:, :7], done[:, :7], carry, sens)
        carry, _, sens = model.local_jacobian(x[:, 7:], done[:, 7:], carry, sens)
    # oracle: h_T as a function of the leaves, fp64
    leaves = {n: getattr(cell, n).detach().double().cpu().requires_grad_() for n in
              ("nu_log", "theta_log", "gamma_log", "B_real", "B_imag")}
    lam = torch.exp(torch.complex(-torch.exp(leaves["nu_log"]), torch.exp(leaves["theta_log"])))
    b_norm = torch.complex(leaves["B_real"], leaves["B_imag"]) * torch.exp(leaves["gamma_log"])[:, None]
    bu = x.double().cpu().to(torch.complex128) @ b_norm.t()
    h_ref, _ = mo.linrec_seq(lam, bu, torch.zeros(bsz, hid, dtype=torch.complex128), done.double().cpu())
    h_t = h_ref[:, -1]
    for name, leaf in leaves.items():
        for b in range(bsz):
            for j in range(hid):
                d_re = torch.autograd.grad(h_t[b, j].real, leaf, retain_graph=True)[0][j]
                d_im = torch.autograd.grad(h_t[b, j].imag, leaf, retain_graph=True)[0][j]
                want = torch.complex(d_re, d_im)
                got = sens[name][b, 0, j].cpu().to(torch.complex128)
                assert float((got - want).abs().max()) <= 1e-4 * max(1.0, float(want.abs().max())), (name, b, j)


def test_rtrl_gradient_equals_backpropagation_through_time():
    """What the phantom term is for: the gradient of a loss on the second segment's outputs, taken with the
    carry detached and the first segment's sensitivities injected, equals the gradient of the same loss when
    both segments are differentiated through in one call."""
    from memorax_b200.memoroid import Memoroid, LRUCell
    torch.manual_seed(22)
    feat, hid, bsz, steps, cut = 4, 8, 3, 20, 9
    cell = LRUCell(feat, hid, r_min=0.5, r_max=0.95, max_phase=1.0).cuda()
    model = Memoroid(cell)
    x = torch.randn(bsz, steps, feat, device="cuda")
    done = torch.zeros(bsz, steps, dtype=torch.bool, device="cuda")
    done[2, 3] = True
    w = torch.randn(bsz, steps - cut, feat, device="cuda")
    carry0 = tuple(c.cuda() for c in cell.initialize_carry(None, (bsz, feat)))
    _, y_full = model(x, done, carry0)
    (y_full[:, cut:] * w).sum().backward()
    bptt = {n: p.grad.clone() for n, p in cell.named_parameters()}
    cell.zero_grad()
    with torch.no_grad():
        carry, _, sens = model.local_jacobian(x[:, :cut], done[:, :cut], carry0,
                                              model.initialize_sensitivity(None, (bsz, feat)))
    _, y2, _ = model.local_jacobian(x[:, cut:], done[:, cut:], carry, sens)
    (y2 * w).sum().backward()
    for n, p in cell.named_parameters():
        err = float((p.grad - bptt[n]).abs().max())
        assert err <= 2e-4 * max(1.0, float(bptt[n].abs().max())), (n, err)


def test_propagate_sensitivities_grouped_decay_path():
    """A parameter leaf of 128 entries per hidden unit takes the grouped-decay kernel (the decay is not
    expanded); same recurrence as the oracle's real linear recurrence with the decay repeated."""
    from memorax_b200.memoroid import Memoroid, LRUCell
    gen = torch.Generator().manual_seed(7)
    bsz, steps, hid, psize = 3, 21, 4, 128
    decay = torch.rand(bsz, steps, hid, generator=gen, dtype=torch.float64)
    jac = torch.randn(bsz, steps, hid, 2, 64, generator=gen, dtype=torch.float64)
    sens = torch.randn(bsz, 1, hid, 2, 64, generator=gen, dtype=torch.float64)
    done = torch.rand(bsz, steps, generator=gen) < 0.1
    model = Memoroid(LRUCell(4, hid))
    nxt = model.propagate_sensitivities(decay.float().cuda(), {"w": jac.float().cuda()}, {"w": sens.float().cuda()},
                                        done.cuda())
    h_ref, _ = mo.linrec_seq(decay.repeat_interleave(psize, dim=-1), jac.reshape(bsz, steps, hid * psize),
                             sens.reshape(bsz, hid * psize), done.double())
    ref = h_ref[:, -1:].reshape(bsz, 1, hid, 2, 64)
    assert nxt["w"].shape == ref.shape
    err = float((nxt["w"].double().cpu() - ref).abs().max())
    assert err <= 1e-5 * max(1.0, float(ref.abs().max())), err


@pytest.mark.parametrize("kind", ["lru", "s5"])
def test_real_gemm_projections_equal_the_complex_formulation(kind):
    """The cells' projections run as real GEMMs over interleaved (re, im) weights; against the reference's
    complex matmuls (lru.py:82-84,99-102; s5.py:126-128,139-143) on the same weights, values and gradients."""
    from memorax_b200.memoroid import LRUCell, S5Cell
    torch.manual_seed(11)
    cell = (LRUCell(24, 64) if kind == "lru" else S5Cell(24, 64)).cuda()
    x = torch.randn(3, 17, 24, device="cuda", requires_grad=True)
    h = torch.randn(3, 17, 64, dtype=torch.complex64, device="cuda", requires_grad=True)
    _, w_in, w_out, skip = cell._weights()
    bu, _ = cell(x)
    y = cell.read((h, None), x)
    bu_ref = torch.matmul(x.to(torch.complex64), w_in.t())
    y_ref = torch.matmul(h, w_out.t()).real + skip * x
    tol = lambda ref: 1e-5 * max(1.0, float(ref.abs().max()))
    assert float((bu - bu_ref).abs().max()) <= tol(bu_ref) and float((y - y_ref).abs().max()) <= tol(y_ref)
    ct_bu, ct_y = torch.randn_like(bu), torch.randn_like(y)
    params = [p for p in cell.parameters()]
    loss = lambda a, b: (torch.view_as_real(a) * torch.view_as_real(ct_bu)).sum() + (b * ct_y).sum()
    got = torch.autograd.grad(loss(bu, y), [x, h] + params, allow_unused=True)
    want = torch.autograd.grad(loss(bu_ref, y_ref), [x, h] + params, allow_unused=True)
    for g, w in zip(got, want):
        assert (g is None) == (w is None)
        if g is not None:
            assert float((g - w).abs().max()) <= 1e-4 * max(1.0, float(w.abs().max()))


def test_mamba_scan_and_read_match_the_reference_vectors():
    """MambaCell.scan_elements / read_state against the vectors produced by the reference's own
    MambaCell source under Memoroid.scan_fn (non-trivial carry, resets)."""
    import os
    import numpy as np
    from memorax_b200.memoroid import MambaCell
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "memoroid_golden.npz"))
    bsz, steps, heads, sdim, hdim = g["mb_z_state"].shape
    cell = MambaCell(8, num_heads=heads, head_dim=hdim, state_dim=sdim).cuda()
    f32 = lambda a: torch.from_numpy(np.asarray(a)).float().cuda()
    with torch.no_grad():
        cell.D.copy_(f32(g["mb_D"]))
    carry = (f32(g["mb_c_state"]), f32(g["mb_c_decay"]))
    h, nxt = cell.scan_elements(f32(g["mb_z_state"]), f32(g["mb_z_decay"]), carry, torch.from_numpy(g["mb_done"]).cuda())
    close = lambda got, ref, what: float((got.double().cpu() - torch.from_numpy(ref)).abs().max()) <= \
        1e-5 * max(1.0, float(np.abs(ref).max())) or pytest.fail(what)
    close(h, g["mb_h_state"], "h")
    close(nxt[0], g["mb_n_state"], "next state")
    close(nxt[1], g["mb_n_decay"], "next decay")
    y = cell.read_state(h, f32(g["mb_hidden"]), f32(g["mb_C"]))
    close(y, g["mb_y_pre_gate"], "read-out")


def test_mamba_model_gradients_match_the_oracle():
    """Memoroid(MambaCell) end to end on the GPU against the fp64 oracle recurrence driven by the same
    projections: outputs, next carry and the gradients of every parameter."""
    from memorax_b200.memoroid import MambaCell, Memoroid
    torch.manual_seed(5)
    bsz, steps, feat = 3, 70, 24
    model = Memoroid(MambaCell(feat, num_heads=2, head_dim=8, state_dim=4)).cuda()
    cell = model.cell
    x = torch.randn(bsz, steps, feat, device="cuda")
    done = (torch.rand(bsz, steps, device="cuda") < 0.05)
    done[0, 0] = True
    carry = (torch.randn(bsz, 1, 2, 4, 8, device="cuda") * 0.3, torch.rand(bsz, 1, 2, 1, 1, device="cuda") * 0.5 + 0.5)
    w = torch.randn(bsz, steps, feat, device="cuda")
    nxt, y = model(x, done, carry)
    ((y * w).sum() + (nxt[0] ** 2).sum()).backward()
    got = {n: p.grad.detach().double().cpu() for n, p in model.named_parameters()}
    model.zero_grad()
    # oracle: same projections (torch, on the device), fp64 sequential recurrence on the host
    hidden, b_proj, c_proj, gate, dt = cell._project(x)
    y_o, h_last, a_last = mo.mamba_seq(hidden.double().cpu(), b_proj.double().cpu(), c_proj.double().cpu(),
                                       dt.double().cpu(), -torch.exp(cell.A_log.double().cpu()), cell.D.double().cpu(),
                                       carry[0][:, 0].double().cpu(), done.double().cpu(),
                                       carry[1][:, 0, :, 0, 0].double().cpu())
    y_o = y_o.reshape(bsz, steps, -1).to("cuda", torch.float32)
    y_ref = cell.output_projection(cell.norm(y_o) * torch.nn.functional.silu(gate))
    ((y_ref * w).sum() + (h_last.to("cuda", torch.float32) ** 2).sum()).backward()
    assert float((y - y_ref).abs().max()) <= 1e-4 * max(1.0, float(y_ref.abs().max()))
    assert float((nxt[0][:, 0].double().cpu() - h_last).abs().max()) <= 1e-5 * max(1.0, float(h_last.abs().max()))
    assert float((nxt[1][:, 0, :, 0, 0].double().cpu() - a_last).abs().max()) <= 1e-5
    for name, p in model.named_parameters():
        ref = p.grad.detach().double().cpu()
        err = float((got[name] - ref).abs().max())
        assert err <= 2e-4 * max(1.0, float(ref.abs().max())), (name, err)


def test_scan_fn_mirror_replays_the_reference_vectors(golden):
    """``Memoroid.scan_fn(z, initial_carry, done) -> (h, next_carry)`` (memoroid.py:60-91) on the elements
    the reference's own LRU and MinGRU cells produced: states at every step and the next carry, decay leaf
    included (returned for the last step only)."""
    import numpy as np
    from memorax_b200.memoroid import LRUCell, Memoroid, MinGRUCell, LinearAttentionCell
    g = golden
    c64 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.complex64).cuda()
    f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).float().cuda()
    done = torch.from_numpy(g["lru_done"]).cuda()
    model = Memoroid(LRUCell(features=5, hidden_dim=4).cuda())
    z = (c64(g["lru_z_state"]), c64(g["lru_z_decay"][0, 0]))        # lru.py:86 broadcasts one lambda
    (h, decay_leaf), (n_state, n_decay) = model.scan_fn(z, (c64(g["lru_c_state"]), c64(g["lru_c_decay"])), done)
    assert decay_leaf is None
    ref = torch.from_numpy(g["lru_h_state"])
    assert float((h.cpu() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    assert n_state.shape == g["lru_n_state"].shape and n_decay.shape == g["lru_n_decay"].shape
    assert float((n_state.cpu() - torch.from_numpy(g["lru_n_state"])).abs().max()) <= 1e-5 * float(ref.abs().max())
    assert float((n_decay.cpu() - torch.from_numpy(g["lru_n_decay"])).abs().max()) <= 1e-5

    gru = Memoroid(MinGRUCell(features=6).cuda())
    (x, _), (nx, nd) = gru.scan_fn((f32(g["gru_z_state"]), f32(g["gru_z_decay"])),
                                   (f32(g["gru_c1_state"]), f32(g["gru_c1_decay"])), torch.from_numpy(g["gru_done"]).cuda())
    assert float((x.cpu() - torch.from_numpy(g["gru_h1_state"])).abs().max()) <= 1e-5 * float(np.abs(g["gru_h1_state"]).max())
    assert float((nx.cpu() - torch.from_numpy(g["gru_n1_state"])).abs().max()) <= 1e-5 * float(np.abs(g["gru_n1_state"]).max())
    assert float((nd.cpu() - torch.from_numpy(g["gru_n1_decay"])).abs().max()) <= 1e-5 * max(1.0, float(np.abs(g["gru_n1_decay"]).max()))

    with pytest.raises(NotImplementedError):
        Memoroid(LinearAttentionCell(features=64, head_dim=64, num_heads=1)).scan_fn(None, None, None)
