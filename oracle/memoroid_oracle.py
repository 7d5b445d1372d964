"""CPU restatement of the memorax sequence-mixing path (TEST INFRASTRUCTURE ONLY).

Two layers, both plain CPU code:

* ``prefix_scan`` / ``memoroid_scan``: the reference's formulation -- an
  inclusive prefix over ``[carry, z_1 .. z_T]`` under a reset-aware wrapper of a
  cell's binary operator (memorax/networks/sequence_models/memoroid.py:60-91),
  with the per-cell operators of lru.py:92-95, s5.py:133-136,
  min_gru.py:67-74, linear_attention.py:82-86, mlstm.py:205-229 and the
  multiplicative-reset linear form of memoroid.py:119-123.  NumPy, any bracketing.
* ``*_seq`` functions: the closed-form sequential recurrences those scans
  equal, written in torch so that fp64 autograd gives the gradient oracle.
  ``tests/test_oracle.py`` proves layer 2 == layer 1, and
  ``tests/golden`` pins both against the reference's own source.

Shapes follow the reference: batch-major, time second, features last;
``done[b, t] = 1`` means step t starts a new episode, i.e. the state before
step t is discarded (memoroid.py:67-85).
"""
from __future__ import annotations

import numpy as np
import torch

# --------------------------------------------------------------------------
# Layer 1: the reference formulation (generic prefix scan + wrapped operator)
# --------------------------------------------------------------------------


def _tmap(fn, *trees):
    """Map over tuples-of-arrays pytrees (the only pytrees on this path)."""
    if isinstance(trees[0], (tuple, list)):
        return tuple(_tmap(fn, *parts) for parts in zip(*trees))
    return fn(*trees)


def prefix_scan(op, elems, bracketing="tree"):
    """Inclusive prefix of ``elems`` along axis 1 under associative ``op``.

    ``bracketing='tree'`` combines in the odd/even recursive-doubling order of
    a work-efficient parallel scan (the order jax.lax.associative_scan, the
    call at memoroid.py:87, uses); ``'left'`` folds left to right.  Both must
    agree up to rounding for an associative operator.
    """
    n = _leaves(elems)[0].shape[1]
    if bracketing == "left":
        acc = _tmap(lambda x: x[:, :1], elems)
        outs = [acc]
        for t in range(1, n):
            acc = op(acc, _tmap(lambda x: x[:, t:t + 1], elems))
            outs.append(acc)
        return _tmap(lambda *xs: np.concatenate(xs, axis=1), *outs)
    if n < 2:
        return elems
    # Pairwise-reduce neighbours, scan the half-length sequence, then fill the
    # even positions from the odd prefixes.
    even = _tmap(lambda x: x[:, 0:n - 1:2], elems)
    odd = _tmap(lambda x: x[:, 1:n:2], elems)
    odd_prefix = prefix_scan(op, op(even, odd), "tree")
    if n % 2 == 0:
        rest = op(_tmap(lambda x: x[:, :-1], odd_prefix),
                  _tmap(lambda x: x[:, 2::2], elems))
    else:
        rest = op(odd_prefix, _tmap(lambda x: x[:, 2::2], elems))
    first = _tmap(lambda x: x[:, :1], elems)
    even_prefix = _tmap(lambda f, r: np.concatenate([f, r], axis=1), first, rest)

    def interleave(e, o):
        out = np.empty((e.shape[0], n) + e.shape[2:], dtype=e.dtype)
        out[:, 0::2] = e
        out[:, 1::2] = o
        return out

    return _tmap(interleave, even_prefix, odd_prefix)


def _leaves(tree):
    if isinstance(tree, (tuple, list)):
        out = []
        for part in tree:
            out.extend(_leaves(part))
        return out
    return [tree]


def _expand_like(flag, leaf):
    while flag.ndim < leaf.ndim:
        flag = flag[..., None]
    return flag


def memoroid_scan(cell_op, z, initial_carry, done, bracketing="tree"):
    """Restates ``Memoroid.scan_fn`` (memoroid.py:60-91).

    The carry is prepended at time 0 with reset flag 0, ``done`` supplies the
    flags of the T real steps, and two prefix elements combine as
    ``where(rhs_reset, rhs, cell_op(lhs, rhs))`` with the flags OR-ed.
    Returns ``(h, next_carry)``: all T prefixes and the last one (time axis
    kept, as memoroid.py:89-90 does).
    """
    elems = _tmap(lambda c, e: np.concatenate([c, e], axis=1), initial_carry, z)
    done = np.asarray(done, dtype=np.float64)
    flags = np.concatenate([np.zeros((done.shape[0], 1)), done], axis=1)

    def wrapped(lhs, rhs):
        lhs_c, lhs_f = lhs
        rhs_c, rhs_f = rhs
        merged = cell_op(lhs_c, rhs_c)
        out = _tmap(lambda r, m: np.where(_expand_like(rhs_f, r) > 0, r, m), rhs_c, merged)
        return out, np.maximum(lhs_f, rhs_f)

    h, _ = prefix_scan(wrapped, (elems, flags), bracketing)
    next_carry = _tmap(lambda x: x[:, -1:], h)
    h = _tmap(lambda x: x[:, 1:], h)
    return h, next_carry


def op_linear(lhs, rhs):
    """(state, decay) operator of LRU / S5 / the RTRL sensitivity scan
    (lru.py:92-95, s5.py:133-136, memoroid.py:119-123)."""
    s_i, a_i = lhs
    s_j, a_j = rhs
    return (a_j * s_i + s_j, a_j * a_i)


def op_log_linear(lhs, rhs):
    """MinGRU's log-space operator (min_gru.py:67-74)."""
    x_i, d_i = lhs
    x_j, d_j = rhs
    return (np.logaddexp(d_j + x_i, x_j), d_i + d_j)


def op_additive(lhs, rhs):
    """Linear attention's additive operator (linear_attention.py:82-86)."""
    return tuple(p + q for p, q in zip(lhs, rhs))


def op_gated_delta(lhs, rhs):
    """Gated delta rule as a monoid over (M, U): state maps compose on the
    right, ``S -> S M + U`` with S of shape (d_v, d_k).  Not in the reference."""
    m_i, u_i = lhs
    m_j, u_j = rhs
    return (m_i @ m_j, u_i @ m_j + u_j)


def op_mlstm(lhs, rhs):
    """mLSTM's operator over (C, log_f, n, m) with the running-max stabiliser (mlstm.py:205-229): the
    left element is decayed by the right one's forget gate, both are rescaled to the larger log
    magnitude, and the stabilised memories add."""
    c_a, f_a, n_a, m_a = lhs
    c_b, f_b, n_b, m_b = rhs
    m_dec = m_a + f_b
    m_new = np.maximum(m_dec, m_b)
    s_a, s_b = np.exp(m_dec - m_new), np.exp(m_b - m_new)
    return (s_a * c_a + s_b * c_b, f_a + f_b, s_a * n_a + s_b * n_b, m_new)


def elu_plus_one(x):
    """Feature map of linear_attention.py:58-60 (works on numpy and torch)."""
    if isinstance(x, torch.Tensor):
        return torch.where(x > 0, x + 1.0, torch.exp(torch.clamp(x, max=0.0)))
    return np.where(x > 0, x + 1.0, np.exp(np.minimum(x, 0.0)))


# --------------------------------------------------------------------------
# Layer 2: closed-form sequential recurrences (torch; fp64 autograd oracle)
# --------------------------------------------------------------------------


def _keep(done, t, like):
    """1 - done[:, t] broadcast against ``like`` (real dtype)."""
    m = 1.0 - done[:, t].to(like.real.dtype if like.is_complex() else like.dtype)
    while m.ndim < like.ndim:
        m = m[..., None]
    return m


def linrec_seq(a, b, h0, done, a0=None):
    """h_t = done_t ? b_t : a_t h_{t-1} + b_t ;  A_t = done_t ? a_t : a_t A_{t-1}.

    ``a`` is (B,T,D) or time-invariant (D,) (lru.py:86); real or complex.
    Returns ``h`` (B,T,D) and the decay leaf of the next carry ``A_T`` (B,D).
    Equals ``memoroid_scan(op_linear, ...)``.
    """
    bsz, steps, _ = b.shape
    if a.ndim == 1:
        a = a.expand(bsz, steps, -1)
    h = h0
    acc = torch.ones_like(h0) if a0 is None else a0
    out = []
    for t in range(steps):
        m = _keep(done, t, h)
        h = a[:, t] * (m * h) + b[:, t]
        acc = torch.where(m > 0, a[:, t] * acc, a[:, t] + 0 * acc)
        out.append(h)
    return torch.stack(out, dim=1), acc


def mingru_seq(log_state, decay, x0, done, a0=None):
    """x_t = done_t ? ls_t : logaddexp(d_t + x_{t-1}, ls_t); A_t likewise with
    sums (min_gru.py:67-74 under the reset wrapper).  ``x0`` may be -inf."""
    bsz, steps, _ = log_state.shape
    x = x0
    acc = torch.zeros_like(x0) if a0 is None else a0
    out = []
    for t in range(steps):
        m = _keep(done, t, x) > 0
        prev = torch.where(m, decay[:, t] + x, torch.full_like(x, -float("inf")))
        x = torch.logaddexp(prev, log_state[:, t])
        acc = torch.where(m, decay[:, t] + acc, decay[:, t])
        out.append(x)
    return torch.stack(out, dim=1), acc


def linattn_seq(q, k, v, s0, z0, done, eps=1e-6, feature_map=True):
    """Causal linear attention with carried (S, z) (linear_attention.py:62-112).

    q,k (B,T,H,dk), v (B,T,H,dv); S (B,H,dv,dk) = sum v (x) phi(k), z (B,H,dk).
    o_t = S_t phi(q_t) / max(phi(q_t).z_t, eps).  Returns (o, S_T, z_T).
    """
    if feature_map:
        q, k = elu_plus_one(q), elu_plus_one(k)
    s, z = s0, z0
    out = []
    for t in range(q.shape[1]):
        m = _keep(done, t, z)
        s = m[..., None] * s + v[:, t, :, :, None] * k[:, t, :, None, :]
        z = m * z + k[:, t]
        num = torch.einsum("bhvk,bhk->bhv", s, q[:, t])
        den = torch.clamp((q[:, t] * z).sum(-1, keepdim=True), min=eps)
        out.append(num / den)
    return torch.stack(out, dim=1), s, z


def gdelta_seq(q, k, v, alpha, beta, s0, done):
    """Gated delta rule: S_t = a_t S'_{t-1} (I - b_t k_t k_t^T) + b_t v_t k_t^T,
    o_t = S_t q_t, with S' = 0 where done_t.  S is (B,H,dv,dk); alpha, beta are
    (B,T,H).  Equals ``memoroid_scan(op_gated_delta, ...)`` on the elements
    ``(alpha (I - beta k k^T), beta v k^T)`` with carry ``(I, S_0)``."""
    s = s0
    out = []
    for t in range(q.shape[1]):
        m = _keep(done, t, alpha[:, t])
        s = (m * alpha[:, t])[..., None, None] * s
        sk = torch.einsum("bhvk,bhk->bhv", s, k[:, t])
        bt = beta[:, t][..., None]
        s = s + (bt * (v[:, t] - sk))[..., None] * k[:, t, :, None, :]
        out.append(torch.einsum("bhvk,bhk->bhv", s, q[:, t]))
    return torch.stack(out, dim=1), s


def mlstm_seq(q, k, v, log_i, log_f, c0, n0, m0, done, f0=None, eps=1e-6, with_den=False):
    """Stabilised mLSTM (mlstm.py:163-229 under the reset rule of ``Memoroid.scan_fn``), sequentially:
      m_t = max(m_{t-1} + log_f_t, log_i_t)
      C_t = exp(m_{t-1} + log_f_t - m_t) C_{t-1} + exp(log_i_t - m_t) k_t v_t^T      (n_t likewise with k_t)
      h_t = q_t^T C_t / (max(|q_t . n_t|, exp(-m_t)) + eps)
    and done_t discards (C, n, m) of the past (the element alone remains: m_t = log_i_t, C_t = k_t v_t^T).
    ``k`` is the key as the cell's element holds it (already divided by sqrt(head_dim), mlstm.py:196).

    q, k, v (B,T,H,d); log_i, log_f (B,T,H); c0 (B,H,d,d) indexed [key, value]; n0 (B,H,d); m0, f0 (B,H).
    Returns h (B,T,H,d) and the next carry (C_T, F_T, n_T, m_T) with F the summed log forget gates
    since the last reset (the carry's log_f leaf); with ``with_den`` also the (B,T,H) denominators."""
    c, n, m = c0, n0, m0
    dens = []
    f = torch.zeros_like(m0) if f0 is None else f0
    neg_inf = torch.full_like(m0, -float("inf"))
    out = []
    for t in range(q.shape[1]):
        keep = (1.0 - done[:, t]).reshape(-1, 1) > 0
        m_dec = torch.where(keep, m, neg_inf) + log_f[:, t]
        m_new = torch.maximum(m_dec, log_i[:, t])
        s_a, s_b = torch.exp(m_dec - m_new), torch.exp(log_i[:, t] - m_new)
        c = s_a[..., None, None] * c + s_b[..., None, None] * k[:, t, :, :, None] * v[:, t, :, None, :]
        n = s_a[..., None] * n + s_b[..., None] * k[:, t]
        f = torch.where(keep, f + log_f[:, t], log_f[:, t])
        m = m_new
        den = torch.maximum((q[:, t] * n).sum(-1).abs(), torch.exp(-m)) + eps
        out.append(torch.einsum("bhj,bhjk->bhk", q[:, t], c) / den[..., None])
        dens.append(den)
    if with_den:
        return torch.stack(out, dim=1), (c, f, n, m), torch.stack(dens, dim=1)
    return torch.stack(out, dim=1), (c, f, n, m)


def mamba_seq(hidden, b_proj, c_proj, dt, a_neg, d_skip, h0, done, a0=None):
    """Selective state-space scan of ``MambaCell`` (mamba.py:109-135) under the reset rule
    of ``Memoroid.scan_fn``: per head, with ``decay_t = exp(dt_t A)`` (A < 0, one scalar per
    head) and ``z_t = (dt_t B_t) (x) x_t`` (state_dim x head_dim),
    ``h_t = done_t ? z_t : decay_t h_{t-1} + z_t``, ``y_t = C_t . h_t + D x_t``.

    hidden (B,T,H,P), b_proj / c_proj (B,T,H,N), dt (B,T,H), a_neg / d_skip (H,),
    h0 (B,H,N,P), a0 the carry's decay leaf (B,H) or None for ones.
    Returns y (B,T,H,P), the last state (B,H,N,P) and the decay leaf of the next carry (B,H).
    """
    bsz, steps = dt.shape[:2]
    decay = torch.exp(dt * a_neg)                                                   # (B,T,H)
    z = torch.einsum("bthn,bthd->bthnd", b_proj * dt[..., None], hidden)            # mamba.py:114
    h = h0
    acc = torch.ones_like(decay[:, 0]) if a0 is None else a0
    ys = []
    for t in range(steps):
        m = (1.0 - done[:, t]).reshape(bsz, 1, 1, 1).to(h.dtype)
        a_t = decay[:, t][..., None, None]
        h = a_t * (m * h) + z[:, t]
        acc = torch.where(m[:, :, 0, 0] > 0, decay[:, t] * acc, decay[:, t] + 0 * acc)
        ys.append(torch.einsum("bhn,bhnd->bhd", c_proj[:, t], h) + d_skip[None, :, None] * hidden[:, t])
    return torch.stack(ys, dim=1), h, acc


def lru_rtrl_seq(x, done, c_state, nu_log, theta_log, gamma_log, b_mat, c_mat, d_skip, sens):
    """One RTRL segment of the LRU cell, sequentially in time (Memoroid.local_jacobian, memoroid.py:143-176,
    with LRUCell.__call__ / read / local_jacobian, lru.py:78-125, and _propagate_sensitivities,
    memoroid.py:114-141).  ``b_mat`` (H,F), ``c_mat`` (F,H) complex; ``sens`` a dict of (B,1,H,*param) leaves.
    Returns ``(h_last (B,H), y (B,T,F), next_sens)``.  The phantom term is zero in value and is left out."""
    lam = torch.exp(torch.complex(-torch.exp(nu_log), torch.exp(theta_log)))
    gam = torch.exp(gamma_log)
    bu = x.to(lam.dtype) @ (b_mat * gam[:, None]).t()                      # (B,T,H), lru.py:82-84
    h = c_state
    s = {k: v[:, 0].clone() for k, v in sens.items()}
    ys = []
    for t in range(x.shape[1]):
        reset = done[:, t] > 0
        prev = torch.where(reset[:, None], torch.zeros_like(h), h)         # memoroid.py:158-168
        jac = {"nu_log": -torch.exp(nu_log) * lam * prev, "theta_log": 1j * torch.exp(theta_log) * lam * prev,
               "gamma_log": bu[:, t],
               "B_real": (gam[None, :, None] * x[:, t, None, :]).to(lam.dtype),
               "B_imag": 1j * (gam[None, :, None] * x[:, t, None, :])}
        h = torch.where(reset[:, None], bu[:, t], lam * h + bu[:, t])      # memoroid.py:72-85 with lru.py:92-95
        for name in s:
            decay = lam.reshape((1, -1) + (1,) * (s[name].dim() - 2))
            keep = (~reset).reshape((-1,) + (1,) * (s[name].dim() - 1))
            s[name] = torch.where(keep, decay * s[name], torch.zeros_like(s[name])) + jac[name]
        ys.append((h @ c_mat.t()).real + d_skip * x[:, t])
    return h, torch.stack(ys, dim=1), {k: v[:, None] for k, v in s.items()}


def s5_discretize(lam, b_tilde, step, kind):
    """(lambda_bar, b_bar) of the diagonal state-space cell (hippo.py:34-50): zero-order hold
    exp(lambda dt), (lambda_bar - 1) / lambda * B; or bilinear (1 + dt/2 lambda) / (1 - dt/2 lambda), dt / (1 - dt/2 lambda) * B."""
    step = step.to(lam.dtype)
    if kind == "zoh":
        lambda_bar = torch.exp(lam * step)
        return lambda_bar, ((lambda_bar - 1.0) / lam)[:, None] * b_tilde
    bl = 1.0 / (1.0 - step / 2.0 * lam)
    return bl * (1.0 + step / 2.0 * lam), (bl * step)[:, None] * b_tilde


def dplr_hippo_lambda(n):
    """Eigenvalues the S5 cell starts from (hippo.py:6-32): real part mean(diag(A + p p^T)), imaginary parts the
    eigenvalues of the Hermitian -i (A + p p^T), A the HiPPO-LegS matrix."""
    idx = np.arange(n, dtype=np.float64)
    q = np.sqrt(1.0 + 2.0 * idx)
    a = -(np.tril(q[:, None] * q[None, :]) - np.diag(idx))
    p = np.sqrt(idx + 0.5)
    s_mat = a + p[:, None] * p[None, :]
    return np.mean(np.diag(s_mat)) + 1j * np.linalg.eigvalsh(s_mat * (-1j))


def jax_cotangent(grad):
    """torch.autograd's gradient of a real loss w.r.t. a complex tensor is the
    conjugate of what JAX's reverse mode (and hence the reference) returns."""
    return grad.conj() if grad.is_complex() else grad


# --------------------------------------------------------------------------
# The chunked form of the mLSTM that the tensor-core kernels evaluate (mlstm_tc.cu, mlstm_tc_bwd.cu), restated
# for one (batch, head) in float64: forward and the hand-derived backward.  tests/test_oracle.py holds it
# against mlstm_seq and its autograd, which pins the kernels' algebra independently of any GPU.
# --------------------------------------------------------------------------
def mlstm_chunked_single(q, k, v, li, lf, done, c0, n0, m0, dh, dc_last, dn_last, dm_last, eps=1e-6, chunk=64):
    """q, k, v, dh (T,d); li, lf, done (T,); c0 (d,d) [key][value], n0 (d,), m0 scalar; cotangents of the next
    carry.  Returns ``(h, (c_T, n_T, m_T), grads)`` with ``grads`` keyed q, k, v, li, lf, c0, n0, m0.
    The stabiliser m is held fixed in every decay factor (it is a gauge of the recurrence) and its one real
    effect -- eps exp(m_t) in the denominator and the scale of the stabilised next carry -- is propagated
    through m_t = max(m_{t-1} + lf_t, li_t) separately."""
    dt = q.dtype
    T, d = q.shape
    nch = (T + chunk - 1) // chunk
    Sx = torch.cat([c0, n0[:, None]], dim=1)
    m_in = m0.clone()
    hs, saved = [], []
    m_all = torch.zeros(T, dtype=dt)
    for c in range(nch):
        t0, t1 = c * chunk, min(T, (c + 1) * chunk)
        L = t1 - t0
        qc, kc, vc, lic, lfc, dn = q[t0:t1], k[t0:t1], v[t0:t1], li[t0:t1], lf[t0:t1], done[t0:t1]
        cumf = torch.cumsum(lfc, 0)
        first = torch.zeros(L, dtype=torch.long)
        last_reset = -1
        for t in range(L):
            if dn[t] > 0:
                last_reset = t
            first[t] = max(last_reset, 0)
        live = torch.tensor([not bool((dn[: t + 1] > 0).any()) for t in range(L)])
        keep = torch.arange(L) >= max(last_reset, 0)
        has_reset = last_reset >= 0
        m = torch.zeros(L, dtype=dt)
        mp = m_in
        for t in range(L):
            m[t] = lic[t] if dn[t] > 0 else torch.maximum(mp + lfc[t], lic[t])
            mp = m[t]
        m_all[t0:t1] = m
        idx = torch.arange(L)
        mask = (idx[None, :] <= idx[:, None]) & (idx[None, :] >= first[:, None])
        log_d = lic[None, :] + cumf[:, None] - cumf[None, :] - m[:, None]
        D = torch.where(mask, torch.exp(log_d), torch.zeros_like(log_d))
        w = torch.where(live, torch.exp(m_in + cumf - m), torch.zeros_like(cumf))
        kap = torch.where(keep, torch.exp(lic + cumf[-1] - cumf - m[-1]), torch.zeros_like(cumf))
        delta = torch.exp(m_in + cumf[-1] - m[-1]) if not has_reset else torch.zeros((), dtype=dt)
        P = D * (qc @ kc.t())
        Vx = torch.cat([vc, torch.ones(L, 1, dtype=dt)], 1)
        inter = (w[:, None] * qc) @ Sx
        Ox = P @ Vx + inter
        den = torch.maximum(Ox[:, d].abs(), torch.exp(-m)) + eps
        hs.append(Ox[:, :d] / den[:, None])
        saved.append(dict(t0=t0, t1=t1, Sx_in=Sx, m=m, D=D, w=w, kap=kap, delta=delta, P=P, Vx=Vx, inter=inter, Ox=Ox,
                          den=den, mask=mask))
        Sx = delta * Sx + kc.t() @ (kap[:, None] * Vx)
        m_in = m[-1]
    h = torch.cat(hs, 0)
    carry_out = (Sx[:, :d].clone(), Sx[:, d].clone(), m_in.clone())

    dSx = torch.cat([dc_last, dn_last[:, None]], 1)
    g = {n: torch.zeros_like(t) for n, t in (("q", q), ("k", k), ("v", v), ("li", li), ("lf", lf))}
    dm_exp = torch.zeros(T, dtype=dt)
    dm_exp[T - 1] += dm_last - (dSx * Sx).sum()       # the stabilised next carry scales with exp(-m_T)
    for c in reversed(range(nch)):
        s = saved[c]
        t0, t1 = s["t0"], s["t1"]
        qc, kc = q[t0:t1], k[t0:t1]
        dhc = dh[t0:t1]
        num, qn, den = s["Ox"][:, :d], s["Ox"][:, d], s["den"]
        dden = -(dhc * num).sum(1) / den ** 2
        dqn = torch.where(qn.abs() >= torch.exp(-s["m"]), torch.sign(qn) * dden, torch.zeros_like(dden))
        dm_exp[t0:t1] += eps * dden
        dOx = torch.cat([dhc / den[:, None], dqn[:, None]], 1)
        dP = (dOx @ s["Vx"].t()) * s["mask"]
        E = dP * s["P"]
        dA = s["D"] * dP
        kapVx = s["kap"][:, None] * s["Vx"]
        y = kc @ dSx
        g["v"][t0:t1] = (s["P"].t() @ dOx + s["kap"][:, None] * y)[:, :d]
        e_kap = (kapVx * y).sum(1)
        g["q"][t0:t1] = dA @ kc + (s["w"][:, None] * dOx) @ s["Sx_in"].t()
        g["k"][t0:t1] = dA.t() @ qc + kapVx @ dSx.t()
        e_w = (dOx * s["inter"]).sum(1)
        e_delta = s["delta"] * (dSx * s["Sx_in"]).sum()
        dcumf = E.sum(1) - E.sum(0) + e_w - e_kap
        dcumf[-1] += e_kap.sum() + e_delta
        g["li"][t0:t1] += E.sum(0) + e_kap
        g["lf"][t0:t1] += torch.flip(torch.cumsum(torch.flip(dcumf, [0]), 0), [0])
        dSx = s["delta"] * dSx + (s["w"][:, None] * qc).t() @ dOx
    carry = torch.zeros((), dtype=dt)
    for t in reversed(range(T)):
        gt = dm_exp[t] + carry
        m_prev = m_all[t - 1] if t > 0 else m0
        if done[t] > 0 or li[t] > m_prev + lf[t]:
            g["li"][t] += gt
            carry = torch.zeros((), dtype=dt)
        else:
            g["lf"][t] += gt
            carry = gt
    g["c0"], g["n0"] = dSx[:, :d], dSx[:, d]
    g["m0"] = carry + (dSx * torch.cat([c0, n0[:, None]], 1)).sum()
    return h, carry_out, g


# --------------------------------------------------------------------------
# fp32 multi-threaded port timed as the CPU baseline of the benchmark
# --------------------------------------------------------------------------


def linattn_reference_form(q, k, v, s0, z0, done, eps=1e-6):
    """The reference's own O(T d^2) formulation, vectorised: materialise every
    per-step outer product (linear_attention.py:78), take the reset-aware
    inclusive prefix over time (memoroid.py:60-91; here segment-wise cumsum,
    which an additive operator's prefix scan equals), then read
    (linear_attention.py:100-109).  Differentiable; used for timing."""
    bsz, steps, heads, _ = q.shape
    fq, fk = elu_plus_one(q), elu_plus_one(k)
    outer = torch.einsum("bthi,bthj->bthij", v, fk)
    outer = torch.cat([s0[:, None], outer], dim=1)
    keys = torch.cat([z0[:, None], fk], dim=1)
    flags = torch.cat([torch.zeros_like(done[:, :1]), done], dim=1)
    seg = torch.cumsum(flags, dim=1)
    cs = torch.cumsum(outer, dim=1)
    cz = torch.cumsum(keys, dim=1)
    # subtract the prefix that ended just before the last reset
    idx = torch.arange(steps + 1, device=q.device)[None].expand(bsz, -1)
    start = torch.where(flags > 0, idx, torch.zeros_like(idx))
    start = torch.cummax(start, dim=1).values
    prev = torch.clamp(start - 1, min=0)
    gate = (start > 0).to(q.dtype)
    base_s = torch.gather(cs, 1, prev[:, :, None, None, None].expand_as(cs))
    base_z = torch.gather(cz, 1, prev[:, :, None, None].expand_as(cz))
    s_all = cs - gate[:, :, None, None, None] * base_s
    z_all = cz - gate[:, :, None, None] * base_z
    del seg
    num = torch.einsum("bthij,bthj->bthi", s_all[:, 1:], fq)
    den = torch.clamp(torch.einsum("bthi,bthi->bth", fq, z_all[:, 1:]), min=eps)
    return num / den[..., None], s_all[:, -1], z_all[:, -1]
