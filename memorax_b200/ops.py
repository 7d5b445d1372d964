"""PyTorch-facing wrappers of the mxk C-ABI: raw launches on device tensors and
``torch.autograd.Function`` classes that mirror a ``custom_vjp`` split (the
forward returns residuals, the backward consumes cotangents).

PyTorch is plumbing only (device memory, streams).  Every function here ends
in a call through ``include/mxk.h``; nothing falls back to PyTorch math.
"""
from __future__ import annotations

import ctypes

import torch
from torch.nn import functional as F

from . import _lib


# ------------------------------------------------------------------ helpers
def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t, dtype, name):
    """Device tensor of the given dtype in the dense layout the C-ABI requires.  The ABI has no stride
    arguments; a strided view (e.g. a time slice ``x[:, :h]``) is copied here, once, before the launch."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (memorax_b200 has no CPU path)")
    if t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _done_bytes(done):
    """(B,T) flags of any dtype -> contiguous uint8 on the device (bool is reinterpreted)."""
    if done is None:
        return None
    if not done.is_cuda:
        raise ValueError("done must be a CUDA tensor")
    if done.dtype == torch.bool:
        return done.contiguous().view(torch.uint8)
    if done.dtype == torch.uint8:
        return done.contiguous()
    return (done != 0).contiguous().view(torch.uint8)


# ------------------------------------------------- diagonal linear recurrence
def linrec_fwd(a, b, h0=None, a0=None, done=None, want_decay=True):
    """h_t = done_t ? b_t : a_t h_{t-1} + b_t over (B,T,D); ``a`` is (B,T,D) or a
    time-invariant (D,).  Returns ``(h, a_last)`` (a_last None unless wanted).
    float32 or complex64, chosen by ``b.dtype``."""
    cplx = b.is_complex()
    dt = torch.complex64 if cplx else torch.float32
    b = _dev(b, dt, "b")
    a = _dev(a, dt, "a")
    h0, a0 = _dev(h0, dt, "h0"), _dev(a0, dt, "a0")
    bsz, steps, dim = b.shape
    tinv = a.dim() == 1
    if tinv:
        assert a.shape == (dim,)
    else:
        assert a.shape == b.shape
    h = torch.empty_like(b)
    a_last = torch.empty(bsz, dim, dtype=dt, device=b.device) if want_decay else None
    fn = "mxk_linrec_c64_fwd" if cplx else "mxk_linrec_f32_fwd"
    _lib.call(fn, _ptr(a), int(tinv), _ptr(b), _ptr(h0), _ptr(a0), _ptr(_done_bytes(done)), _ptr(h),
              _ptr(a_last), bsz, steps, dim, _stream())
    return h, a_last


def linrec_bwd(a, h, h0, done, gh, gh_last=None, need_ga=True, need_gh0=True, conjugate=False):
    """Cotangents ``(gb, ga, gh0)`` of :func:`linrec_fwd`.  For complex inputs the
    cotangents are in JAX's convention unless ``conjugate`` (torch's)."""
    cplx = h.is_complex()
    dt = torch.complex64 if cplx else torch.float32
    a, h, gh = _dev(a, dt, "a"), _dev(h, dt, "h"), _dev(gh, dt, "gh")
    h0, gh_last = _dev(h0, dt, "h0"), _dev(gh_last, dt, "gh_last")
    bsz, steps, dim = h.shape
    tinv = a.dim() == 1
    gb = torch.empty_like(h)
    ga = (torch.empty_like(a) if need_ga else None)
    gh0 = torch.empty(bsz, dim, dtype=dt, device=h.device) if need_gh0 else None
    ws, ws_bytes = None, 0
    if need_ga and tinv:
        ws_bytes = _lib.lib.mxk_linrec_bwd_workspace_bytes(int(cplx), 1, bsz, steps, dim)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=h.device)
    args = [_ptr(a), int(tinv), _ptr(h), _ptr(h0), _ptr(_done_bytes(done)), _ptr(gh), _ptr(gh_last), _ptr(gb),
            _ptr(ga), _ptr(gh0), _ptr(ws), ws_bytes, bsz, steps, dim]
    if cplx:
        _lib.call("mxk_linrec_c64_bwd", *args, int(conjugate), _stream())
    else:
        _lib.call("mxk_linrec_f32_bwd", *args, _stream())
    return gb, ga, gh0


class LinRec(torch.autograd.Function):
    """(a, b, h0, a0, done) -> (h, a_last).  ``a_last`` (the decay leaf of the
    next carry) is returned for state parity with memoroid.py:89 but carries no
    gradient: no read-out in the reference consumes it."""

    @staticmethod
    def forward(ctx, a, b, h0, a0, done):
        h, a_last = linrec_fwd(a, b, h0, a0, done, want_decay=True)
        ctx.save_for_backward(a, h, h0, done)
        ctx.mark_non_differentiable(a_last)
        return h, a_last

    @staticmethod
    def backward(ctx, gh, _ga_last):
        a, h, h0, done = ctx.saved_tensors
        need_a, need_b, need_h0 = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        gb, ga, gh0 = linrec_bwd(a, h, h0, done, gh.contiguous(), None, need_ga=need_a,
                                 need_gh0=need_h0 and h0 is not None, conjugate=True)
        return ga, (gb if need_b else None), gh0, None, None


# ------------------------------------------- real recurrence, decay per group
def grouped_decay_supported(dim, groups):
    """Whether the grouped-decay kernels take this shape (each group a multiple of 128 channels)."""
    return groups > 0 and dim % groups == 0 and (dim // groups) % 128 == 0


def linrec_last(a, b, h0=None, done=None):
    """The state after the last step, h_T (B,D), of :func:`linrec_fwd`'s recurrence, without storing the T states."""
    cplx = b.is_complex()
    dt = torch.complex64 if cplx else torch.float32
    a, b, h0 = _dev(a, dt, "a"), _dev(b, dt, "b"), _dev(h0, dt, "h0")
    bsz, steps, dim = b.shape
    tinv = a.dim() == 1
    assert a.shape == ((dim,) if tinv else b.shape)
    h_last = torch.empty(bsz, dim, dtype=dt, device=b.device)
    _lib.call("mxk_linrec_c64_last" if cplx else "mxk_linrec_f32_last", _ptr(a), int(tinv), _ptr(b), _ptr(h0),
              _ptr(_done_bytes(done)), _ptr(h_last), bsz, steps, dim, _stream())
    return h_last


def linrec_grouped_last(a, b, h0=None, done=None):
    """h_T (B,D) of :func:`linrec_grouped_fwd`'s recurrence, without storing the T states."""
    a, b, h0 = _dev(a, torch.float32, "a"), _dev(b, torch.float32, "b"), _dev(h0, torch.float32, "h0")
    bsz, steps, dim = b.shape
    groups = a.shape[-1]
    assert a.shape == (bsz, steps, groups)
    h_last = torch.empty(bsz, dim, dtype=torch.float32, device=b.device)
    _lib.call("mxk_linrec_f32_grouped_last", _ptr(a), _ptr(b), _ptr(h0), _ptr(_done_bytes(done)), _ptr(h_last),
              bsz, steps, dim, groups, _stream())
    return h_last


def linrec_grouped_fwd(a, b, h0=None, a0=None, done=None, want_decay=True):
    """h_t[c] = done_t ? b_t[c] : a_t[c // group] h_{t-1}[c] + b_t[c]; ``a`` is (B,T,G), ``b`` (B,T,D) with
    D = G * group.  Returns ``(h, a_last)`` with the carry's decay leaf ``a_last`` (B,G)."""
    a, b = _dev(a, torch.float32, "a"), _dev(b, torch.float32, "b")
    h0, a0 = _dev(h0, torch.float32, "h0"), _dev(a0, torch.float32, "a0")
    bsz, steps, dim = b.shape
    groups = a.shape[-1]
    assert a.shape == (bsz, steps, groups)
    h = torch.empty_like(b)
    a_last = torch.empty(bsz, groups, dtype=torch.float32, device=b.device) if want_decay else None
    _lib.call("mxk_linrec_f32_grouped_fwd", _ptr(a), _ptr(b), _ptr(h0), _ptr(a0), _ptr(_done_bytes(done)), _ptr(h),
              _ptr(a_last), bsz, steps, dim, groups, _stream())
    return h, a_last


def linrec_grouped_bwd(a, h, h0, done, gh, gh_last=None, need_ga=True, need_gh0=True):
    """Cotangents ``(gb, ga, gh0)`` of :func:`linrec_grouped_fwd`; ``ga`` is (B,T,G)."""
    a, h, gh = _dev(a, torch.float32, "a"), _dev(h, torch.float32, "h"), _dev(gh, torch.float32, "gh")
    h0, gh_last = _dev(h0, torch.float32, "h0"), _dev(gh_last, torch.float32, "gh_last")
    bsz, steps, dim = h.shape
    groups = a.shape[-1]
    gb = torch.empty_like(h)
    ga = torch.empty_like(a) if need_ga else None
    gh0 = torch.empty(bsz, dim, dtype=torch.float32, device=h.device) if need_gh0 else None
    ws_bytes = _lib.lib.mxk_linrec_grouped_bwd_workspace_bytes(bsz, steps, dim, groups) if need_ga else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=h.device) if ws_bytes else None
    _lib.call("mxk_linrec_f32_grouped_bwd", _ptr(a), _ptr(h), _ptr(h0), _ptr(_done_bytes(done)), _ptr(gh),
              _ptr(gh_last), _ptr(gb), _ptr(ga), _ptr(gh0), _ptr(ws), ws_bytes, bsz, steps, dim, groups, _stream())
    return gb, ga, gh0


class LinRecGrouped(torch.autograd.Function):
    """(a (B,T,G), b (B,T,D), h0, a0 (B,G), done) -> (h, a_last (B,G)); ``a_last`` carries no gradient."""

    @staticmethod
    def forward(ctx, a, b, h0, a0, done):
        h, a_last = linrec_grouped_fwd(a, b, h0, a0, done, want_decay=True)
        ctx.save_for_backward(a, h, h0, done)
        ctx.mark_non_differentiable(a_last)
        return h, a_last

    @staticmethod
    def backward(ctx, gh, _ga_last):
        a, h, h0, done = ctx.saved_tensors
        gb, ga, gh0 = linrec_grouped_bwd(a, h, h0, done, gh.contiguous(), None, need_ga=ctx.needs_input_grad[0],
                                         need_gh0=ctx.needs_input_grad[2] and h0 is not None)
        return ga, (gb if ctx.needs_input_grad[1] else None), gh0, None, None


# --------------------------------------------------------- log-space (MinGRU)
def loglinrec_fwd(ls, d, x0=None, a0=None, done=None, want_y=True, want_decay=True):
    ls, d = _dev(ls, torch.float32, "ls"), _dev(d, torch.float32, "d")
    x0, a0 = _dev(x0, torch.float32, "x0"), _dev(a0, torch.float32, "a0")
    bsz, steps, dim = ls.shape
    x = torch.empty_like(ls)
    y = torch.empty_like(ls) if want_y else None
    a_last = torch.empty(bsz, dim, dtype=torch.float32, device=ls.device) if want_decay else None
    _lib.call("mxk_loglinrec_f32_fwd", _ptr(ls), _ptr(d), _ptr(x0), _ptr(a0), _ptr(_done_bytes(done)), _ptr(x),
              _ptr(y), _ptr(a_last), bsz, steps, dim, _stream())
    return x, y, a_last


def loglinrec_bwd(d, x, x0, done, gx=None, gy=None, gx_last=None, need_gx0=True):
    d, x = _dev(d, torch.float32, "d"), _dev(x, torch.float32, "x")
    x0, gx, gy = _dev(x0, torch.float32, "x0"), _dev(gx, torch.float32, "gx"), _dev(gy, torch.float32, "gy")
    gx_last = _dev(gx_last, torch.float32, "gx_last")
    bsz, steps, dim = x.shape
    gls, gd = torch.empty_like(x), torch.empty_like(x)
    gx0 = torch.empty(bsz, dim, dtype=torch.float32, device=x.device) if need_gx0 else None
    _lib.call("mxk_loglinrec_f32_bwd", _ptr(d), _ptr(x), _ptr(x0), _ptr(_done_bytes(done)), _ptr(gx), _ptr(gy),
              _ptr(gx_last), _ptr(gls), _ptr(gd), _ptr(gx0), bsz, steps, dim, _stream())
    return gls, gd, gx0


class LogLinRec(torch.autograd.Function):
    """(ls, d, x0, a0, done) -> (x, y = exp(x), a_last)."""

    @staticmethod
    def forward(ctx, ls, d, x0, a0, done):
        x, y, a_last = loglinrec_fwd(ls, d, x0, a0, done)
        ctx.save_for_backward(d, x, x0, done)
        ctx.mark_non_differentiable(a_last)
        return x, y, a_last

    @staticmethod
    def backward(ctx, gx, gy, _ga_last):
        d, x, x0, done = ctx.saved_tensors
        gls, gd, gx0 = loglinrec_bwd(d, x, x0, done, gx.contiguous(), gy.contiguous(), None,
                                     need_gx0=x0 is not None and ctx.needs_input_grad[2])
        return gls, gd, gx0, None, None


class MinGRUFused(torch.autograd.Function):
    """(z, h_tilde, x0, a0, done) -> (x, y = exp(x), a_last): MinGRU's gate math (min_gru.py:52-61), scan and
    read-out in one kernel per direction; ``z`` / ``h_tilde`` are the Dense layers' pre-activations."""

    @staticmethod
    def forward(ctx, z, h_tilde, x0, a0, done):
        z, h_tilde = _dev(z, torch.float32, "z"), _dev(h_tilde, torch.float32, "h_tilde")
        x0, a0 = _dev(x0, torch.float32, "x0"), _dev(a0, torch.float32, "a0")
        bsz, steps, dim = z.shape
        x, y = torch.empty_like(z), torch.empty_like(z)
        a_last = torch.empty(bsz, dim, dtype=torch.float32, device=z.device)
        _lib.call("mxk_mingru_f32_fwd", _ptr(z), _ptr(h_tilde), _ptr(x0), _ptr(a0), _ptr(_done_bytes(done)), _ptr(x),
                  _ptr(y), _ptr(a_last), bsz, steps, dim, _stream())
        ctx.save_for_backward(z, h_tilde, x, x0, done)
        ctx.mark_non_differentiable(a_last)
        return x, y, a_last

    @staticmethod
    def backward(ctx, gx, gy, _ga_last):
        z, h_tilde, x, x0, done = ctx.saved_tensors
        bsz, steps, dim = z.shape
        gz, gh = torch.empty_like(z), torch.empty_like(z)
        gx0 = torch.empty(bsz, dim, dtype=torch.float32, device=z.device) if (x0 is not None and ctx.needs_input_grad[2]) else None
        _lib.call("mxk_mingru_f32_bwd", _ptr(z), _ptr(h_tilde), _ptr(x), _ptr(x0), _ptr(_done_bytes(done)),
                  _ptr(gx.contiguous()), _ptr(gy.contiguous()), None, _ptr(gz), _ptr(gh), _ptr(gx0), bsz, steps, dim, _stream())
        return gz, gh, gx0, None, None


# ------------------------------------------------------- device status word
# One int32 per device that every tensor-core launch is handed: a kernel whose bounded wait gave up
# sets it to 1 and drains.  ``check=True`` on a wrapper reads it right after the launch (one host
# sync); the autograd Functions never sync -- call :func:`check_status` where a sync is affordable
# (end of a training step, end of a rollout).
_STATUS_WORDS = {}


def _status_word(device):
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS_WORDS.get(key)
    if word is None:
        word = _STATUS_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return word


def _check_status(word, what):
    value = int(word.item())
    if value != 0:
        word.zero_()
        raise _lib.MxkError(what, value, "a bounded device-side wait gave up; the results of launches since "
                                         "the last check are undefined")


def check_status(device=None):
    """Raise :class:`MxkError` if any launch on ``device`` since the last check reported that a bounded
    device-side wait gave up (synchronises with the device).  The word is cleared on failure."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _check_status(_status_word(device), "memorax_b200 kernels")


def selftest_bounded_wait(polls=2, device=None):
    """Launch the library's failure-path self-test: a kernel that waits, bounded, on a barrier nothing
    completes.  Returns the status word's value afterwards (1 = the wait gave up and reported it)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = torch.zeros(1, dtype=torch.int32, device=device)
    _lib.call("mxk_selftest_bounded_wait", _ptr(word), int(polls), _stream())
    return int(word.item())


# ------------------------------------------------------- linear attention


def linattn_fwd(q, k, v, s0=None, z0=None, done=None, eps=1e-6, feature_map=True, save_states=False,
                check=False):
    """Chunked causal linear attention; q, k, v are (B,T,H,d) bf16, d a multiple of 8 up to 64.  Returns
    ``(o, s_last, z_last, chunk_states)`` (chunk_states None unless asked for)."""
    q, k, v = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    s0, z0 = _dev(s0, torch.float32, "s0"), _dev(z0, torch.float32, "z0")
    bsz, steps, heads, dim = q.shape
    assert k.shape == q.shape and v.shape == q.shape
    o = torch.empty_like(q)
    s_last = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device)
    z_last = torch.empty(bsz, heads, dim, dtype=torch.float32, device=q.device)
    states = None
    if save_states:
        nbytes = _lib.lib.mxk_linattn_chunk_states_bytes(bsz, steps, heads, dim)
        states = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    status = _status_word(q.device)
    _lib.call("mxk_linattn_bf16_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(s0), _ptr(z0), _ptr(_done_bytes(done)),
              _ptr(o), _ptr(s_last), _ptr(z_last), _ptr(states), _ptr(status), bsz, steps, heads, dim,
              float(eps), int(feature_map), _stream())
    if check:
        _check_status(status, "mxk_linattn_bf16_fwd")
    return o, s_last, z_last, states


def linattn_bwd(q, k, v, d_o, chunk_states, done=None, ds_last=None, dz_last=None, eps=1e-6, feature_map=True,
                check=False, need_state_grads=True):
    """Cotangents ``(dq, dk, dv, ds0, dz0)`` of :func:`linattn_fwd` (the last two ``None`` unless wanted)."""
    q, k, v, d_o = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v"), (d_o, "d_o")))
    ds_last, dz_last = _dev(ds_last, torch.float32, "ds_last"), _dev(dz_last, torch.float32, "dz_last")
    bsz, steps, heads, dim = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    ds0 = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device) if need_state_grads else None
    dz0 = torch.empty(bsz, heads, dim, dtype=torch.float32, device=q.device) if need_state_grads else None
    status = _status_word(q.device)
    _lib.call("mxk_linattn_bf16_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(d_o), _ptr(chunk_states),
              _ptr(_done_bytes(done)), _ptr(ds_last), _ptr(dz_last), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(ds0),
              _ptr(dz0), _ptr(status), bsz, steps, heads, dim, float(eps), int(feature_map), _stream())
    if check:
        _check_status(status, "mxk_linattn_bf16_bwd")
    return dq, dk, dv, ds0, dz0


class LinAttn(torch.autograd.Function):
    """(q, k, v, s0, z0, done) -> (o, s_last, z_last); the forward keeps the
    per-chunk states as its residual."""

    @staticmethod
    def forward(ctx, q, k, v, s0, z0, done, eps, feature_map):
        o, s_last, z_last, states = linattn_fwd(q, k, v, s0, z0, done, eps, feature_map, save_states=True)
        ctx.save_for_backward(q, k, v, states, done)
        ctx.eps, ctx.feature_map = eps, feature_map
        ctx.has_state = (s0 is not None, z0 is not None)
        ctx.set_materialize_grads(False)     # an unused carry arrives as None, not as a tensor of zeros
        return o, s_last, z_last

    @staticmethod
    def backward(ctx, d_o, ds_last, dz_last):
        q, k, v, states, done = ctx.saved_tensors
        if d_o is None:
            d_o = torch.zeros_like(q)
        dq, dk, dv, ds0, dz0 = linattn_bwd(q, k, v, d_o, states, done, ds_last, dz_last, ctx.eps, ctx.feature_map,
                                           need_state_grads=any(ctx.has_state))
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), ds0 if ctx.has_state[0] else None,
                dz0 if ctx.has_state[1] else None, None, None, None)


# -------------------------------------------------------------------- mLSTM
def mlstm_fwd(q, k, v, log_i, log_f, c0=None, n0=None, m0=None, f0=None, done=None, eps=1e-6):
    """Stabilised mLSTM scan + read-out; q, k, v (B,T,H,d) fp32 (k already divided by sqrt(d)), gates (B,T,H).
    Returns ``(h, c_last, n_last, m_last, f_last)``."""
    q, k, v = (_dev(t, torch.float32, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    log_i, log_f = _dev(log_i, torch.float32, "log_i"), _dev(log_f, torch.float32, "log_f")
    c0, n0, m0, f0 = (_dev(t, torch.float32, n) for t, n in ((c0, "c0"), (n0, "n0"), (m0, "m0"), (f0, "f0")))
    bsz, steps, heads, dim = q.shape
    assert log_i.shape == (bsz, steps, heads) and log_f.shape == log_i.shape
    h = torch.empty_like(q)
    c_last = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device)
    n_last = torch.empty(bsz, heads, dim, dtype=torch.float32, device=q.device)
    m_last = torch.empty(bsz, heads, dtype=torch.float32, device=q.device)
    f_last = torch.empty(bsz, heads, dtype=torch.float32, device=q.device)
    _lib.call("mxk_mlstm_f32_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(log_i), _ptr(log_f), _ptr(c0), _ptr(n0), _ptr(m0),
              _ptr(f0), _ptr(_done_bytes(done)), _ptr(h), _ptr(c_last), _ptr(n_last), _ptr(m_last), _ptr(f_last),
              bsz, steps, heads, dim, float(eps), _stream())
    return h, c_last, n_last, m_last, f_last


def mlstm_bwd(q, k, v, log_i, log_f, c0, n0, m0, done, dh, dc_last=None, dn_last=None, dm_last=None, eps=1e-6):
    """Cotangents ``(dq, dk, dv, dlog_i, dlog_f, dc0, dn0, dm0)`` of :func:`mlstm_fwd`."""
    q, k, v, dh = (_dev(t, torch.float32, n) for t, n in ((q, "q"), (k, "k"), (v, "v"), (dh, "dh")))
    log_i, log_f = _dev(log_i, torch.float32, "log_i"), _dev(log_f, torch.float32, "log_f")
    c0, n0, m0 = (_dev(t, torch.float32, n) for t, n in ((c0, "c0"), (n0, "n0"), (m0, "m0")))
    dc_last, dn_last, dm_last = (_dev(t, torch.float32, n) for t, n in ((dc_last, "dc_last"), (dn_last, "dn_last"),
                                                                         (dm_last, "dm_last")))
    bsz, steps, heads, dim = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    dli, dlf = torch.empty_like(log_i), torch.empty_like(log_f)
    dc0 = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device)
    dn0 = torch.empty(bsz, heads, dim, dtype=torch.float32, device=q.device)
    dm0 = torch.empty(bsz, heads, dtype=torch.float32, device=q.device)
    ws_bytes = _lib.lib.mxk_mlstm_bwd_workspace_bytes(bsz, steps, heads, dim)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    _lib.call("mxk_mlstm_f32_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(log_i), _ptr(log_f), _ptr(c0), _ptr(n0), _ptr(m0),
              _ptr(_done_bytes(done)), _ptr(dh), _ptr(dc_last), _ptr(dn_last), _ptr(dm_last), _ptr(dq), _ptr(dk),
              _ptr(dv), _ptr(dli), _ptr(dlf), _ptr(dc0), _ptr(dn0), _ptr(dm0), _ptr(ws), ws_bytes, bsz, steps, heads, dim,
              float(eps), _stream())
    return dq, dk, dv, dli, dlf, dc0, dn0, dm0


class MLSTM(torch.autograd.Function):
    """(q, k, v, log_i, log_f, c0, n0, m0, f0, done) -> (h, c_last, n_last, m_last, f_last); the log_f leaf of
    the carry (f0 / f_last) is returned for state parity and carries no gradient."""

    @staticmethod
    def forward(ctx, q, k, v, log_i, log_f, c0, n0, m0, f0, done, eps):
        h, c_last, n_last, m_last, f_last = mlstm_fwd(q, k, v, log_i, log_f, c0, n0, m0, f0, done, eps)
        ctx.save_for_backward(q, k, v, log_i, log_f, c0, n0, m0, done)
        ctx.eps = eps
        ctx.mark_non_differentiable(f_last)
        return h, c_last, n_last, m_last, f_last

    @staticmethod
    def backward(ctx, dh, dc_last, dn_last, dm_last, _df_last):
        q, k, v, log_i, log_f, c0, n0, m0, done = ctx.saved_tensors
        dq, dk, dv, dli, dlf, dc0, dn0, dm0 = mlstm_bwd(q, k, v, log_i, log_f, c0, n0, m0, done, dh.contiguous(),
                                                        dc_last, dn_last, dm_last, ctx.eps)
        return (dq, dk, dv, dli, dlf, dc0 if c0 is not None else None, dn0 if n0 is not None else None,
                dm0 if m0 is not None else None, None, None, None)


# --------------------------------------------------------- gated delta rule
def gdelta_fwd(q, k, v, alpha, beta, s0=None, done=None, save_states=False, check=False):
    """Gated delta rule; q, k, v (B,T,H,d) bf16 with d = 128 or 64, alpha/beta (B,T,H) fp32.
    Returns ``(o, s_last, chunk_states)``; with ``save_states`` the third item is the pair
    ``(chunk_states, workspace)`` that :func:`gdelta_bwd` takes."""
    q, k, v = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    alpha, beta = _dev(alpha, torch.float32, "alpha"), _dev(beta, torch.float32, "beta")
    s0 = _dev(s0, torch.float32, "s0")
    bsz, steps, heads, dim = q.shape
    assert alpha.shape == (bsz, steps, heads) and beta.shape == alpha.shape
    o = torch.empty_like(q)
    s_last = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device)
    states = None
    if save_states:
        states = torch.empty(_lib.lib.mxk_gdelta_chunk_states_bytes(bsz, steps, heads, dim), dtype=torch.uint8,
                             device=q.device)
    ws_bytes = _lib.lib.mxk_gdelta_workspace_bytes(bsz, steps, heads, dim)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    status = _status_word(q.device)
    _lib.call("mxk_gdelta_bf16_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(alpha), _ptr(beta), _ptr(s0),
              _ptr(_done_bytes(done)), _ptr(o), _ptr(s_last), _ptr(states), _ptr(workspace), ws_bytes, _ptr(status),
              bsz, steps, heads, dim, _stream())
    if check:
        _check_status(status, "mxk_gdelta_bf16_fwd")
    return o, s_last, ((states, workspace) if save_states else None)


def gdelta_bwd(q, k, v, alpha, beta, d_o, chunk_states, done=None, ds_last=None, check=False, need_ds0=True):
    """Cotangents ``(dq, dk, dv, dalpha, dbeta, ds0)`` of :func:`gdelta_fwd` (``ds0`` ``None`` unless wanted)."""
    q, k, v, d_o = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v"), (d_o, "d_o")))
    alpha, beta = _dev(alpha, torch.float32, "alpha"), _dev(beta, torch.float32, "beta")
    ds_last = _dev(ds_last, torch.float32, "ds_last")
    chunk_states, workspace = chunk_states
    bsz, steps, heads, dim = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    dalpha, dbeta = torch.empty_like(alpha), torch.empty_like(beta)
    ds0 = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=q.device) if need_ds0 else None
    status = _status_word(q.device)
    _lib.call("mxk_gdelta_bf16_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(alpha), _ptr(beta), _ptr(d_o),
              _ptr(chunk_states), _ptr(workspace), _ptr(_done_bytes(done)), _ptr(ds_last), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dalpha),
              _ptr(dbeta), _ptr(ds0), _ptr(status), bsz, steps, heads, dim, _stream())
    if check:
        _check_status(status, "mxk_gdelta_bf16_bwd")
    return dq, dk, dv, dalpha, dbeta, ds0


class GatedDelta(torch.autograd.Function):
    """(q, k, v, alpha, beta, s0, done) -> (o, s_last)."""

    @staticmethod
    def forward(ctx, q, k, v, alpha, beta, s0, done):
        o, s_last, (states, workspace) = gdelta_fwd(q, k, v, alpha, beta, s0, done, save_states=True)
        ctx.save_for_backward(q, k, v, alpha, beta, states, workspace, done)
        ctx.has_state = s0 is not None
        ctx.set_materialize_grads(False)     # an unused carry arrives as None, not as a tensor of zeros
        return o, s_last

    @staticmethod
    def backward(ctx, d_o, ds_last):
        q, k, v, alpha, beta, states, workspace, done = ctx.saved_tensors
        if d_o is None:
            d_o = torch.zeros_like(q)
        dq, dk, dv, dalpha, dbeta, ds0 = gdelta_bwd(q, k, v, alpha, beta, d_o, (states, workspace), done, ds_last,
                                                    need_ds0=ctx.has_state)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dalpha.to(alpha.dtype), dbeta.to(beta.dtype),
                ds0 if ctx.has_state else None, None)


# --------------------------------------------------- mLSTM on the tensor cores
def mlstm_tc_fwd(q, k, v, log_i, log_f, c0=None, n0=None, m0=None, f0=None, done=None, eps=1e-6, save=False,
                 check=False):
    """Chunked mLSTM scan + read-out on the tensor cores; q, k, v (B,T,H,d) bf16 (k already divided by sqrt(d)),
    d a multiple of 8 up to 64; gates (B,T,H) fp32.  Returns ``(h, c_last, n_last, m_last, f_last, residual)``
    with ``residual = (m_steps, chunk_states)`` when ``save`` (else None)."""
    q, k, v = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    log_i, log_f = _dev(log_i, torch.float32, "log_i"), _dev(log_f, torch.float32, "log_f")
    c0, n0, m0, f0 = (_dev(t, torch.float32, n) for t, n in ((c0, "c0"), (n0, "n0"), (m0, "m0"), (f0, "f0")))
    bsz, steps, heads, dim = q.shape
    assert log_i.shape == (bsz, steps, heads) and log_f.shape == log_i.shape
    dev = q.device
    h = torch.empty_like(q)
    c_last = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=dev)
    n_last = torch.empty(bsz, heads, dim, dtype=torch.float32, device=dev)
    m_last = torch.empty(bsz, heads, dtype=torch.float32, device=dev)
    f_last = torch.empty(bsz, heads, dtype=torch.float32, device=dev)
    m_steps = states = None
    if save:
        m_steps = torch.empty(bsz, steps, heads, dtype=torch.float32, device=dev)
        states = torch.empty(_lib.lib.mxk_mlstm_bf16_chunk_states_bytes(bsz, steps, heads, dim), dtype=torch.uint8, device=dev)
    status = _status_word(dev)
    _lib.call("mxk_mlstm_bf16_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(log_i), _ptr(log_f), _ptr(c0), _ptr(n0), _ptr(m0),
              _ptr(f0), _ptr(_done_bytes(done)), _ptr(h), _ptr(c_last), _ptr(n_last), _ptr(m_last), _ptr(f_last),
              _ptr(m_steps), _ptr(states), _ptr(status), bsz, steps, heads, dim, float(eps), _stream())
    if check:
        _check_status(status, "mxk_mlstm_bf16_fwd")
    return h, c_last, n_last, m_last, f_last, ((m_steps, states) if save else None)


def mlstm_tc_bwd(q, k, v, log_i, log_f, c0, n0, m0, done, dh, c_last, n_last, residual, dc_last=None, dn_last=None,
                 dm_last=None, eps=1e-6, need_state_grads=True, check=False):
    """Cotangents ``(dq, dk, dv, dlog_i, dlog_f, dc0, dn0, dm0)`` of :func:`mlstm_tc_fwd`; ``residual`` is what the
    forward call returned with ``save``, ``c_last`` / ``n_last`` its next carry."""
    q, k, v, dh = (_dev(t, torch.bfloat16, n) for t, n in ((q, "q"), (k, "k"), (v, "v"), (dh, "dh")))
    log_i, log_f = _dev(log_i, torch.float32, "log_i"), _dev(log_f, torch.float32, "log_f")
    c0, n0, m0 = (_dev(t, torch.float32, n) for t, n in ((c0, "c0"), (n0, "n0"), (m0, "m0")))
    dc_last, dn_last, dm_last = (_dev(t, torch.float32, n) for t, n in ((dc_last, "dc_last"), (dn_last, "dn_last"),
                                                                        (dm_last, "dm_last")))
    m_steps, states = residual
    bsz, steps, heads, dim = q.shape
    dev = q.device
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    dli, dlf = torch.empty_like(log_i), torch.empty_like(log_f)
    dc0 = dn0 = dm0 = None
    if need_state_grads:
        dc0 = torch.empty(bsz, heads, dim, dim, dtype=torch.float32, device=dev)
        dn0 = torch.empty(bsz, heads, dim, dtype=torch.float32, device=dev)
        dm0 = torch.empty(bsz, heads, dtype=torch.float32, device=dev)
    status = _status_word(dev)
    _lib.call("mxk_mlstm_bf16_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(log_i), _ptr(log_f), _ptr(c0), _ptr(n0), _ptr(m0),
              _ptr(_done_bytes(done)), _ptr(dh), _ptr(c_last), _ptr(n_last), _ptr(m_steps), _ptr(states), _ptr(dc_last),
              _ptr(dn_last), _ptr(dm_last), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dli), _ptr(dlf), _ptr(dc0), _ptr(dn0),
              _ptr(dm0), _ptr(status), bsz, steps, heads, dim, float(eps), _stream())
    if check:
        _check_status(status, "mxk_mlstm_bf16_bwd")
    return dq, dk, dv, dli, dlf, dc0, dn0, dm0


class MLSTMTensorCore(torch.autograd.Function):
    """(q, k, v, log_i, log_f, c0, n0, m0, f0, done) -> (h, c_last, n_last, m_last, f_last) on the tensor cores
    (bf16 q, k, v, h).  The carry's log_f leaf has no cotangent."""

    @staticmethod
    def forward(ctx, q, k, v, log_i, log_f, c0, n0, m0, f0, done, eps):
        h, c_last, n_last, m_last, f_last, residual = mlstm_tc_fwd(q, k, v, log_i, log_f, c0, n0, m0, f0, done, eps, save=True)
        ctx.save_for_backward(q, k, v, log_i, log_f, c0, n0, m0, done, c_last, n_last, *residual)
        ctx.eps = eps
        ctx.has_state = any(t is not None for t in (c0, n0, m0))
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(f_last)
        return h, c_last, n_last, m_last, f_last

    @staticmethod
    def backward(ctx, dh, dc_last, dn_last, dm_last, _df_last):
        q, k, v, log_i, log_f, c0, n0, m0, done, c_last, n_last, m_steps, states = ctx.saved_tensors
        if dh is None:
            dh = torch.zeros_like(q)
        dq, dk, dv, dli, dlf, dc0, dn0, dm0 = mlstm_tc_bwd(q, k, v, log_i, log_f, c0, n0, m0, done, dh, c_last, n_last,
                                                           (m_steps, states), dc_last, dn_last, dm_last, ctx.eps,
                                                           need_state_grads=ctx.has_state)
        return (dq, dk, dv, dli, dlf, dc0 if c0 is not None else None, dn0 if n0 is not None else None,
                dm0 if m0 is not None else None, None, None, None)


# ------------------------------------------------------ fused row-wise glue
def _glue_ok(x, dim):
    return x.is_cuda and x.dtype == torch.bfloat16 and dim % 256 == 0 and dim <= 1024


class FusedNorm(torch.autograd.Function):
    """LayerNorm (``rms=False``) or RMSNorm over the last dimension, bf16, one kernel per direction."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        x = x.contiguous()
        dim = x.shape[-1]
        rows = x.numel() // dim
        y = torch.empty_like(x)
        mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _lib.call("mxk_norm_bf16_fwd", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _ptr(mean), _ptr(rstd), rows, dim,
                  float(eps), int(rms), _stream())
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.rms, ctx.has_bias = rms, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dim = x.shape[-1]
        rows = x.numel() // dim
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dgamma = torch.empty(dim, dtype=torch.float32, device=x.device)
        dbeta = None if ctx.rms else torch.empty(dim, dtype=torch.float32, device=x.device)
        ws_bytes = _lib.lib.mxk_norm_bwd_workspace_bytes(rows, dim)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
        _lib.call("mxk_norm_bf16_bwd", _ptr(x), _ptr(weight), _ptr(mean), _ptr(rstd), _ptr(dy), _ptr(dx), _ptr(dgamma),
                  _ptr(dbeta), _ptr(ws), ws_bytes, rows, dim, int(ctx.rms), _stream())
        return (dx, dgamma.to(weight.dtype), dbeta.to(weight.dtype) if (dbeta is not None and ctx.has_bias) else None,
                None, None)


def layer_norm(x, weight, bias, eps=1e-5):
    """nn.LayerNorm over the last dimension; the fused kernels for bf16 CUDA rows of 256..1024 elements."""
    if _glue_ok(x, x.shape[-1]) and weight.dtype == torch.bfloat16 and bias is not None:
        return FusedNorm.apply(x, weight, bias, eps, False)
    return torch.nn.functional.layer_norm(x, x.shape[-1:], weight, bias, eps)


def rms_norm(x, weight, eps=1e-6):
    if _glue_ok(x, x.shape[-1]) and weight.dtype == torch.bfloat16:
        return FusedNorm.apply(x, weight, None, eps, True)
    return torch.nn.functional.rms_norm(x, x.shape[-1:], weight, eps)


class GatedResidual(torch.autograd.Function):
    """y = x + sigmoid(g) * o (blocks/residual.py:53-59), bf16, one kernel per direction."""

    @staticmethod
    def forward(ctx, x, g, o):
        x, g, o = x.contiguous(), g.contiguous(), o.contiguous()
        y = torch.empty_like(x)
        _lib.call("mxk_gated_residual_bf16_fwd", _ptr(x), _ptr(g), _ptr(o), _ptr(y), x.numel(), _stream())
        ctx.save_for_backward(g, o)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, o = ctx.saved_tensors
        dy = dy.contiguous()
        dg, d_o = torch.empty_like(g), torch.empty_like(o)
        _lib.call("mxk_gated_residual_bf16_bwd", _ptr(dy), _ptr(g), _ptr(o), _ptr(dg), _ptr(d_o), dy.numel(), _stream())
        return dy, dg, d_o


def gated_residual(x, g, o):
    if x.is_cuda and x.dtype == g.dtype == o.dtype == torch.bfloat16 and x.numel() % 8 == 0 and x.shape == g.shape == o.shape:
        return GatedResidual.apply(x, g, o)
    return x + torch.sigmoid(g) * o


class L2NormHeads(torch.autograd.Function):
    """x (..., H * head_dim) bf16 -> each head vector divided by max(its norm, eps), bf16."""

    @staticmethod
    def forward(ctx, x, head_dim, eps):
        x = x.contiguous()
        y = torch.empty_like(x)
        _lib.call("mxk_l2norm_heads_bf16", _ptr(x), None, _ptr(y), x.numel() // head_dim, head_dim, float(eps), _stream())
        ctx.save_for_backward(x)
        ctx.head_dim, ctx.eps = head_dim, eps
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        _lib.call("mxk_l2norm_heads_bf16", _ptr(x), _ptr(dy.contiguous()), _ptr(dx), x.numel() // ctx.head_dim, ctx.head_dim,
                  float(ctx.eps), _stream())
        return dx, None, None


class Gelu(torch.autograd.Function):
    """tanh-form GELU (flax's ``nn.gelu`` default) of a bf16 CUDA tensor, one streaming pass each way."""

    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        _lib.call("mxk_gelu_bf16", _ptr(x), None, _ptr(y), x.numel(), _stream())
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        _lib.call("mxk_gelu_bf16", _ptr(x), _ptr(dy.contiguous()), _ptr(dx), x.numel(), _stream())
        return dx


def gelu(x):
    """``flax.linen.gelu`` (tanh form).  bf16 CUDA tensors whose size is a multiple of 8 take the fused kernel."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and x.numel() > 0:
        return Gelu.apply(x)
    return F.gelu(x, approximate="tanh")


def colsum(x):
    """Sum over the rows of a (rows, cols) bf16 matrix (fp32 accumulation, fixed order), -> (cols,) bf16."""
    x = x.contiguous()
    rows, cols = x.shape
    out = torch.empty(cols, dtype=torch.bfloat16, device=x.device)
    ws_bytes = _lib.lib.mxk_colsum_workspace_bytes(rows, cols)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    _lib.call("mxk_colsum_bf16", _ptr(x), _ptr(out), _ptr(ws), ws_bytes, rows, cols, _stream())
    return out


class DenseBias(torch.autograd.Function):
    """y = x W^T + b for bf16 CUDA tensors: the two GEMMs of the backward are the library's, the bias gradient
    (a column sum of dy) is this library's fixed-order kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.matmul(dy, weight)
        if ctx.needs_input_grad[1]:
            dw = torch.mm(dy2.t(), x.reshape(-1, x.shape[-1]))
        if ctx.needs_input_grad[2]:
            db = colsum(dy2)
        return dx, dw, db


def dense(x, weight, bias=None):
    """``F.linear`` whose bias gradient runs on :func:`colsum` when it can (bf16 CUDA, out features % 8 == 0)."""
    if (bias is not None and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and bias.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and torch.is_grad_enabled()):
        return DenseBias.apply(x, weight, bias)
    return F.linear(x, weight, bias)


def l2norm_heads(x, head_dim, eps=1e-12):
    """(..., H * head_dim) -> (..., H, head_dim) with every head vector L2-normalised."""
    heads = x.shape[-1] // head_dim
    if x.is_cuda and x.dtype == torch.bfloat16 and head_dim in (64, 128):
        return L2NormHeads.apply(x, head_dim, eps).view(*x.shape[:-1], heads, head_dim)
    return torch.nn.functional.normalize(x.view(*x.shape[:-1], heads, head_dim).float(), dim=-1, eps=eps)


# ------------------------------------------------------------------- Adam
def adam_step(params, grads, m, v, step, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, grad_scale=1.0, master=None):
    """In-place fused Adam on flat buffers (bf16 params/grads, fp32 moments).  With ``master`` (fp32, same
    length) the update is applied to the fp32 copy and ``params`` receives its bf16 rounding."""
    assert params.dtype == torch.bfloat16 and grads.dtype == torch.bfloat16
    assert m.dtype == torch.float32 and v.dtype == torch.float32 and params.is_contiguous() and grads.is_contiguous()
    if master is not None:
        assert master.dtype == torch.float32 and master.is_contiguous() and master.numel() == params.numel()
    _lib.call("mxk_adam_bf16_master", _ptr(params), _ptr(master), _ptr(grads), _ptr(m), _ptr(v), params.numel(),
              float(lr), float(betas[0]), float(betas[1]), float(eps), int(step), float(grad_scale), _stream())
