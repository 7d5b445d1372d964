"""Host-side mirror of memorax's sequence-model interface for the scan path.

Same names, call signatures and carry pytrees as
``memorax/networks/sequence_models/{sequence_model,memoroid,lru,min_gru,
linear_attention}.py``; the time-axis scan that the reference runs with
``jax.lax.associative_scan`` is one fused CUDA launch through the C-ABI here.

* ``SequenceModel.__call__(inputs, done, initial_carry=None) -> (next_carry, y)``
  and ``initialize_carry(key, input_shape)`` (sequence_model.py:8-19);
* ``MemoroidCellBase``: ``__call__(x) -> z``, ``binary_operator(a, b)``,
  ``read(h, x) -> y``, ``initialize_carry`` (memoroid.py:20-54);
* ``Memoroid(cell)`` (memoroid.py:57-112): ``z = cell(x)``; scan; ``y = read``.

Carries keep the reference's singleton time axis: ``(B, 1, ...)``.

Two deliberate differences, both forced by not materialising O(T d^2) data:
the linear-attention and delta-rule cells emit *factored* elements (k, v, ...)
instead of per-step outer products, and their ``scan`` returns the read-out
together with the last state (the reference's ``read`` over every S_t is
fused into the kernel).  ``binary_operator`` is kept on every cell as the
algebraic definition (used by the tests); the product path never calls it.
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F

from . import ops


def get_input_shape(inputs):
    """(B, T, F) -> (B, F)   (utils/axes.py:46-49)."""
    return inputs.shape[:1] + inputs.shape[2:]


def _squeeze_carry(carry, leaves):
    """Carry pytree with the reference's singleton time axis -> per-leaf (B, ...)
    tensors for the C-ABI; ``None`` (default carry) stays ``None`` per leaf."""
    if carry is None:
        return (None,) * leaves
    return tuple(None if c is None else c[:, 0].contiguous() for c in carry)


class SequenceModel(nn.Module):
    def forward(self, inputs, done, initial_carry=None, **kwargs):
        raise NotImplementedError

    def initialize_carry(self, key, input_shape):
        raise NotImplementedError


class MemoroidCellBase(nn.Module):
    """Plugin protocol of a cell (memoroid.py:20-54) plus ``scan``, the fused
    replacement of ``Memoroid.scan_fn`` + ``read`` for this cell."""

    def forward(self, x, **kwargs):
        raise NotImplementedError

    def binary_operator(self, a, b):
        raise NotImplementedError

    def read(self, h, x, **kwargs):
        raise NotImplementedError

    def initialize_carry(self, key, input_shape):
        raise NotImplementedError

    def scan(self, z, initial_carry, done, inputs):
        """-> (next_carry, y)"""
        raise NotImplementedError

    # ---- RTRL hooks (memoroid.py:35-54); a cell without local Jacobians returns None ----
    def local_jacobian(self, carry, z, inputs, **kwargs):
        return None

    def compute_phantom(self, sensitivity):
        """sum over the leaves of S . (param - stop_gradient(param)): zero in value, its gradient with respect
        to the parameters is the sensitivity (memoroid.py:38-47).  Leaves are named by attribute path."""
        phantom = 0
        for name, sens in sensitivity.items():
            param = self
            for key in name.split("/"):
                param = getattr(param, key)
            diff = param - param.detach()
            term = sens * diff
            if term.dim() > 3:            # (an empty dim tuple would mean "all axes" to torch)
                term = term.sum(dim=tuple(range(3, term.dim())))
            phantom = phantom + term
        return phantom

    def inject_phantom(self, carry, phantom):
        state, *rest = carry
        return (state.detach() + phantom, *rest)

    def initialize_sensitivity(self, key, input_shape):
        return None

    def scan_states(self, z, initial_carry, done):
        """The time scan without the read-out, -> (h, next_carry) as ``Memoroid.scan_fn``
        (memoroid.py:60-91).  Cells whose read-out over every state is fused into the kernel
        (linear attention, delta rule: the per-step states are O(T d^2) and never exist) do not
        offer it."""
        raise NotImplementedError(f"{type(self).__name__} never materialises its per-step states; use scan()")


class Memoroid(SequenceModel):
    def __init__(self, cell: MemoroidCellBase):
        super().__init__()
        self.cell = cell

    def forward(self, inputs, done, initial_carry=None, **kwargs):
        # initial_carry=None means the cell's initialize_carry() value (memoroid.py:101-103);
        # the kernels take that default as NULL pointers, so it is never materialised.
        z = self.cell(inputs, **kwargs)
        next_carry, y = self.cell.scan(z, initial_carry, done, inputs)
        return next_carry, y

    def initialize_carry(self, key, input_shape):
        return self.cell.initialize_carry(key, input_shape)

    def scan_fn(self, z, initial_carry, done):
        """``Memoroid.scan_fn(z, initial_carry, done) -> (h, next_carry)`` (memoroid.py:60-91): every
        prefix of ``[carry, z_1 .. z_T]`` under the cell's operator with the reset rule, and the last one.
        ``h`` is the cell's ``(state, decay)`` pair with the decay leaf ``None``: of that leaf only the
        last step is ever read (memoroid.py:89; every ``read`` ignores it), so the kernels return it in
        ``next_carry`` and never write the (B, T, ...) tensor."""
        return self.cell.scan_states(z, initial_carry, done)

    def propagate_sensitivities(self, decay, jacobians, sensitivity, done):
        """RTRL sensitivities after T steps (``Memoroid._propagate_sensitivities``,
        memoroid.py:114-141): for every parameter leaf, S_t = done_t ? J_t : decay_t S_{t-1} + J_t
        with ``decay`` (B,T,H) broadcast over the leaf's parameter axes, ``jacobians[name]``
        (B,T,H,*param_shape), ``sensitivity[name]`` (B,1,H,*param_shape); returns the dict of
        S_T, shaped like ``sensitivity``.  One last-state-only linear-recurrence launch per leaf -- the reference's
        ``where(done, 0, decay)`` is the kernel's reset rule.  Real or complex (the LRU's); the decay is
        never expanded to the leaf's width when it need not be: a decay that is one (H,) vector broadcast
        over (B,T) (the LRU's lambda, lru.py:118) goes to the kernels as a time-invariant decay, and a
        real decay whose leaf has a multiple of 128 entries per hidden unit takes the grouped-decay kernel."""
        bsz, steps, hid = decay.shape
        cplx = decay.is_complex() or any(t.is_complex() for t in jacobians.values()) or \
            any(t.is_complex() for t in sensitivity.values())
        dt = torch.complex64 if cplx else torch.float32
        broadcast = decay.stride(0) == 0 and decay.stride(1) == 0      # lambda.expand(B, T, H)
        out = {}
        for name in sorted(jacobians.keys()):
            jac, sens = jacobians[name], sensitivity[name]
            param_shape = tuple(jac.shape[3:])
            psize = math.prod(param_shape)
            b_flat = jac.to(dt).reshape(bsz, steps, hid * psize)
            s_flat = sens.to(dt).reshape(bsz, hid * psize)
            # only S_T is returned, so the kernels store nothing per step (one read stream over the Jacobians)
            if broadcast:
                a = decay[0, 0].to(dt).repeat_interleave(psize)
                last = ops.linrec_last(a, b_flat, s_flat, done)
            elif not cplx and ops.grouped_decay_supported(hid * psize, hid):
                # one decay per hidden unit, broadcast over its parameter axes inside the kernel
                last = ops.linrec_grouped_last(decay.float(), b_flat, s_flat, done)
            else:
                a = decay.to(dt).repeat_interleave(psize, dim=-1)
                last = ops.linrec_last(a, b_flat, s_flat, done)
            out[name] = last.reshape(bsz, 1, hid, *param_shape)
        return out

    def local_jacobian(self, inputs, done, carry, sensitivity=None, **kwargs):
        """One RTRL segment (``Memoroid.local_jacobian``, memoroid.py:143-176), -> (next_carry, y,
        next_sensitivity): the carried state re-enters through the phantom term (zero in value, it routes the
        parameters' gradients through the sensitivities), the scan and read-out run as in ``__call__``, and the
        cell's local Jacobians are propagated from ``sensitivity`` over the segment.  ``carry`` must be given
        (the cell's ``initialize_carry`` for a fresh start)."""
        z = self.cell(inputs, **kwargs)
        if sensitivity is not None:
            carry = self.cell.inject_phantom(carry, self.cell.compute_phantom(sensitivity))
        h, next_carry = self.cell.scan_states(z, carry, done)
        y = self.cell.read(h, inputs, **kwargs)
        next_sensitivity = None
        if sensitivity is not None:
            # the state every step starts from: the carry, then h_1 .. h_{T-1}, zero where the step resets
            prev_state = torch.cat([carry[0].to(h[0].dtype), h[0][:, :-1]], dim=1)
            prev_state = torch.where((done != 0)[..., None], torch.zeros_like(prev_state), prev_state)
            local = self.cell.local_jacobian((prev_state, None), z, inputs)
            if local is not None and local[1]:
                next_sensitivity = self.propagate_sensitivities(local[0], local[1], sensitivity, done)
            else:
                next_sensitivity = sensitivity
        return next_carry, y, next_sensitivity

    def initialize_sensitivity(self, key, input_shape):
        return self.cell.initialize_sensitivity(key, input_shape)


# ---------------------------------------------------- complex-diagonal cells
def _project_to_complex(x, w):
    """``x @ w.T`` for real ``x`` (B,T,F) and complex ``w`` (N,F) as ONE real GEMM: the weight rows are
    interleaved (re_0, im_0, re_1, ...), so the (B,T,2N) product is the complex64 result in memory."""
    n, f = w.shape
    w2 = torch.view_as_real(w).permute(0, 2, 1).reshape(2 * n, f)
    out = F.linear(x.float(), w2)
    return torch.view_as_complex(out.view(*out.shape[:-1], n, 2))


def _read_real_part(h, c):
    """``(h @ c.T).real`` for complex ``h`` (B,T,N) and ``c`` (F,N) as ONE real GEMM over the
    interleaved (re, im) view of ``h``: Re(h c) = h_re c_re - h_im c_im."""
    f, n = c.shape
    w2 = torch.stack([c.real, -c.imag], dim=-1).reshape(f, 2 * n)
    hr = torch.view_as_real(h)
    return F.linear(hr.reshape(*hr.shape[:-2], 2 * n), w2)


class _ComplexDiagonalCell(MemoroidCellBase):
    """What the LRU and S5 cells share around the scan kernel (lru.py:78-108, s5.py:123-149):
    the complex projections written as real GEMMs (half the multiply-adds of a complex matmul whose
    imaginary input or output part is discarded, and no complex copy of the inputs) and the scan."""

    def _weights(self):
        """-> (decay (N,), input projection (N,F) complex, read-out (F,N) complex, skip (F,))"""
        raise NotImplementedError

    def forward(self, x, **kwargs):
        lam, w_in, _, _ = self._weights()
        return _project_to_complex(x, w_in), lam

    def read(self, h, x, **kwargs):
        _, _, w_out, skip = self._weights()
        # one pass for the skip term (y + skip * x as a single fused multiply-add over the output)
        return torch.addcmul(_read_real_part(h[0], w_out), x, skip)

    def binary_operator(self, a, b):
        s_i, a_i = a
        s_j, a_j = b
        return a_j * s_i + s_j, a_j * a_i

    def scan_states(self, z, initial_carry, done):
        state, lam = z
        h0, a0 = _squeeze_carry(initial_carry, 2)
        h, a_last = ops.LinRec.apply(lam, state.contiguous(), h0, a0, done)
        return (h, None), (h[:, -1:], a_last[:, None])

    def scan(self, z, initial_carry, done, inputs):
        h, next_carry = self.scan_states(z, initial_carry, done)
        return next_carry, self.read(h, inputs)


# ---------------------------------------------------------------------- LRU
class LRUCell(_ComplexDiagonalCell):
    """Complex diagonal linear recurrence with time-invariant decay (lru.py:32-108)."""

    def __init__(self, features, hidden_dim, r_min=0.0, r_max=1.0, max_phase=6.28):
        super().__init__()
        self.features, self.hidden_dim = features, hidden_dim
        u1, u2 = torch.rand(hidden_dim), torch.rand(hidden_dim)
        self.nu_log = nn.Parameter(torch.log(-0.5 * torch.log(u1 * (r_max ** 2 - r_min ** 2) + r_min ** 2)))
        self.theta_log = nn.Parameter(torch.log(max_phase * u2))
        lam_abs = torch.exp(-torch.exp(self.nu_log.detach()))
        self.gamma_log = nn.Parameter(torch.log(torch.sqrt(1 - lam_abs ** 2)))
        self.B_real = nn.Parameter(torch.randn(hidden_dim, features) / math.sqrt(2 * features))
        self.B_imag = nn.Parameter(torch.randn(hidden_dim, features) / math.sqrt(2 * features))
        self.C_real = nn.Parameter(torch.randn(features, hidden_dim) / math.sqrt(hidden_dim))
        self.C_imag = nn.Parameter(torch.randn(features, hidden_dim) / math.sqrt(hidden_dim))
        self.D = nn.Parameter(torch.randn(features))

    def diag_lambda(self):
        return torch.exp(torch.complex(-torch.exp(self.nu_log), torch.exp(self.theta_log)))

    def _weights(self):
        # the decay is one lambda for every (b, t) (lru.py:86), so it is passed un-broadcast
        b_norm = torch.complex(self.B_real, self.B_imag) * torch.exp(self.gamma_log)[:, None]
        return self.diag_lambda(), b_norm, torch.complex(self.C_real, self.C_imag), self.D

    def local_jacobian(self, carry, z, inputs, **kwargs):
        """-> (decay (B,T,H) as a broadcast view of lambda, {leaf: d state_t / d leaf given state_{t-1}})
        (lru.py:110-125)."""
        prev_state = carry[0]
        state_contrib, _ = z
        lam = self.diag_lambda()
        gamma_exp = torch.exp(self.gamma_log)
        bsz, steps = inputs.shape[:2]
        # gamma (x) u and i gamma (x) u, each written once in the propagation's complex dtype (a real product, its
        # complex copy and the multiplication by i would be three passes over the (B,T,H,F) tensors)
        g_c = gamma_exp.to(torch.complex64)[None, None, :, None]
        u_c = inputs.float().to(torch.complex64)[:, :, None, :]
        return lam.expand(bsz, steps, self.hidden_dim), {
            "nu_log": -torch.exp(self.nu_log) * lam * prev_state,
            "theta_log": 1j * torch.exp(self.theta_log) * lam * prev_state,
            "gamma_log": state_contrib,
            "B_real": g_c * u_c,
            "B_imag": (1j * g_c) * u_c,
        }

    def initialize_sensitivity(self, key, input_shape):
        *batch, _ = input_shape
        dev = self.nu_log.device
        z = lambda *shape: torch.zeros(*batch, 1, *shape, dtype=torch.complex64, device=dev)
        h = self.hidden_dim
        return {"nu_log": z(h), "theta_log": z(h), "gamma_log": z(h), "B_real": z(h, self.features),
                "B_imag": z(h, self.features)}

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.zeros(*batch, 1, self.hidden_dim, dtype=torch.complex64),
                torch.ones(*batch, 1, self.hidden_dim, dtype=torch.complex64))


# ------------------------------------------------------------------- MinGRU
class MinGRUPreactivations(tuple):
    """(z, h_tilde): what ``MinGRUCell`` hands its fused scan instead of the (log_state, decay) elements."""


class MinGRUCell(MemoroidCellBase):
    """Log-space minimal GRU (min_gru.py:14-90).  With ``fused_gates`` (default) the gate math of
    min_gru.py:52-61 runs inside the scan kernels: ``forward`` returns the two Dense pre-activations and the
    (B,T,F) log_state / decay tensors are never written; ``elements(x)`` gives the reference's elements."""

    def __init__(self, features, in_features=None, fused_gates=True):
        super().__init__()
        self.features, self.fused_gates = features, fused_gates
        in_features = in_features or features
        self.z = nn.Linear(in_features, features, bias=False)
        self.h = nn.Linear(in_features, features, bias=False)

    def forward(self, x, **kwargs):
        if self.fused_gates:
            return MinGRUPreactivations((self.z(x), self.h(x)))
        return self.elements(x)

    def elements(self, x):
        z, h_tilde = self.z(x), self.h(x)
        log_z = -torch.nn.functional.softplus(-z)
        log_h = torch.where(h_tilde >= 0, torch.log(torch.relu(h_tilde) + 0.5),
                            -torch.nn.functional.softplus(-h_tilde))
        return log_z + log_h, -torch.nn.functional.softplus(z)

    def binary_operator(self, a, b):
        x_i, d_i = a
        x_j, d_j = b
        return torch.logaddexp(d_j + x_i, x_j), d_i + d_j

    def read(self, h, x, **kwargs):
        return torch.exp(h[0])

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.full((*batch, 1, self.features), -float("inf")), torch.zeros(*batch, 1, self.features))

    def scan_states(self, z, initial_carry, done):
        log_state, decay = z
        x0, a0 = _squeeze_carry(initial_carry, 2)
        x, _, a_last = ops.LogLinRec.apply(log_state.contiguous(), decay.contiguous(), x0, a0, done)
        return (x, None), (x[:, -1:], a_last[:, None])

    def scan(self, z, initial_carry, done, inputs):
        x0, a0 = _squeeze_carry(initial_carry, 2)
        if isinstance(z, MinGRUPreactivations):
            x, y, a_last = ops.MinGRUFused.apply(z[0].contiguous(), z[1].contiguous(), x0, a0, done)
        else:
            log_state, decay = z
            x, y, a_last = ops.LogLinRec.apply(log_state.contiguous(), decay.contiguous(), x0, a0, done)
        return (x[:, -1:], a_last[:, None]), y


# --------------------------------------------------------- linear attention
class LinearAttentionCell(MemoroidCellBase):
    """ELU+1 linear attention (linear_attention.py:14-124).  ``head_dim``: a multiple of 8, at most 64."""

    def __init__(self, features, head_dim, num_heads, eps=1e-6, in_features=None):
        super().__init__()
        self.features, self.head_dim, self.num_heads, self.eps = features, head_dim, num_heads, eps
        in_features = in_features or features
        hidden = num_heads * head_dim
        self.key = nn.Linear(in_features, hidden, bias=False)
        self.value = nn.Linear(in_features, hidden, bias=False)
        self.query = nn.Linear(in_features, hidden, bias=False)
        self.norm = nn.RMSNorm(hidden, eps=1e-6)   # flax.linen.RMSNorm's default epsilon
        self.output_projection = nn.Linear(hidden, features)

    def _heads(self, t):
        return t.view(*t.shape[:2], self.num_heads, self.head_dim)

    def forward(self, x, **kwargs):
        """-> factored elements (k, v) with k, v (B,T,H,hd): S_t = v_t (x) phi(k_t)
        and z_t = phi(k_t) (linear_attention.py:75-80) are never materialised;
        the feature map is applied inside the kernel."""
        return self._heads(self.key(x)), self._heads(self.value(x))

    def binary_operator(self, a, b):
        return tuple(p + q for p, q in zip(a, b))

    def read(self, h, x, **kwargs):
        raise RuntimeError("the read-out over every S_t is fused into scan(); see the module docstring")

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.zeros(*batch, 1, self.num_heads, self.head_dim, self.head_dim),
                torch.zeros(*batch, 1, self.num_heads, self.head_dim))

    def scan(self, z, initial_carry, done, inputs):
        k, v = z
        q = self._heads(self.query(inputs))
        s0, z0 = _squeeze_carry(initial_carry, 2)
        bf = torch.bfloat16
        o, s_last, z_last = ops.LinAttn.apply(q.to(bf), k.to(bf), v.to(bf), s0, z0, done, self.eps, True)
        o = o.reshape(*o.shape[:2], -1).to(inputs.dtype)
        y = ops.dense(self.norm(o), self.output_projection.weight, self.output_projection.bias)
        return (s_last[:, None], z_last[:, None]), y


# ------------------------------------------------------- gated delta rule
class DeltaNetCell(MemoroidCellBase):
    """Gated delta-rule mixer.  The reference has no such cell; this one follows
    its cell protocol.  As a monoid the element is
    ``(alpha (I - beta k k^T), beta v k^T)`` with operator
    ``((M_i, U_i), (M_j, U_j)) -> (M_i M_j, U_i M_j + U_j)``; the carry keeps
    only the state ``S (B,1,H,d_v,d_k)`` (the map leaf is O(d_k^2) per step and
    no read-out uses it).  ``head_dim`` is 128 or 64 (a 64-wide head runs on the
    128-wide kernels with the upper half of every tile zero-filled by the tensor maps)."""

    def __init__(self, features, head_dim, num_heads, in_features=None):
        super().__init__()
        self.features, self.head_dim, self.num_heads = features, head_dim, num_heads
        in_features = in_features or features
        hidden = num_heads * head_dim
        self.query = nn.Linear(in_features, hidden, bias=False)
        self.key = nn.Linear(in_features, hidden, bias=False)
        self.value = nn.Linear(in_features, hidden, bias=False)
        self.gate = nn.Linear(in_features, 2 * num_heads)   # -> (beta logits, decay logits)
        self.norm = nn.RMSNorm(hidden, eps=1e-6)   # flax.linen.RMSNorm's default epsilon
        self.output_projection = nn.Linear(hidden, features)

    def _heads(self, t):
        return t.view(*t.shape[:2], self.num_heads, self.head_dim)

    def forward(self, x, **kwargs):
        """-> factored elements (k, v, alpha, beta); k is L2-normalised per head."""
        k = ops.l2norm_heads(self.key(x), self.head_dim)
        v = self._heads(self.value(x))
        b_logit, a_logit = ops.dense(x, self.gate.weight, self.gate.bias).float().chunk(2, dim=-1)
        return k, v, torch.exp(-torch.nn.functional.softplus(a_logit)), torch.sigmoid(b_logit)

    def binary_operator(self, a, b):
        m_i, u_i = a
        m_j, u_j = b
        return m_i @ m_j, u_i @ m_j + u_j

    def read(self, h, x, **kwargs):
        raise RuntimeError("the read-out o_t = S_t q_t is fused into scan()")

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.zeros(*batch, 1, self.num_heads, self.head_dim, self.head_dim),)

    def scan(self, z, initial_carry, done, inputs):
        k, v, alpha, beta = z
        q = ops.l2norm_heads(self.query(inputs), self.head_dim)
        (s0,) = _squeeze_carry(initial_carry, 1)
        bf = torch.bfloat16
        o, s_last = ops.GatedDelta.apply(q.to(bf), k.to(bf), v.to(bf), alpha.contiguous(), beta.contiguous(), s0, done)
        o = o.reshape(*o.shape[:2], -1).to(inputs.dtype)
        return (s_last[:, None],), ops.dense(ops.rms_norm(o, self.norm.weight, self.norm.eps), self.output_projection.weight,
                                          self.output_projection.bias)


# -------------------------------------------------------------------- mLSTM
class mLSTMCell(MemoroidCellBase):
    """Matrix-memory LSTM (mlstm.py:31-240): gated linear attention with a per-head scalar forget gate and
    the running-max stabiliser.  Projections as the reference (up-projection, causal depthwise convolution +
    SiLU, block-diagonal q / k / v, Dense gates on [q, k, v], head-wise LayerNorm with residual scale,
    learnable skip, SiLU(z) gate, output projection); the element ``(k (x) v, log_f, k, m = log_i)`` of
    mlstm.py:198-203 stays factored as ``(k, v, log_i, log_f)`` -- the (B,T,H,d,d) outer products and the
    per-step memories never exist -- and scan + read-out are one kernel.  ``head_dim`` = hidden_dim /
    num_heads must be 32, 64 or 128 for the float32 kernels (the reference's arithmetic).  With
    ``tensor_cores=True`` the scan runs in chunked form on the tensor cores instead: q, k, v and the read-out in
    bf16, gates and state in fp32 (the numerical class of the linear-attention kernels), head_dim a multiple of 8
    up to 64, about ten times the throughput."""

    def __init__(self, features, hidden_dim, num_heads=4, conv_kernel_size=4, in_features=None, eps=1e-6,
                 tensor_cores=False):
        super().__init__()
        self.tensor_cores = tensor_cores
        if hidden_dim % num_heads:
            raise ValueError(f"hidden_dim ({hidden_dim}) must be divisible by num_heads ({num_heads}).")
        self.features, self.hidden_dim, self.num_heads, self.eps = features, hidden_dim, num_heads, eps
        self.head_dim = hidden_dim // num_heads
        fin = in_features or features
        self.up_projection = nn.Linear(fin, 2 * hidden_dim, bias=False)
        self.causal_conv = nn.Conv1d(hidden_dim, hidden_dim, conv_kernel_size, groups=hidden_dim,
                                     padding=conv_kernel_size - 1)
        block = lambda: nn.Parameter(torch.randn(num_heads, self.head_dim, self.head_dim) / math.sqrt(self.head_dim))
        self.query, self.key, self.value = block(), block(), block()     # BlockDiagonalDense kernels [h][out][in]
        self.i_gate = nn.Linear(3 * hidden_dim, num_heads)
        self.f_gate = nn.Linear(3 * hidden_dim, num_heads)
        with torch.no_grad():      # mlstm.py:110-125: zero kernels, bias N(0, 0.1) / linspace(3, 6)
            self.i_gate.weight.zero_(); self.f_gate.weight.zero_()
            self.i_gate.bias.normal_(std=0.1)
            self.f_gate.bias.copy_(torch.linspace(3.0, 6.0, num_heads))
        self.learnable_skip = nn.Parameter(torch.ones(hidden_dim))
        self.norm_weight = nn.Parameter(torch.zeros(num_heads, self.head_dim))   # MultiHeadLayerNorm: scale = 1 + weight
        self.output_projection = nn.Linear(hidden_dim, features, bias=False)

    def _block(self, x, kernel):
        bsz, steps, _ = x.shape
        return torch.einsum("bthd,hod->btho", x.view(bsz, steps, self.num_heads, self.head_dim), kernel)

    def _project(self, x):
        steps = x.shape[1]
        x_mlstm, z = self.up_projection(x).chunk(2, dim=-1)
        u = torch.nn.functional.silu(self.causal_conv(x_mlstm.transpose(1, 2))[..., :steps].transpose(1, 2))
        return self._block(u, self.query), self._block(u, self.key), self._block(x_mlstm, self.value), z, u

    def forward(self, x, **kwargs):
        """-> factored elements (k / sqrt(d), v, log_i, log_f) plus what the read-out needs."""
        q, k, v, z, u = self._project(x)
        gate_in = torch.cat([q, k, v], dim=-1).reshape(*x.shape[:2], -1)
        log_i = self.i_gate(gate_in)
        log_f = -torch.nn.functional.softplus(-self.f_gate(gate_in))
        return k / math.sqrt(self.head_dim), v, log_i, log_f, (q, z, u)

    def binary_operator(self, a, b):
        c_a, f_a, n_a, m_a = a
        c_b, f_b, n_b, m_b = b
        m_dec = m_a + f_b
        m_new = torch.maximum(m_dec, m_b)
        s_a, s_b = torch.exp(m_dec - m_new), torch.exp(m_b - m_new)
        return s_a * c_a + s_b * c_b, f_a + f_b, s_a * n_a + s_b * n_b, m_new

    def read(self, h, x, **kwargs):
        raise RuntimeError("the read-out over every C_t is fused into scan()")

    def finish(self, h_tilde, z, u):
        """Everything of ``read`` after the memory read-out (mlstm.py:220-229)."""
        bsz, steps = h_tilde.shape[:2]
        y = torch.nn.functional.layer_norm(h_tilde, (self.head_dim,), eps=1e-5) * (1.0 + self.norm_weight)
        y = y.reshape(bsz, steps, self.hidden_dim) + self.learnable_skip * u
        return self.output_projection(y * torch.nn.functional.silu(z))

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        hd = self.head_dim
        return (torch.zeros(*batch, 1, self.num_heads, hd, hd), torch.zeros(*batch, 1, self.num_heads, 1, 1),
                torch.zeros(*batch, 1, self.num_heads, hd, 1), torch.full((*batch, 1, self.num_heads, 1, 1), -1e9))

    def scan(self, z, initial_carry, done, inputs):
        k, v, log_i, log_f, (q, zgate, u) = z
        c0 = f0 = n0 = m0 = None
        if initial_carry is not None:
            c0, f0, n0, m0 = initial_carry
            c0, f0 = c0[:, 0].contiguous(), f0[:, 0, :, 0, 0].contiguous()
            n0, m0 = n0[:, 0, :, :, 0].contiguous(), m0[:, 0, :, 0, 0].contiguous()
        if self.tensor_cores:
            bf = lambda t: t.to(torch.bfloat16).contiguous()
            h, c_last, n_last, m_last, f_last = ops.MLSTMTensorCore.apply(bf(q), bf(k), bf(v), log_i.float().contiguous(),
                                                                          log_f.float().contiguous(), c0, n0, m0, f0, done,
                                                                          self.eps)
        else:
            h, c_last, n_last, m_last, f_last = ops.MLSTM.apply(q.float().contiguous(), k.float().contiguous(),
                                                                v.float().contiguous(), log_i.float().contiguous(),
                                                                log_f.float().contiguous(), c0, n0, m0, f0, done, self.eps)
        next_carry = (c_last[:, None], f_last[:, None, :, None, None], n_last[:, None, :, :, None],
                      m_last[:, None, :, None, None])
        return next_carry, self.finish(h.to(inputs.dtype), zgate, u)


# ----------------------------------------------------------------------- S5
def make_dplr_hippo(n):
    """HiPPO-LegS in diagonal-plus-low-rank form (hippo.py:6-32): eigenvalues ``lambda`` (n,) and eigenvectors
    ``v`` (n,n) of the normal part S = A + p p^T of the HiPPO matrix (real part: the mean of S's diagonal,
    -1/2; imaginary parts: the eigenvalues of the Hermitian -i S).  Initialisation-time host arithmetic in
    float64, returned as complex128 tensors."""
    idx = torch.arange(n, dtype=torch.float64)
    q = torch.sqrt(1.0 + 2.0 * idx)
    a = -(torch.tril(q[:, None] * q[None, :]) - torch.diag(idx))
    p = torch.sqrt(idx + 0.5)
    s_mat = a + p[:, None] * p[None, :]
    lambda_real = torch.diagonal(s_mat).mean() * torch.ones(n, dtype=torch.float64)
    lambda_imag, v = torch.linalg.eigh(s_mat.to(torch.complex128) * (-1j))
    return torch.complex(lambda_real, lambda_imag), v


class S5Cell(_ComplexDiagonalCell):
    """Diagonal state-space cell (s5.py:29-149): the same (state, decay) operator as the LRU with a discretised,
    time-invariant ``lambda_bar`` (ZOH or bilinear, hippo.py:34-50).  Initialised as the reference's ``setup``:
    ``lambda`` from the HiPPO-DPLR eigenvalues, ``B`` a lecun-normal matrix taken into the eigenbasis
    (``V^H B``, initializers/hippo.py:19-26), ``C`` a lecun-normal complex matrix times ``V``
    (initializers/hippo.py:29-37), ``log_step`` uniform in [log dt_min, log dt_max]."""

    def __init__(self, features, state_size, discretization="zoh", dt_min=0.001, dt_max=0.1, step_rescale=1.0,
                 clip_eigens=False):
        super().__init__()
        self.features, self.state_size = features, state_size
        self.discretization, self.step_rescale, self.clip_eigens = discretization, step_rescale, clip_eigens
        lam, v = make_dplr_hippo(state_size)
        self.lambda_real = nn.Parameter(lam.real.float())
        self.lambda_imag = nn.Parameter(lam.imag.float())
        b = torch.randn(state_size, features, dtype=torch.float64) / math.sqrt(features)          # lecun normal
        self.B = nn.Parameter(torch.view_as_real(v.conj().t() @ b.to(torch.complex128)).float())
        c = torch.view_as_complex(torch.randn(features, state_size, 2, dtype=torch.float64) / math.sqrt(state_size))
        self.C = nn.Parameter(torch.view_as_real(c @ v).float())
        self.d = nn.Parameter(torch.randn(features))
        u = torch.rand(state_size, 1)
        self.log_step = nn.Parameter(u * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))

    def _discretized(self):
        lam_re = torch.clamp(self.lambda_real, max=-1e-4) if self.clip_eigens else self.lambda_real
        lam = torch.complex(lam_re, self.lambda_imag)
        b_tilde = torch.view_as_complex(self.B.contiguous())
        step = (self.step_rescale * torch.exp(self.log_step[:, 0])).to(torch.complex64)
        if self.discretization == "zoh":
            lambda_bar = torch.exp(lam * step)
            b_bar = ((lambda_bar - 1.0) / lam)[:, None] * b_tilde
        elif self.discretization == "bilinear":
            bl = 1.0 / (1.0 - step / 2.0 * lam)
            lambda_bar = bl * (1.0 + step / 2.0 * lam)
            b_bar = (bl * step)[:, None] * b_tilde
        else:
            raise ValueError(f"Invalid discretization: {self.discretization}")
        return lambda_bar, b_bar

    def _weights(self):
        lambda_bar, b_bar = self._discretized()
        return lambda_bar, b_bar, torch.view_as_complex(self.C.contiguous()), self.d

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.zeros(*batch, 1, self.state_size, dtype=torch.complex64),
                torch.ones(*batch, 1, self.state_size, dtype=torch.complex64))


# -------------------------------------------------------------------- Mamba
class MambaCell(MemoroidCellBase):
    """Selective state-space cell (mamba.py:33-150): per head a (state_dim x head_dim) matrix
    state with one scalar decay per (b, t, head).  Elements and read-out follow the
    reference -- ``h_t = (dt B_t) (x) x_t`` (mamba.py:109-117), operator
    ``(decay_j h_i + h_j, decay_j decay_i)`` (:119-122), ``y = C . h + D x`` gated by
    ``silu(z)`` after an RMSNorm (:124-135) -- and, like the reference, the scan runs over the
    materialised (B, T, H, N, P) elements: here as ONE real linear-recurrence launch over
    H*N*P channels instead of ~2 log2(T) passes.  When a head's N*P state elements are a multiple of
    128 (the default 16 x 16 is) the kernels read the per-head decay (B,T,H) directly and reduce its
    gradient per head (``ops.LinRecGrouped``); otherwise the decay is expanded (``ops.LinRec``)."""

    def __init__(self, features, num_heads=8, head_dim=16, state_dim=16, conv_dim=4, in_features=None):
        super().__init__()
        self.features, self.num_heads, self.head_dim, self.state_dim = features, num_heads, head_dim, state_dim
        self.conv_dim = conv_dim
        fin = in_features or features
        hidden, sproj = num_heads * head_dim, num_heads * state_dim
        self.A_log = nn.Parameter(torch.log(torch.empty(num_heads).uniform_(1.0, 16.0)))
        self.D = nn.Parameter(torch.ones(num_heads))
        dt0 = torch.exp(torch.rand(num_heads) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        self.dt_bias = nn.Parameter(dt0 + torch.log(-torch.expm1(-dt0)))
        self.input_projection = nn.Linear(fin, 2 * hidden, bias=False)
        self.B = nn.Linear(fin, sproj, bias=False)
        self.C = nn.Linear(fin, sproj, bias=False)
        self.dt = nn.Linear(fin, num_heads, bias=False)
        channels = hidden + 2 * sproj
        self.conv = nn.Conv1d(channels, channels, conv_dim, groups=channels, padding=conv_dim - 1)
        self.norm = nn.RMSNorm(hidden, eps=1e-6)   # flax.linen.RMSNorm's default epsilon
        self.output_projection = nn.Linear(hidden, features)

    def _project(self, x):
        bsz, steps, _ = x.shape
        hidden_dim, sproj = self.num_heads * self.head_dim, self.num_heads * self.state_dim
        hidden, gate = self.input_projection(x).chunk(2, dim=-1)
        conv_in = torch.cat([hidden, self.B(x), self.C(x)], dim=-1).transpose(1, 2)
        conv = torch.nn.functional.silu(self.conv(conv_in)[..., :steps]).transpose(1, 2)   # causal (left padding)
        hidden = conv[..., :hidden_dim].reshape(bsz, steps, self.num_heads, self.head_dim)
        b_proj = conv[..., hidden_dim:hidden_dim + sproj].reshape(bsz, steps, self.num_heads, self.state_dim)
        c_proj = conv[..., hidden_dim + sproj:].reshape(bsz, steps, self.num_heads, self.state_dim)
        dt = torch.nn.functional.softplus(self.dt(x) + self.dt_bias)
        return hidden, b_proj, c_proj, gate, dt

    def forward(self, x, **kwargs):
        """-> (h (B,T,H,N,P), decay (B,T,H,1,1)) as mamba.py:109-117, plus what ``read`` needs."""
        hidden, b_proj, c_proj, gate, dt = self._project(x)
        decay = torch.exp(dt * -torch.exp(self.A_log))[..., None, None]
        h = torch.einsum("bthn,bthd->bthnd", b_proj * dt[..., None], hidden)
        return h, decay, (hidden, c_proj, gate)

    def binary_operator(self, a, b):
        h_i, d_i = a
        h_j, d_j = b
        return d_j * h_i + h_j, d_j * d_i

    def read_state(self, h, hidden, c_proj):
        """The read-out in front of the norm and the gate: ``C . h + D x`` (mamba.py:130-131)."""
        return torch.einsum("bthn,bthnd->bthd", c_proj, h) + self.D[None, None, :, None] * hidden

    def read(self, h, x, projected=None, **kwargs):
        state, _ = h
        hidden, c_proj, gate = projected if projected is not None else self.forward(x)[2]
        bsz, steps = state.shape[:2]
        y = self.read_state(state, hidden, c_proj).reshape(bsz, steps, self.num_heads * self.head_dim)
        return self.output_projection(self.norm(y) * torch.nn.functional.silu(gate))

    def initialize_carry(self, key, input_shape):
        *batch, _ = input_shape
        return (torch.zeros(*batch, 1, self.num_heads, self.state_dim, self.head_dim),
                torch.ones(*batch, 1, self.num_heads, 1, 1))

    def scan_elements(self, h_elems, decay, initial_carry, done):
        """The time scan alone: elements (B,T,H,N,P), decay (B,T,H,1,1), carry as
        ``initialize_carry`` -> (h (B,T,H,N,P), next_carry)."""
        bsz, steps, heads, sdim, hdim = h_elems.shape
        width = heads * sdim * hdim
        if ops.grouped_decay_supported(width, heads):
            # one decay per head, read as such by the kernel: the (B,T,H) tensor is never expanded
            h0 = a0 = None
            if initial_carry is not None:
                h0 = initial_carry[0].reshape(bsz, width).contiguous()
                a0 = initial_carry[1].reshape(bsz, heads).contiguous()
            h, a_last = ops.LinRecGrouped.apply(decay.reshape(bsz, steps, heads).contiguous(),
                                                h_elems.reshape(bsz, steps, width).contiguous(), h0, a0, done)
            h = h.reshape(bsz, steps, heads, sdim, hdim)
            return h, (h[:, -1:], a_last.reshape(bsz, 1, heads, 1, 1))
        a = decay.expand(bsz, steps, heads, sdim, hdim).reshape(bsz, steps, width).contiguous()
        h0 = a0 = None
        if initial_carry is not None:
            h0 = initial_carry[0].reshape(bsz, width).contiguous()
            a0 = initial_carry[1].expand(bsz, 1, heads, sdim, hdim).reshape(bsz, width).contiguous()
        h, a_last = ops.LinRec.apply(a, h_elems.reshape(bsz, steps, width).contiguous(), h0, a0, done)
        h = h.reshape(bsz, steps, heads, sdim, hdim)
        return h, (h[:, -1:], a_last.reshape(bsz, 1, heads, sdim, hdim)[..., :1, :1])

    def scan_states(self, z, initial_carry, done):
        h_elems, decay = z[0], z[1]
        h, next_carry = self.scan_elements(h_elems, decay, initial_carry, done)
        return (h, None), next_carry

    def scan(self, z, initial_carry, done, inputs):
        h_elems, decay, projected = z
        h, next_carry = self.scan_elements(h_elems, decay, initial_carry, done)
        return next_carry, self.read((h, None), inputs, projected=projected)
