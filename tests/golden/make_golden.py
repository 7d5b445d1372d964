"""Generate tests/golden/memoroid_golden.npz by executing the reference's own
source files for the sequence-mixing path.

The reference (memorax 1.0.1) is pure Python on top of JAX/Flax, neither of
which can be installed in the build image.  This script therefore loads the
reference's files *unmodified* from a checkout (``--reference DIR``; nothing is
copied) under a minimal NumPy stand-in for the JAX/Flax symbols those files
touch: ``jax.numpy`` is NumPy, ``jax.vmap`` maps over axis 0 with a Python
loop, ``jax.tree.map`` maps over tuples, ``flax.linen.Module`` is a plain
attribute bag, and ``jax.lax.associative_scan`` is a left-to-right fold (any
bracketing of an associative operator gives the same prefix).  Everything is
evaluated in float64, so the vectors pin the reference's *semantics* --
operators, reset rule, carry layout, read-outs -- not XLA's rounding.

Files executed: memorax/utils/axes.py,
memorax/networks/sequence_models/{sequence_model,memoroid,lru,min_gru,
linear_attention,mamba,mlstm}.py.

Run (only where the reference checkout exists):
    python tests/golden/make_golden.py --reference /path/to/memorax
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys
import types
import zlib

import numpy as np

F64 = np.float64


# ----------------------------------------------------------------------------
# stand-ins
# ----------------------------------------------------------------------------
def _tree_map(fn, *trees):
    first = trees[0]
    if isinstance(first, (tuple, list)):
        return tuple(_tree_map(fn, *parts) for parts in zip(*trees))
    if isinstance(first, dict):
        return {k: _tree_map(fn, *(t[k] for t in trees)) for k in first}
    return fn(*trees)


def _vmap(fn):
    def mapped(*args):
        n = None

        def probe(x):
            nonlocal n
            n = x.shape[0]
            return x

        _tree_map(probe, args)
        outs = [fn(*_tree_map(lambda x: x[i], args)) for i in range(n)]
        return _tree_map(lambda *xs: np.stack(xs, axis=0), *outs)

    return mapped


def _fold_scan(fn, elems, axis=0):
    take = lambda x, t: np.take(x, [t], axis=axis)
    n = None

    def probe(x):
        nonlocal n
        n = x.shape[axis]
        return x

    _tree_map(probe, elems)
    acc = _tree_map(lambda x: take(x, 0), elems)
    outs = [acc]
    for t in range(1, n):
        acc = fn(acc, _tree_map(lambda x: take(x, t), elems))
        outs.append(acc)
    return _tree_map(lambda *xs: np.concatenate(xs, axis=axis), *outs)


def _softplus(x):
    return np.logaddexp(x, 0.0)


class _Module:
    """Attribute bag with the few Flax hooks the reference's cells call."""

    def __init__(self, **fields):
        for name, value in fields.items():
            setattr(self, name, value)
        self._params = {}
        if hasattr(self, "setup"):
            self.setup()

    def param(self, name, init_fn, *args):
        rng = np.random.default_rng(zlib.crc32(name.encode()))
        shape = next((a for a in args if isinstance(a, tuple) and all(isinstance(i, int) for i in a)), None)
        if shape is None:  # gamma_log style: derived from other params
            value = init_fn(None, *args)
        else:
            value = rng.normal(size=shape).astype(F64) * 0.5
        self._params[name] = value
        return value

    def sow(self, *a, **k):
        return None

    @property
    def variables(self):
        return {"params": self._params}


class _Dense(_Module):
    """Bias-free projection with lazily drawn float64 weights."""

    def __init__(self, features=None, name="dense", **_):
        self.features = features if isinstance(features, tuple) else (features,)
        self.name = name
        self.kernel = None

    def __call__(self, x):
        if self.kernel is None:
            rng = np.random.default_rng(zlib.crc32(self.name.encode()))
            self.kernel = rng.normal(size=(x.shape[-1],) + self.features).astype(F64) / np.sqrt(x.shape[-1])
        return np.tensordot(x, self.kernel, axes=([-1], [0]))


class _Identity(_Module):
    def __init__(self, *a, **k):
        pass

    def __call__(self, x):
        return x


def install_stand_ins(reference_dir):
    jnp = types.ModuleType("jax.numpy")
    jnp.__dict__.update({k: getattr(np, k) for k in dir(np) if not k.startswith("_")})
    is_cplx = lambda dtype: dtype in (np.complex64, np.complex128)
    jnp.zeros = lambda shape, dtype=None: np.zeros(shape, dtype=np.complex128 if is_cplx(dtype) else F64)
    jnp.ones = lambda shape, dtype=None: np.ones(shape, dtype=np.complex128 if is_cplx(dtype) else F64)
    # everything runs in double precision: the reference's float32 / complex64 casts keep the value
    jnp.float32, jnp.complex64 = np.float64, np.complex128
    jnp.full = lambda shape, v, dtype=None: np.full(shape, v, dtype=F64)

    lax = types.ModuleType("jax.lax")
    lax.associative_scan = _fold_scan
    lax.complex = lambda re, im: re + 1j * im
    lax.stop_gradient = lambda x: x

    tree = types.ModuleType("jax.tree")
    tree.map = _tree_map

    rnd = types.ModuleType("jax.random")
    rnd.key = lambda seed: seed

    jnn = types.ModuleType("jax.nn")
    jnn.softplus = _softplus
    jnn_inits = types.ModuleType("jax.nn.initializers")       # names s5.py imports; used only in setup()
    jnn_inits.lecun_normal = jnn_inits.normal = lambda *a, **k: None
    jnn.initializers = jnn_inits

    jax = types.ModuleType("jax")
    jax.numpy, jax.lax, jax.tree, jax.random, jax.nn = jnp, lax, tree, rnd, jnn
    jax.vmap = _vmap
    jax.Array = np.ndarray

    nn = types.ModuleType("flax.linen")
    nn.Module = _Module
    nn.compact = lambda f: f
    nn.elu = lambda x: np.where(x > 0, x, np.expm1(np.minimum(x, 0)))
    nn.relu = lambda x: np.maximum(x, 0)
    nn.softplus = _softplus
    nn.silu = lambda x: x / (1.0 + np.exp(-x))
    nn.Dense = _Dense
    nn.DenseGeneral = _Dense
    nn.RMSNorm = _Identity
    inits = types.ModuleType("flax.linen.initializers")
    inits.lecun_normal = lambda *a, **k: None
    inits.zeros_init = lambda *a, **k: None
    inits.ones = lambda *a, **k: None
    inits.normal = lambda *a, **k: None
    nn.initializers = inits
    nn.Conv = nn.Dropout = _Identity
    flax = types.ModuleType("flax")
    flax.linen = nn
    ftyping = types.ModuleType("flax.typing")
    ftyping.Dtype = ftyping.Initializer = object

    mods = {"jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.tree": tree, "jax.random": rnd, "jax.nn": jnn,
            "jax.nn.initializers": jnn_inits,
            "flax": flax, "flax.linen": nn, "flax.linen.initializers": inits, "flax.typing": ftyping}
    # layers / initialisers that mlstm.py imports by name but only uses in setup(), which is bypassed
    net_inits = types.ModuleType("memorax.networks.initializers")
    net_inits.wang = lambda *a, **k: None
    net_inits.init_cv = net_inits.init_v_inv_b = net_inits.log_step = net_inits.truncated_standard_normal = \
        lambda *a, **k: None
    net_layers = types.ModuleType("memorax.networks.layers")
    net_layers.BlockDiagonalDense = net_layers.MultiHeadLayerNorm = _Identity
    mods["memorax.networks.initializers"], mods["memorax.networks.layers"] = net_inits, net_layers

    # Bare packages whose __path__ points into the checkout, so that the
    # reference's modules import each other without running the package
    # __init__ files (which pull in the whole library).
    root = os.path.join(reference_dir, "memorax")
    for name, rel in [("memorax", ""), ("memorax.utils", "utils"), ("memorax.networks", "networks"),
                      ("memorax.networks.sequence_models", "networks/sequence_models")]:
        pkg = types.ModuleType(name)
        pkg.__path__ = [os.path.join(root, rel)]
        mods[name] = pkg
    typing_stub = types.ModuleType("memorax.utils.typing")
    typing_stub.Array = typing_stub.Carry = typing_stub.Key = object
    mods["memorax.utils.typing"] = typing_stub
    sys.modules.update(mods)


# ----------------------------------------------------------------------------
# cases
# ----------------------------------------------------------------------------
def done_patterns(rng, bsz, steps):
    done = (rng.random((bsz, steps)) < 0.25).astype(F64)
    done[0, 0] = 1.0                      # reset at the very first step
    if steps > 4:
        done[1, 2:4] = 1.0                # consecutive resets
        done[-1, :] = 0.0                 # a row with no reset at all
    return done


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a memorax 1.0.1 checkout")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "memoroid_golden.npz"))
    args = ap.parse_args()
    install_stand_ins(args.reference)

    sm = "memorax.networks.sequence_models."
    memoroid = importlib.import_module(sm + "memoroid")
    lru = importlib.import_module(sm + "lru")
    min_gru = importlib.import_module(sm + "min_gru")
    linattn = importlib.import_module(sm + "linear_attention")

    rng = np.random.default_rng(20240611)
    out = {}

    # ---- LRU (complex diagonal, time-invariant decay) through Memoroid ----
    bsz, steps, feat, hid = 3, 9, 5, 4
    cell = lru.LRUCell(features=feat, hidden_dim=hid)
    # keep |lambda| < 1 and the phase moderate
    cell.nu_log = np.log(rng.uniform(0.05, 0.6, hid))
    cell.theta_log = np.log(rng.uniform(0.05, 0.6, hid))
    model = memoroid.Memoroid(cell=cell)
    x = rng.normal(size=(bsz, steps, feat))
    done = done_patterns(rng, bsz, steps)
    carry = (rng.normal(size=(bsz, 1, hid)) + 1j * rng.normal(size=(bsz, 1, hid)),
             rng.normal(size=(bsz, 1, hid)) * 0.3 + 1j * rng.normal(size=(bsz, 1, hid)) * 0.3)
    z = cell(x)
    h, nxt = model.scan_fn(z, carry, done)
    nxt2, y = model(x, done, carry)
    assert all(np.array_equal(p, q) for p, q in zip(nxt, nxt2))
    out.update(lru_x=x, lru_done=done, lru_c_state=carry[0], lru_c_decay=carry[1],
               lru_z_state=z[0], lru_z_decay=z[1], lru_h_state=h[0], lru_h_decay=h[1],
               lru_n_state=nxt[0], lru_n_decay=nxt[1], lru_y=y,
               lru_C=cell.C_real + 1j * cell.C_imag, lru_D=cell.D)
    # default carry (initialize_carry) path
    nxt0, y0 = model(x, done, None)
    out.update(lru_default_n_state=nxt0[0], lru_default_n_decay=nxt0[1], lru_default_y=y0)

    # ---- MinGRU (log space, -inf initial carry) --------------------------
    bsz, steps, feat = 3, 8, 6
    cell = min_gru.MinGRUCell(features=feat)
    cell.dtype, cell.param_dtype = None, F64
    model = memoroid.Memoroid(cell=cell)
    x = rng.normal(size=(bsz, steps, 4)) * 2.0
    done = done_patterns(rng, bsz, steps)
    z = cell(x)
    carry0 = cell.initialize_carry(0, (bsz, feat))
    assert np.all(np.isneginf(carry0[0]))
    with np.errstate(invalid="ignore"):
        h, nxt = model.scan_fn(z, carry0, done)
        _, y = model(x, done, None)
    carry1 = (rng.normal(size=(bsz, 1, feat)), -np.abs(rng.normal(size=(bsz, 1, feat))))
    h1, nxt1 = model.scan_fn(z, carry1, done)
    out.update(gru_done=done, gru_z_state=z[0], gru_z_decay=z[1],
               gru_h_state=h[0], gru_h_decay=h[1], gru_n_state=nxt[0], gru_n_decay=nxt[1], gru_y=y,
               gru_c1_state=carry1[0], gru_c1_decay=carry1[1],
               gru_h1_state=h1[0], gru_n1_state=nxt1[0], gru_n1_decay=nxt1[1])

    # ---- Linear attention (ELU+1, carried S and z) ------------------------
    bsz, steps, heads, hd, feat = 2, 11, 2, 4, 6
    cell = linattn.LinearAttentionCell(features=feat, head_dim=hd, num_heads=heads)
    cell.output_projection = _Identity()   # kernel boundary = before RMSNorm / output Dense
    model = memoroid.Memoroid(cell=cell)
    x = rng.normal(size=(bsz, steps, feat))
    done = done_patterns(rng, bsz, steps)
    carry = (rng.normal(size=(bsz, 1, heads, hd, hd)) * 0.3, np.abs(rng.normal(size=(bsz, 1, heads, hd))) * 0.3)
    nxt, y = model(x, done, carry)
    out.update(la_done=done, la_q=cell.query(x), la_k=cell.key(x), la_v=cell.value(x),
               la_c_S=carry[0], la_c_z=carry[1], la_n_S=nxt[0], la_n_z=nxt[1],
               la_y=y.reshape(bsz, steps, heads, hd))
    # clamp branch: a state that drives the denominator below eps
    carry_neg = (carry[0], -np.abs(carry[1]) * 50.0)
    nxt, y = model(x, done, carry_neg)
    out.update(la_neg_c_z=carry_neg[1], la_neg_n_z=nxt[1], la_neg_y=y.reshape(bsz, steps, heads, hd))

    # ---- multiplicative-reset linear scan (RTRL sensitivities) ------------
    bsz, steps, hid, psize = 3, 10, 4, 3
    decay = rng.uniform(0.2, 0.95, size=(bsz, steps, hid))
    jac = {"w": rng.normal(size=(bsz, steps, hid, psize))}
    sens = {"w": rng.normal(size=(bsz, 1, hid, psize))}
    done = done_patterns(rng, bsz, steps)
    nxt = memoroid.Memoroid._propagate_sensitivities(None, decay, jac, sens, done)
    out.update(rt_decay=decay, rt_jac=jac["w"], rt_sens=sens["w"], rt_done=done, rt_next=nxt["w"])

    # ---- Mamba selective scan: the cell's own __call__, binary_operator and read; the
    #      projections / convolution in front of them are replaced by fixed arrays ----
    mamba = importlib.import_module(sm + "mamba")
    bsz, steps, heads, sdim, hdim = 2, 9, 3, 4, 5
    cell = object.__new__(mamba.MambaCell)          # no setup(): parameters are set by hand below
    cell.num_heads, cell.head_dim, cell.state_dim = heads, hdim, sdim
    cell.A_log = np.log(rng.uniform(1.0, 4.0, heads))
    cell.D = rng.normal(size=heads)
    cell.norm = _Identity()
    cell.output_projection = _Identity()
    proj = (rng.normal(size=(bsz, steps, heads, hdim)), rng.normal(size=(bsz, steps, heads, sdim)),
            rng.normal(size=(bsz, steps, heads, sdim)), rng.normal(size=(bsz, steps, heads * hdim)),
            _softplus(rng.normal(size=(bsz, steps, heads))))
    cell._project = lambda x: proj                  # (hidden, B, C, gate z, dt) of mamba.py:80-107
    model = memoroid.Memoroid(cell=cell)
    x = np.zeros((bsz, steps, 1))
    done = done_patterns(rng, bsz, steps)
    carry = (rng.normal(size=(bsz, 1, heads, sdim, hdim)), rng.uniform(0.3, 1.0, size=(bsz, 1, heads, 1, 1)))
    z = cell(x)
    h, nxt = model.scan_fn(z, carry, done)
    nxt2, y = model(x, done, carry)
    assert all(np.array_equal(p, q) for p, q in zip(nxt, nxt2))
    gate = proj[3] / (1.0 + np.exp(-proj[3]))
    out.update(mb_hidden=proj[0], mb_B=proj[1], mb_C=proj[2], mb_gate_in=proj[3], mb_dt=proj[4],
               mb_A_log=cell.A_log, mb_D=cell.D, mb_done=done, mb_c_state=carry[0], mb_c_decay=carry[1],
               mb_z_state=z[0], mb_z_decay=z[1], mb_h_state=h[0], mb_n_state=nxt[0], mb_n_decay=nxt[1],
               mb_y=y, mb_y_pre_gate=(y / gate).reshape(bsz, steps, heads, hdim))

    # ---- mLSTM: the cell's own __call__ (elements with the stabiliser leaf), binary_operator, read and
    #      initialize_carry under Memoroid.scan_fn; projections, gates' Dense layers, the head-wise norm and the
    #      output projection are replaced by fixed arrays / identities, so y / silu(z) is the read-out h_tilde ----
    mlstm = importlib.import_module(sm + "mlstm")
    bsz, steps, heads, hd = 2, 10, 2, 4
    cell = object.__new__(mlstm.mLSTMCell)          # no setup(): fields are set by hand below
    cell.features, cell.hidden_dim, cell.num_heads = heads * hd, heads * hd, heads
    proj = (rng.normal(size=(bsz, steps, heads, hd)), rng.normal(size=(bsz, steps, heads, hd)),
            rng.normal(size=(bsz, steps, heads, hd)), rng.normal(size=(bsz, steps, heads * hd)),
            np.zeros((bsz, steps, heads * hd)))
    cell._project = lambda x: proj                  # (query, key, value, z, u) of mlstm.py:148-161
    i_pre = rng.normal(size=(bsz, steps, heads)) * 1.5
    f_pre = rng.normal(size=(bsz, steps, heads)) * 2.0 + 1.0
    cell.i_gate = lambda g: i_pre
    cell.f_gate = lambda g: f_pre
    cell.norm = _Identity()
    cell.learnable_skip = np.zeros(heads * hd)
    cell.output_projection = _Identity()
    cell.drop = lambda y, deterministic=True: y
    cell.has_rng = lambda name: False
    model = memoroid.Memoroid(cell=cell)
    x = np.zeros((bsz, steps, 1))
    done = done_patterns(rng, bsz, steps)
    carry = (rng.normal(size=(bsz, 1, heads, hd, hd)) * 0.5, -np.abs(rng.normal(size=(bsz, 1, heads, 1, 1))),
             rng.normal(size=(bsz, 1, heads, hd, 1)) * 0.5, rng.normal(size=(bsz, 1, heads, 1, 1)))
    z = cell(x)
    h, nxt = model.scan_fn(z, carry, done)
    nxt2, y = model(x, done, carry)
    assert all(np.array_equal(p, q) for p, q in zip(nxt, nxt2))
    silu = proj[3] / (1.0 + np.exp(-proj[3]))
    out.update(ml_q=proj[0], ml_k=proj[1], ml_v=proj[2], ml_i_pre=i_pre, ml_f_pre=f_pre, ml_done=done,
               ml_c_C=carry[0], ml_c_logf=carry[1], ml_c_n=carry[2], ml_c_m=carry[3],
               ml_z_C=z[0], ml_z_logf=z[1], ml_z_n=z[2], ml_z_m=z[3],
               ml_h_C=h[0], ml_h_logf=h[1], ml_h_n=h[2], ml_h_m=h[3],
               ml_n_C=nxt[0], ml_n_logf=nxt[1], ml_n_n=nxt[2], ml_n_m=nxt[3],
               ml_h_tilde=(y / silu).reshape(bsz, steps, heads, hd))
    # default carry (initialize_carry: zeros with m = -1e9)
    carry0 = cell.initialize_carry(0, (bsz, heads * hd))
    nxt0, y0 = model(x, done, None)
    out.update(ml_default_c_m=carry0[3], ml_default_n_C=nxt0[0], ml_default_n_n=nxt0[2], ml_default_n_m=nxt0[3],
               ml_default_h_tilde=(y0 / silu).reshape(bsz, steps, heads, hd))

    # ---- RTRL through Memoroid.local_jacobian with the LRU cell (memoroid.py:143-176, lru.py:110-139):
    #      phantom injection, scan, read-out, the cell's local Jacobians and their propagation.  Own generator,
    #      so that the draws of every case above stay what they were. ----
    rng2 = np.random.default_rng(20250217)
    bsz, steps, feat, hid = 3, 9, 5, 4
    cell = lru.LRUCell(features=feat, hidden_dim=hid)
    for name, lo, hi in (("nu_log", 0.05, 0.6), ("theta_log", 0.05, 0.6)):
        cell._params[name] = np.log(rng2.uniform(lo, hi, hid))
        setattr(cell, name, cell._params[name])
    model = memoroid.Memoroid(cell=cell)
    x = rng2.normal(size=(bsz, steps, feat))
    done = done_patterns(rng2, bsz, steps)
    cplx = lambda *s: rng2.normal(size=s) + 1j * rng2.normal(size=s)
    carry = (cplx(bsz, 1, hid), cplx(bsz, 1, hid) * 0.3)
    sens = {"nu_log": cplx(bsz, 1, hid), "theta_log": cplx(bsz, 1, hid), "gamma_log": cplx(bsz, 1, hid),
            "B_real": cplx(bsz, 1, hid, feat), "B_imag": cplx(bsz, 1, hid, feat)}
    nxt, y, nsens = model.local_jacobian(x, done, carry, sens)
    zero_sens = cell.initialize_sensitivity(0, (bsz, feat))
    _, _, nsens0 = model.local_jacobian(x, done, carry, zero_sens)
    out.update(lj_x=x, lj_done=done, lj_c_state=carry[0], lj_c_decay=carry[1], lj_n_state=nxt[0], lj_n_decay=nxt[1],
               lj_y=y, lj_nu_log=cell.nu_log, lj_theta_log=cell.theta_log, lj_gamma_log=cell.gamma_log,
               lj_B=cell.B_real + 1j * cell.B_imag, lj_C=cell.C_real + 1j * cell.C_imag, lj_D=cell.D)
    for name in sens:
        out["lj_s_" + name], out["lj_ns_" + name], out["lj_ns0_" + name] = sens[name], nsens[name], nsens0[name]

    # ---- S5: the reference's own discretisation (hippo.py:34-50), elements, operator and read-out
    #      (s5.py:97-143) under Memoroid, and the HiPPO-DPLR eigenvalues its setup() starts from
    #      (hippo.py:20-32).  setup() is bypassed: parameters are set by hand. ----
    s5 = importlib.import_module(sm + "s5")
    hippo = importlib.import_module("memorax.networks.hippo")
    rng3 = np.random.default_rng(20250218)
    bsz, steps, feat, nstate = 3, 10, 4, 6
    x = rng3.normal(size=(bsz, steps, feat))
    done = done_patterns(rng3, bsz, steps)
    cplx = lambda *s: rng3.normal(size=s) + 1j * rng3.normal(size=s)
    carry = (cplx(bsz, 1, nstate), cplx(bsz, 1, nstate) * 0.3)
    params = dict(lambda_real=-np.abs(rng3.normal(size=nstate)) - 0.1, lambda_imag=rng3.normal(size=nstate) * 3.0,
                  B=rng3.normal(size=(nstate, feat, 2)) * 0.5, C=rng3.normal(size=(feat, nstate, 2)) * 0.5,
                  d=rng3.normal(size=feat), log_step=np.log(rng3.uniform(0.001, 0.1, size=(nstate, 1))))
    out.update(s5_x=x, s5_done=done, s5_c_state=carry[0], s5_c_decay=carry[1], **{"s5_p_" + k: v for k, v in params.items()})
    for disc in ("zoh", "bilinear"):
        cell = object.__new__(s5.S5Cell)
        cell.features, cell.state_size, cell.discretization = feat, nstate, disc
        cell.clip_eigens, cell.step_rescale, cell.dtype = False, 1.0, F64
        for k, v in params.items():
            setattr(cell, k, v)
        model = memoroid.Memoroid(cell=cell)
        z = cell(x)
        nxt, y = model(x, done, carry)
        out.update({f"s5_{disc}_z_state": z[0], f"s5_{disc}_lambda_bar": z[1][0, 0], f"s5_{disc}_n_state": nxt[0],
                    f"s5_{disc}_n_decay": nxt[1], f"s5_{disc}_y": y})
    for n in (4, 16):
        out[f"hippo_lambda_{n}"] = hippo.make_dplr_hippo(n)[0]

    np.savez_compressed(args.out, **out)
    print("wrote", args.out, "with", len(out), "arrays")


if __name__ == "__main__":
    main()
