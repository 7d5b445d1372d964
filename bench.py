#!/usr/bin/env python
"""Benchmark of the sequence-mixing hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c1|c5|a7|n1|n1t|n2|n3|n4]
    python bench.py --impl reference ...      # CPU arm: the oracle port, host cores

A step is one pass of the hot path over one batch of seeded synthetic input:
forward + backward of the op for c2 / c4, forward only for c1 (the shapes and
value distributions of the reference's headline configurations; the reference
names no dataset).  One process per GPU; every rank owns a full batch of
independent sequences (weak scaling, no data-path collective).  Rank 0 prints
ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
NSETS = 4  # input sets rotated between steps so that no step finds its inputs in L2


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------- workloads
class LinAttnC2:
    """Causal linear attention fwd+bwd: B=256, H=4, T=256, d=64, bf16 in, fp32
    state, chunk 64, done ~ Bernoulli(0.01), initial state ~ N(0, 0.1)."""
    name = "c2_linear_attention_fwd_bwd"
    dtype = "bf16"
    B, H, T, D = 256, 4, 256, 64
    p_done = 0.01
    seed = 1234 + 2
    # bytes of q,k,v,o (fwd) and q,k,v,do,dq,dk,dv (bwd) per token-head, bf16
    fwd_bytes_per_token_head = 4 * 64 * 2
    bwd_bytes_per_token_head = 7 * 64 * 2
    dominant = "linattn_bwd_kernel"
    launches_per_step = 2
    # consecutive steps stream (copy-in of step i+1 under the copy-out of step i), which keeps both copy engines busy;
    # cutting a step into batch slices on top of that only multiplies the copies (measured: 0.91 of the wire floor
    # with 4 slices, 0.97 with 1)
    e2e_slices = 1
    e2e_mode = "stream"
    # dram__bytes_read.sum + dram__bytes_write.sum of one linattn_bwd_kernel launch at
    # this size (ncu capture summarised under profiles/)
    dominant_traffic_bytes = 251.8e6

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        shp = (self.B, self.T, self.H, self.D)
        mk = lambda *s: torch.randn(*s, generator=g, device=device)
        return dict(
            q=(mk(*shp) / 8).bfloat16(), k=(mk(*shp) / 8).bfloat16(), v=(mk(*shp) / 8).bfloat16(),
            d_o=mk(*shp).bfloat16(),
            s0=mk(self.B, self.H, self.D, self.D) * 0.1, z0=mk(self.B, self.H, self.D).abs() * 0.1,
            done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def state_bytes(self):
        return self.B * self.H * (self.D * self.D + self.D) * 4

    def algorithmic_bytes(self):
        th = self.B * self.T * self.H
        fwd = th * self.fwd_bytes_per_token_head + 2 * self.state_bytes()
        bwd = th * self.bwd_bytes_per_token_head + 2 * self.state_bytes()
        return {"linattn_fwd_kernel": fwd, "linattn_bwd_kernel": bwd}

    def algorithmic_flops(self):
        # dense 64 x 64 tiles: fwd 2(C d_k + C d_v + 2 d_k d_v), bwd 2C(3 d_k + 2 d_v) + 10 d_k d_v per token-head
        th = self.B * self.T * self.H
        return {"linattn_fwd_kernel": th * 32768, "linattn_bwd_kernel": th * 81920}

    def step(self, x, ops, mark=None):
        o, s_last, z_last, states = ops.linattn_fwd(x["q"], x["k"], x["v"], x["s0"], x["z0"], x["done"],
                                                    save_states=True)
        if mark:
            mark[0].record()
        dq, dk, dv, ds0, dz0 = ops.linattn_bwd(x["q"], x["k"], x["v"], x["d_o"], states, x["done"])
        if mark:
            mark[1].record()
        return (o, s_last, z_last, dq, dk, dv, ds0, dz0)

    def cpu_step(self, x):
        """The reference's own formulation (every S_t materialised, prefix over
        time, read-out; autograd backward) in fp32 on the host cores."""
        from oracle import memoroid_oracle as mo
        q, k, v = (x[n].float().requires_grad_() for n in ("q", "k", "v"))
        o, s_last, z_last = mo.linattn_reference_form(q, k, v, x["s0"], x["z0"], x["done"].float())
        (o * x["d_o"].float()).sum().backward()
        return o

    cpu_sample_batch = 64


class LruC4:
    """Complex diagonal LRU recurrence fwd+bwd, complex64, time-invariant lambda:
    B=1024, T=1024, D=512, |lambda|~U[0.9,0.999], phase~U[0,pi/10], done~Bern(0.002)."""
    name = "c4_complex_lru_fwd_bwd"
    dtype = "c64"
    B, T, D = 1024, 1024, 512
    p_done = 0.002
    seed = 1234 + 4
    dominant = "linrec_bwd_kernel"
    launches_per_step = 3
    # one linrec_bwd_kernel launch: 5602.0 MB measured at B=448 (ncu capture summarised under profiles/),
    # scaled by 1024 / 448 (traffic is proportional to the batch)
    dominant_traffic_bytes = 5602.0e6 * 1024 / 448
    cpu_sample_batch = 64
    e2e_mode = "stream"   # 8.6 GB in, 4.3 GB out per step: the copy-in of step i+1 runs under the copy-out of step i

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        mag = 0.9 + 0.099 * torch.rand(self.D, generator=g, device=device)
        ph = torch.rand(self.D, generator=g, device=device) * math.pi / 10
        shp = (self.B, self.T, self.D)
        cplx = lambda: torch.view_as_complex(torch.randn(*shp, 2, generator=g, device=device))
        return dict(lam=torch.polar(mag, ph).to(torch.complex64), bu=cplx(), gh=cplx(),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        n = self.B * self.T * self.D
        return {"linrec_fwd_kernel": 16 * n, "linrec_bwd_kernel": 24 * n}

    def algorithmic_flops(self):
        n = self.B * self.T * self.D   # one complex multiply-add per element forward, two backward
        return {"linrec_fwd_kernel": 8 * n, "linrec_bwd_kernel": 16 * n}

    def step(self, x, ops, mark=None):
        h, _ = ops.linrec_fwd(x["lam"], x["bu"], None, None, x["done"], want_decay=False)
        if mark:
            mark[0].record()
        gb, ga, _ = ops.linrec_bwd(x["lam"], h, None, x["done"], x["gh"], None, need_ga=True, need_gh0=False)
        if mark:
            mark[1].record()
        return (h[:, -1], gb, ga)

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        lam, bu = x["lam"].clone().requires_grad_(), x["bu"].clone().requires_grad_()
        h0 = torch.zeros(bu.shape[0], bu.shape[2], dtype=bu.dtype)
        h, _ = mo.linrec_seq(lam, bu, h0, x["done"].float())
        (h * x["gh"]).sum().real.backward()
        return h


class LinRecC1:
    """Real diagonal recurrence, forward only, fp32: B=64, T=128, D=256,
    a = sigmoid(N(0,1)), done ~ Bernoulli(0.01), carried h0."""
    name = "c1_real_linrec_fwd"
    dtype = "f32"
    B, T, D = 64, 128, 256
    p_done = 0.01
    seed = 1234 + 1
    dominant = "linrec_fwd_kernel"
    launches_per_step = 1
    dominant_traffic_bytes = None
    cpu_sample_batch = 64
    use_graph = True   # a 25 MB step is shorter than a Python launch: replay it as a CUDA graph

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        shp = (self.B, self.T, self.D)
        rn = lambda *s: torch.randn(*s, generator=g, device=device)
        return dict(a=torch.sigmoid(rn(*shp)), b=rn(*shp), h0=rn(self.B, self.D),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        return {"linrec_fwd_kernel": 12 * self.B * self.T * self.D}

    def algorithmic_flops(self):
        return {"linrec_fwd_kernel": 2 * self.B * self.T * self.D}

    def step(self, x, ops, mark=None):
        if mark:
            mark[0].record()
        h, _ = ops.linrec_fwd(x["a"], x["b"], x["h0"], None, x["done"], want_decay=False)
        if mark:
            mark[1].record()
        return (h,)

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        with torch.no_grad():
            return mo.linrec_seq(x["a"], x["b"], x["h0"], x["done"].float())[0]


class GDeltaC3:
    """Gated delta rule fwd+bwd: B=128, H=8, T=512, d=128, bf16 in, fp32 state
    (zero-initialised), q,k L2-normalised, beta=sigmoid(N), alpha=exp(-softplus(N)),
    done ~ Bernoulli(0.005)."""
    name = "c3_gated_delta_rule_fwd_bwd"
    dtype = "bf16"
    B, H, T, D = 128, 8, 512, 128
    p_done = 0.005
    seed = 1234 + 3
    dominant = "gdelta_bwd_kernel"
    launches_per_step = 3
    e2e_slices = 1   # as for c2: the streaming of consecutive steps is the overlap (0.97 -> 0.995 of the wire floor)
    e2e_mode = "stream"
    # one gdelta_bwd_kernel launch: 304.4 MB measured at B=32 (profiles/), scaled by 128 / 32
    dominant_traffic_bytes = 304.4e6 * 4
    cpu_sample_batch = 4

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        shp = (self.B, self.T, self.H, self.D)
        mk = lambda *s: torch.randn(*s, generator=g, device=device)
        nrm = lambda x: x / x.norm(dim=-1, keepdim=True)
        return dict(q=nrm(mk(*shp)).bfloat16(), k=nrm(mk(*shp)).bfloat16(), v=mk(*shp).bfloat16(),
                    d_o=mk(*shp).bfloat16(), beta=torch.sigmoid(mk(*shp[:3])),
                    alpha=torch.exp(-torch.nn.functional.softplus(mk(*shp[:3]))),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        th = self.B * self.T * self.H
        state = self.B * self.H * self.D * self.D * 4
        # q,k,v,o bf16 + alpha,beta fp32 | q,k,v,do,dq,dk,dv bf16 + alpha,beta,dalpha,dbeta fp32
        return {"gdelta_fwd_kernel": th * (4 * 256 + 8) + state, "gdelta_bwd_kernel": th * (7 * 256 + 16) + state}

    # FLOP per token-head of the algorithm the kernels run (tensor-core products plus the fp32 triangular work)
    fwd_flop_per_token_head = 155648
    bwd_flop_per_token_head = 426000

    def algorithmic_flops(self):
        th = self.B * self.T * self.H
        return {"gdelta_fwd_kernel": th * self.fwd_flop_per_token_head, "gdelta_bwd_kernel": th * self.bwd_flop_per_token_head}

    def step(self, x, ops, mark=None):
        o, s_last, states = ops.gdelta_fwd(x["q"], x["k"], x["v"], x["alpha"], x["beta"], None, x["done"],
                                           save_states=True)
        if mark:
            mark[0].record()
        outs = ops.gdelta_bwd(x["q"], x["k"], x["v"], x["alpha"], x["beta"], x["d_o"], states, x["done"])
        if mark:
            mark[1].record()
        return (o, s_last) + tuple(outs)

    def cpu_step(self, x):
        """Sequential recurrence (the definition of the op) with autograd, fp32, host cores."""
        from oracle import memoroid_oracle as mo
        q, k, v = (x[n].float().requires_grad_() for n in ("q", "k", "v"))
        s0 = torch.zeros(q.shape[0], self.H, self.D, self.D)
        o, _ = mo.gdelta_seq(q, k, v, x["alpha"], x["beta"], s0, x["done"].float())
        (o * x["d_o"].float()).sum().backward()
        return o


class TrainC5:
    """Training step (fwd + bwd + gradient all-reduce + Adam) of a 4-layer GTrXL-style value
    network with the delta-rule mixer: d_model 512, MLP 4x, bf16 parameters, fp32 Adam moments,
    512 sequences x 256 steps of 128-dim observations per GPU (4096 sequences over 8 GPUs),
    done ~ Bernoulli(0.005); the mixer has 8 heads of 64."""
    name = "c5_gtrxl_deltanet_train_step"
    dtype = "bf16"
    B, T, OBS = 512, 256, 128
    p_done = 0.005
    seed = 1234 + 5
    dominant = "train_step"
    # this library's kernels per step: per layer 3 delta-rule launches (prep, fwd, bwd), 9 norm launches (three norms:
    # fwd, bwd, bwd reduce), 4 gated-residual, 4 L2-normalise, 12 column-sum launches (six biased Dense layers x 2);
    # plus the embedding's column sum (2) and the Adam step
    launches_per_step = 4 * (3 + 9 + 4 + 4 + 12) + 2 + 1
    dominant_traffic_bytes = None
    cpu_sample_batch = 2

    def __init__(self, batch=None):
        self.B = batch or self.B
        self.trainer = None

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        return dict(obs=torch.randn(self.B, self.T, self.OBS, generator=g, device=device).bfloat16(),
                    target=torch.randn(self.B, self.T, generator=g, device=device),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def _build(self, device):
        import torch.distributed as dist
        from memorax_b200.blocks import FlatAdamTrainer, GTrXLStyleValueNet
        torch.manual_seed(0)   # same initial parameters on every rank
        model = GTrXLStyleValueNet(obs_dim=self.OBS).to(device=device, dtype=torch.bfloat16)
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.trainer = FlatAdamTrainer(model, world_size=world)
        dense = sum(m.weight.numel() for m in model.modules() if isinstance(m, torch.nn.Linear))
        # 6 FLOP per dense weight per token (fwd + bwd) + the mixer's own 582 kFLOP per token-head
        self.flop_per_token = 6.0 * dense + 4 * 8 * 582e3 / 4   # per token-head at d = 64: a quarter of d = 128's products

    def step(self, x, ops, mark=None):
        if self.trainer is None:
            self._build(x["obs"].device)
        if mark:
            mark[0].record()
        loss = self.trainer.step(x["obs"], x["done"], x["target"])
        if mark:
            mark[1].record()
        return (loss.reshape(1),)

    def algorithmic_bytes(self):
        return {"train_step": 0}

    def roofline(self, dominant_ms):
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                peak, kind = float(json.load(fh)["bf16_tflops_sustained"]), "measured (sustained)"
        except Exception:
            peak, kind = 1400.0, "fallback"
        achieved = self.flop_per_token * self.tokens() / (dominant_ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "whole training step (library GEMMs + this library's kernels)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_kind": f"of {kind}",
                "traffic": None, "flop_per_step": self.flop_per_token * self.tokens(), "ms_per_launch": dominant_ms,
                "parameters": self.trainer.num_params}

    def cpu_step(self, x):
        """Same network on the host cores in fp32 with the oracle's sequential delta rule."""
        from oracle import memoroid_oracle as mo
        if not hasattr(self, "_cpu"):
            torch.manual_seed(0)
            d, H, hd = 512, 8, 64
            lin = lambda i, o: torch.nn.Linear(i, o)
            self._cpu = dict(embed=lin(self.OBS, d), head=lin(d, 1), layers=[
                dict(n1=torch.nn.LayerNorm(d), q=lin(d, d), k=lin(d, d), v=lin(d, d), gate=lin(d, 2 * H), rms=torch.nn.RMSNorm(d, eps=1e-6),
                     out=lin(d, d), g1=lin(d, d), n2=torch.nn.LayerNorm(d), up=lin(d, 4 * d), down=lin(4 * d, d), g2=lin(d, d))
                for _ in range(4)])
        P, F = self._cpu, torch.nn.functional
        h = P["embed"](x["obs"].float())
        B, T, _ = h.shape
        for L in P["layers"]:
            y = L["n1"](h)
            hv = lambda t: t.view(B, T, 8, 64)
            q, k = F.normalize(hv(L["q"](y)), dim=-1), F.normalize(hv(L["k"](y)), dim=-1)
            bl, al = L["gate"](y).chunk(2, -1)
            o, _ = mo.gdelta_seq(q, k, hv(L["v"](y)), torch.exp(-F.softplus(al)), torch.sigmoid(bl),
                                 torch.zeros(B, 8, 64, 64), x["done"].float())
            h = h + torch.sigmoid(L["g1"](h)) * L["out"](L["rms"](o.reshape(B, T, -1)))
            h = h + torch.sigmoid(L["g2"](h)) * L["down"](F.gelu(L["up"](L["n2"](h)), approximate="tanh"))
        loss = 0.5 * (P["head"](h).squeeze(-1) - x["target"]).square().mean()
        loss.backward()
        return loss


class MambaN2:
    """Mamba selective scan fwd+bwd (the scan of MambaCell, mamba.py:109-122, at the shipped example's
    size, examples/gradient_ppo_craftax.py:70-98: MambaCell(features=512) = 8 heads x 16 x 16 state,
    128 environments per device; T widened from 64 to 256 steps so that the inputs exceed L2): real fp32
    recurrence over H*N*P = 2048 channels with a per-(b,t,head) decay that the kernels read un-expanded
    (one value per group of N*P = 256 channels) and whose gradient they reduce per head."""
    name = "n2_mamba_scan_fwd_bwd"
    dtype = "f32"
    B, T, H, N, P = 128, 256, 8, 16, 16
    p_done = 0.01
    seed = 1234 + 6
    dominant = "linrec_grouped_bwd_kernel"
    launches_per_step = 2
    dominant_traffic_bytes = None
    cpu_sample_batch = 16

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        width = self.H * self.N * self.P
        rn = lambda *s: torch.randn(*s, generator=g, device=device)
        dt = torch.nn.functional.softplus(rn(self.B, self.T, self.H) - 2.0)
        a_neg = -torch.exp(torch.rand(self.H, generator=g, device=device) * math.log(16.0))
        decay = torch.exp(dt * a_neg)
        return dict(a=decay.contiguous(), z=rn(self.B, self.T, width) * 0.1, gh=rn(self.B, self.T, width),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        n = self.B * self.T * self.H * self.N * self.P
        # fwd: read z, write h (+ the per-head decay); bwd: read h, gh, write gz (+ decay in, its gradient out)
        small = 4 * self.B * self.T * self.H
        return {"linrec_grouped_fwd_kernel": 8 * n + small, "linrec_grouped_bwd_kernel": 12 * n + 2 * small}

    def algorithmic_flops(self):
        n = self.B * self.T * self.H * self.N * self.P
        return {"linrec_grouped_fwd_kernel": 2 * n, "linrec_grouped_bwd_kernel": 4 * n}

    def step(self, x, ops, mark=None):
        h, _ = ops.linrec_grouped_fwd(x["a"], x["z"], None, None, x["done"], want_decay=False)
        if mark:
            mark[0].record()
        gb, ga, _ = ops.linrec_grouped_bwd(x["a"], h, None, x["done"], x["gh"], None, need_ga=True, need_gh0=False)
        if mark:
            mark[1].record()
        return (h[:, -1], gb, ga)

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        a, z = x["a"].clone().requires_grad_(), x["z"].clone().requires_grad_()
        h, _ = mo.linrec_seq(a.repeat_interleave(self.N * self.P, dim=-1), z, torch.zeros(z.shape[0], z.shape[2]),
                             x["done"].float())
        (h * x["gh"]).sum().backward()
        return h


class MinGruA7:
    """MinGRU scan with its gate math fused in (min_gru.py:52-78 under the reset wrapper of memoroid.py:60-91),
    fwd+bwd: the two Dense pre-activations z, h~ in, log-space states and read-out h = exp(x) out, cotangents of the
    pre-activations back.  B=256, T=256, D=1024, fp32, done ~ Bernoulli(0.01), default (-inf) carry."""
    name = "a7_mingru_fused_gates_fwd_bwd"
    dtype = "f32"
    B, T, D = 256, 256, 1024
    p_done = 0.01
    seed = 1234 + 9
    dominant = "loglinrec_bwd_kernel"
    launches_per_step = 2
    dominant_traffic_bytes = None
    cpu_sample_batch = 32

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        rn = lambda *s: torch.randn(*s, generator=g, device=device)
        shp = (self.B, self.T, self.D)
        return dict(z=rn(*shp) * 2.0, ht=rn(*shp) * 2.0, gy=rn(*shp),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        n = self.B * self.T * self.D
        # fwd: read z, h~; write x, y.  bwd: read z, h~, x, the cotangents of x and y; write the cotangents of z, h~
        return {"loglinrec_fwd_kernel": 16 * n, "loglinrec_bwd_kernel": 28 * n}

    def algorithmic_flops(self):
        n = self.B * self.T * self.D
        return {"loglinrec_fwd_kernel": 20 * n, "loglinrec_bwd_kernel": 30 * n}

    def step(self, x, ops, mark=None):
        z, ht = x["z"].detach().requires_grad_(), x["ht"].detach().requires_grad_()
        xs, y, _ = ops.MinGRUFused.apply(z, ht, None, None, x["done"])
        if mark:
            mark[0].record()
        gz, gh = torch.autograd.grad((y,), (z, ht), (x["gy"],))
        if mark:
            mark[1].record()
        return (xs[:, -1], y, gz, gh)

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        sp = torch.nn.functional.softplus
        z, ht = x["z"].clone().requires_grad_(), x["ht"].clone().requires_grad_()
        log_state = -sp(-z) + torch.where(ht >= 0, torch.log(torch.relu(ht) + 0.5), -sp(-ht))
        xs, _ = mo.mingru_seq(log_state, -sp(z), torch.full((z.shape[0], z.shape[2]), -float("inf")), x["done"].float())
        (xs.exp() * x["gy"]).sum().backward()
        return xs


class RtrlN3:
    """One RTRL segment of the LRU cell (Memoroid.local_jacobian, memoroid.py:143-176 with lru.py:110-139): scan,
    read-out, the five local Jacobians and their propagation to the sensitivities after the last step.  B=64
    sequences x T=64 steps, F=64 features, N=128 hidden units, fp32 / complex64, done ~ Bernoulli(0.01)."""
    name = "n3_rtrl_lru_segment"
    dtype = "c64"
    B, T, F, N = 64, 64, 64, 128
    p_done = 0.01
    seed = 1234 + 10
    dominant = "linrec_fwd_kernel"
    launches_per_step = 6
    dominant_traffic_bytes = None
    cpu_sample_batch = 8
    roofline_of_step = True

    def __init__(self, batch=None):
        self.B = batch or self.B
        self.model = None

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        return dict(x=torch.randn(self.B, self.T, self.F, generator=g, device=device),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def _model(self, device):
        if self.model is None:
            from memorax_b200.memoroid import LRUCell, Memoroid
            torch.manual_seed(self.seed)
            self.model = Memoroid(LRUCell(self.F, self.N, r_min=0.9, r_max=0.999, max_phase=math.pi / 10).to(device))
            self.carry = tuple(c.to(device) for c in self.model.cell.initialize_carry(None, (self.B, self.F)))
            self.sens = self.model.initialize_sensitivity(None, (self.B, self.F))
        return self.model

    def algorithmic_bytes(self):
        # the formulation's own traffic: the two (B,T,N,F) complex Jacobians of the input matrix written and read once,
        # the three (B,T,N) ones likewise, inputs in, read-out and sensitivities out
        big = 2 * 8 * self.B * self.T * self.N * self.F
        small = 3 * 8 * self.B * self.T * self.N
        return 2 * (big + small) + 8 * self.B * self.T * self.F + 8 * self.B * self.N * (2 * self.F + 3)

    def roofline(self, step_ms):
        hbm, _, kind = measured_peaks()
        byts = self.algorithmic_bytes()
        return {"bound": "hbm", "achieved": byts / (step_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                "frac": byts / (step_ms * 1e-3) / 1e9 / hbm, "peak_kind": f"of {kind}", "algorithmic_bytes_per_step": byts,
                "note": "whole segment: library GEMMs and PyTorch elementwise ops build the Jacobians, this repository's "
                        "kernels run the scan and the five last-state-only propagations"}

    def step(self, x, ops, mark=None):
        model = self._model(x["x"].device)
        if mark:
            mark[0].record()
        with torch.no_grad():
            carry, y, sens = model.local_jacobian(x["x"], x["done"], self.carry, self.sens)
        if mark:
            mark[1].record()
        return (y, carry[0][:, 0]) + tuple(sens[k] for k in sorted(sens))

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        cell = self._model("cpu").cell if self.model is None else self.model.cell
        p = {n: getattr(cell, n).detach().cpu() for n in ("nu_log", "theta_log", "gamma_log", "B_real", "B_imag", "C_real", "C_imag", "D")}
        nb = x["x"].shape[0]
        sens = {"nu_log": torch.zeros(nb, 1, self.N, dtype=torch.complex64), "theta_log": torch.zeros(nb, 1, self.N, dtype=torch.complex64),
                "gamma_log": torch.zeros(nb, 1, self.N, dtype=torch.complex64),
                "B_real": torch.zeros(nb, 1, self.N, self.F, dtype=torch.complex64), "B_imag": torch.zeros(nb, 1, self.N, self.F, dtype=torch.complex64)}
        with torch.no_grad():
            return mo.lru_rtrl_seq(x["x"], x["done"].float(), torch.zeros(nb, self.N, dtype=torch.complex64), p["nu_log"], p["theta_log"],
                                   p["gamma_log"], torch.complex(p["B_real"], p["B_imag"]), torch.complex(p["C_real"], p["C_imag"]), p["D"], sens)


class MlstmN1:
    """mLSTM scan + read-out fwd+bwd (mlstm.py:163-240) at the linear-attention configuration's size: B=256,
    H=4, T=256, head dim 64, fp32; log_i ~ N(0, 0.1^2) (the cell's gate bias init), log_f = -softplus(-N(4.5, 1))
    (forget-gate bias linspace(3, 6)), q, k, v ~ N(0,1) with k / sqrt(64); done ~ Bernoulli(0.01)."""
    name = "n1_mlstm_fwd_bwd"
    dtype = "f32"
    B, H, T, D = 256, 4, 256, 64
    p_done = 0.01
    seed = 1234 + 7
    dominant = "mlstm_bwd_kernel"
    launches_per_step = 2
    dominant_traffic_bytes = None
    cpu_sample_batch = 4

    def __init__(self, batch=None):
        self.B = batch or self.B

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        shp = (self.B, self.T, self.H, self.D)
        rn = lambda *s: torch.randn(*s, generator=g, device=device)
        return dict(q=rn(*shp), k=rn(*shp) / math.sqrt(self.D), v=rn(*shp), dh=rn(*shp), log_i=rn(*shp[:3]) * 0.1,
                    log_f=-torch.nn.functional.softplus(-(rn(*shp[:3]) + 4.5)),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def algorithmic_bytes(self):
        th = self.B * self.T * self.H
        # q,k,v in, h out (+ gates) | q,k,v,dh in, dq,dk,dv out (+ gates in, their gradients out), fp32
        return {"mlstm_fwd_kernel": th * (4 * 4 * self.D + 8), "mlstm_bwd_kernel": th * (7 * 4 * self.D + 16)}

    def algorithmic_flops(self):
        th = self.B * self.T * self.H
        # per step: update + read of a d x d memory forward (4 d^2), twice that plus the two cotangent copies backward
        return {"mlstm_fwd_kernel": th * 4 * self.D * self.D, "mlstm_bwd_kernel": th * 14 * self.D * self.D}

    def step(self, x, ops, mark=None):
        h, c_t, n_t, m_t, _ = ops.mlstm_fwd(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], None, None, None, None, x["done"])
        if mark:
            mark[0].record()
        outs = ops.mlstm_bwd(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], None, None, None, x["done"], x["dh"])
        if mark:
            mark[1].record()
        return (h, c_t) + tuple(outs[:5])

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        q, k, v, li, lf = (x[n].clone().requires_grad_() for n in ("q", "k", "v", "log_i", "log_f"))
        b = q.shape[0]
        h, _ = mo.mlstm_seq(q, k, v, li, lf, torch.zeros(b, self.H, self.D, self.D), torch.zeros(b, self.H, self.D),
                            torch.full((b, self.H), -1e9), x["done"].float())
        (h * x["dh"]).sum().backward()
        return h


class MlstmTcN1(MlstmN1):
    """The mLSTM workload n1 through the chunked tensor-core kernels: same shapes and gate distributions, q, k, v and
    the read-out in bf16 (the numerical class of configuration 2), gates and state fp32."""
    name = "n1_mlstm_tensor_core_fwd_bwd"
    dtype = "bf16"
    dominant = "mlstm_tc_bwd_kernel"
    cpu_sample_batch = 4

    def host_inputs(self, seed_offset=0, device="cpu"):
        x = super().host_inputs(seed_offset, device)
        for key in ("q", "k", "v", "dh"):
            x[key] = x[key].bfloat16()
        return x

    def algorithmic_bytes(self):
        n = self.B * self.T * self.H
        gates = 2 * 4 * n
        # fwd: q, k, v in, h out (bf16), gates, per-step stabiliser out; bwd: q, k, v, dh in, dq, dk, dv out, gates in, gate gradients out
        return {"mlstm_tc_fwd_kernel": 4 * 2 * self.D * n + gates + 4 * n,
                "mlstm_tc_bwd_kernel": 7 * 2 * self.D * n + 2 * gates + 4 * n}

    def algorithmic_flops(self):
        n = self.B * self.T * self.H
        c, d = 64, self.D
        # per token-head: QK^T, P~(V|1), Q S, K^T(V|1) forward; P, dA, R, Y and the four phase-2 groups backward
        return {"mlstm_tc_fwd_kernel": n * 2 * (c * d + c * (d + 8) + d * (d + 8) + d * (d + 8)),
                "mlstm_tc_bwd_kernel": n * 2 * (2 * c * d + 2 * d * (d + 8) + 2 * c * d + 2 * d * (d + 16) + 2 * c * d + d * (d + 8))}

    def step(self, x, ops, mark=None):
        h, c_last, n_last, _, _, res = ops.mlstm_tc_fwd(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], None, None, None, None,
                                                        x["done"], save=True)
        if mark:
            mark[0].record()
        out = ops.mlstm_tc_bwd(x["q"], x["k"], x["v"], x["log_i"], x["log_f"], None, None, None, x["done"], x["dh"], c_last,
                               n_last, res, need_state_grads=False)
        if mark:
            mark[1].record()
        return (h, out[0], out[1], out[2], out[3], out[4])

    def cpu_step(self, x):
        return super().cpu_step({k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in x.items()})


class LruLayerN4:
    """The LRU layer as the reference's Memoroid runs it at inference (lru.py:78-108 around memoroid.py:93-109):
    input projection B_norm u, the complex scan of configuration 4 (B=1024, T=1024, N=512 states), read-out
    (C h).real + D u; features F=256, fp32 inputs, forward only, TF32 GEMMs (XLA's default for f32 dots on
    NVIDIA GPUs).  The measured call is ``Memoroid(LRUCell)``: both projections as ONE real library GEMM each over
    interleaved (re, im) weights, the scan by this repository's kernel.  ``variants_ms`` times the same layer as the
    reference formulation writes it (complex matmuls of a complex copy of the inputs, real part taken afterwards)."""
    name = "n4_lru_layer_inference"
    dtype = "c64"
    B, T, F, N = 1024, 1024, 256, 512
    p_done = 0.002
    seed = 1234 + 8
    dominant = "linrec_fwd_kernel"
    launches_per_step = 1
    dominant_traffic_bytes = None
    cpu_sample_batch = 8
    roofline_of_step = True

    def __init__(self, batch=None):
        self.B = batch or self.B
        self.cell = None

    def tokens(self):
        return self.B * self.T

    def host_inputs(self, seed_offset=0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(self.seed + seed_offset)
        return dict(x=torch.randn(self.B, self.T, self.F, generator=g, device=device),
                    done=(torch.rand(self.B, self.T, generator=g, device=device) < self.p_done).to(torch.uint8))

    def _cell(self, device):
        if self.cell is None:
            from memorax_b200.memoroid import LRUCell
            torch.manual_seed(self.seed)
            self.cell = LRUCell(self.F, self.N, r_min=0.9, r_max=0.999, max_phase=math.pi / 10).to(device)
        return self.cell

    def algorithmic_bytes(self):
        # inputs in and outputs out (fp32), and the (B,T,N) complex64 intermediates between the three launches:
        # projected inputs written and read, states written and read
        return 2 * 4 * self.B * self.T * self.F + 4 * 8 * self.B * self.T * self.N

    def roofline(self, step_ms):
        hbm, tc, kind = measured_peaks()
        byts = self.algorithmic_bytes()
        flop = 2 * self.B * self.T * (2 * self.N) * self.F * 2 + 8 * self.B * self.T * self.N
        return {"bound": "hbm", "achieved": byts / (step_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                "frac": byts / (step_ms * 1e-3) / 1e9 / hbm, "peak_kind": f"of {kind}",
                "algorithmic_bytes_per_step": byts, "algorithmic_flop_per_step": flop,
                "tf32_gemm_tflops": flop / (step_ms * 1e-3) / 1e12,
                "note": "whole layer, three launches with their intermediates in HBM; the two projections are library "
                        "GEMMs, the scan is this repository's kernel"}

    def _run(self, fn):
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            with torch.no_grad():
                return fn()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev

    def step(self, x, ops, mark=None):
        from memorax_b200.memoroid import Memoroid
        model = Memoroid(self._cell(x["x"].device))
        if mark:
            mark[0].record()
        carry, y = self._run(lambda: model(x["x"], x["done"]))
        if mark:
            mark[1].record()
        return (carry[0][:, 0], y)

    def variants(self, x, ops, reps=3):
        cell = self._cell(x["x"].device)

        def reference_form():
            lam = cell.diag_lambda()
            b_norm = torch.complex(cell.B_real, cell.B_imag) * torch.exp(cell.gamma_log)[:, None]
            bu = torch.matmul(x["x"].to(torch.complex64), b_norm.t())
            h, _ = ops.linrec_fwd(lam, bu, None, None, x["done"], want_decay=False)
            return torch.matmul(h, torch.complex(cell.C_real, cell.C_imag).t()).real + cell.D * x["x"]

        self._run(reference_form)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            self._run(reference_form)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        return {"complex_matmul_formulation": e0.elapsed_time(e1) / reps}

    def cpu_step(self, x):
        from oracle import memoroid_oracle as mo
        cell = self._cell("cpu")
        with torch.no_grad():
            lam = cell.diag_lambda()
            b_norm = torch.complex(cell.B_real, cell.B_imag) * torch.exp(cell.gamma_log)[:, None]
            bu = torch.matmul(x["x"].to(torch.complex64), b_norm.t())
            h, _ = mo.linrec_seq(lam, bu, torch.zeros(bu.shape[0], bu.shape[2], dtype=bu.dtype), x["done"].float())
            return torch.matmul(h, torch.complex(cell.C_real, cell.C_imag).t()).real + cell.D * x["x"]


WORKLOADS = {"n3": RtrlN3, "a7": MinGruA7, "n4": LruLayerN4, "n1": MlstmN1, "n1t": MlstmTcN1, "c2": LinAttnC2, "c3": GDeltaC3, "c4": LruC4, "c1": LinRecC1, "c5": TrainC5, "n2": MambaN2}


# ------------------------------------------------------------ clock sampling
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)
    from a background thread while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------ CPU arm
def time_cpu(workload_cls, steps, warmup, batch=None):
    """Times the oracle port on the host cores over a bounded sample of the
    workload (fewer sequences, same T / heads / widths)."""
    torch.set_num_threads(os.cpu_count() or 1)
    w = workload_cls(batch=batch or workload_cls.cpu_sample_batch)
    x = w.host_inputs()
    for _ in range(warmup):
        w.cpu_step(x)
    t0 = time.perf_counter()
    for _ in range(steps):
        w.cpu_step(x)
    dt = (time.perf_counter() - t0) / steps
    return w, dt


def bounded_cpu_batch(workload_cls, passes, limit_s=90.0):
    """Largest sample (in sequences) for which `passes` passes fit the time limit,
    from one calibration pass on a few sequences."""
    probe = min(4, workload_cls.cpu_sample_batch)
    _, dt = time_cpu(workload_cls, steps=1, warmup=1, batch=probe)
    per_seq = dt / probe
    return int(max(1, min(workload_cls.cpu_sample_batch, limit_s / (per_seq * max(passes, 1)))))


def cpu_baseline(workload_cls):
    w, dt = time_cpu(workload_cls, steps=2, warmup=1)
    return {"value": w.tokens() / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{w.B} of {workload_cls.B} sequences of the same workload, fp32 torch-CPU oracle port, "
                      f"{dt:.3f} s per pass"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    batch = bounded_cpu_batch(cls, args.steps + args.warmup)
    w, dt = time_cpu(cls, steps=args.steps, warmup=args.warmup, batch=batch)
    val = w.tokens() / dt
    base = {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{w.B} of {cls.B} sequences per step, fp32 torch-CPU oracle port (reference formulation)"}
    print(json.dumps({
        "impl": "reference", "metric": "tokens/s", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cls.name, "sample_batch": w.B, "note": "jax is not installable here; the timed code "
                   "is the CPU restatement of the reference's algorithm"},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ------------------------------------------------------------------ GPU arm
def to_device(x, dev):
    return {k: v.to(dev, non_blocking=True) for k, v in x.items()}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, 1590.0, "fallback"


def bind_to_gpu_numa_node(local):
    """Pins this rank's host threads (and hence its pinned staging buffers, first-touch) to the CPUs
    the kernel lists as local to its GPU's PCIe slot.  Read-only on the GPU side; returns a short
    description for the JSON line."""
    try:
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        dev = torch.cuda.get_device_properties(local).pci_device_id
        base = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0"
        with open(base + "/numa_node") as fh:
            node = int(fh.read().strip())
        with open(base + "/local_cpulist") as fh:
            cpulist = fh.read().strip()
        cpus = set()
        for part in cpulist.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed
        if target and target != allowed:
            os.sched_setaffinity(0, target)
            return f"numa node {node}: bound to {len(target)} of {len(allowed)} cpus"
        return f"numa node {node}: local cpus = all allowed cpus ({len(allowed)}), nothing to bind"
    except Exception as exc:   # no sysfs entry (virtualised PCI topology): leave the affinity alone
        return f"not bound ({type(exc).__name__})"


class Harness:
    """One process per GPU; times blocks of K steps between barriers, max over ranks."""

    def __init__(self, args):
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: memorax_b200 has no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.binding = bind_to_gpu_numa_node(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        from memorax_b200 import ops  # raises if libmxk.so is missing
        self.ops = ops

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if not self.dist:
            return ms
        t = torch.tensor([ms], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def input_sets(self, w, on_device):
        """Enough distinct input sets that a step never finds its inputs in the 126 MB L2."""
        where = self.dev if on_device else "cpu"
        first = w.host_inputs(seed_offset=1000 * self.rank, device=where)
        in_bytes = sum(v.numel() * v.element_size() for v in first.values())
        nsets = 1 if in_bytes > (1 << 30) else min(64, max(NSETS, -(-(512 << 20) // in_bytes)))
        sets = [to_device(first, self.dev)]
        for i in range(1, nsets):
            sets.append(to_device(w.host_inputs(seed_offset=1000 * self.rank + i, device=where), self.dev))
        torch.cuda.synchronize()
        return first, sets, in_bytes

    def time_workload(self, w, sets, steps, warmup, min_seconds):
        """Blocks of exactly `steps` steps, each bracketed by barrier + synchronize, repeated until at least
        `min_seconds` of device time have been measured; the reported block is the median one (max over
        ranks per block).  Returns (ms_per_step, per-phase ms of the median block, blocks, clock summary)."""
        ops, nsets = self.ops, len(sets)
        for i in range(max(warmup, 3)):
            w.step(sets[i % nsets], ops)
        self.barrier()
        graph = None
        if getattr(w, "use_graph", False):
            # launch-bound workload: up to 32 consecutive steps of a timed block are captured as ONE graph (rotating
            # over the input sets as the direct path does; outputs stay alive in the graph's pool), so that the
            # host's launch rate is not what gets measured; a block is steps // 32 replays plus the rest directly
            keep = []
            graph_steps = min(steps, 32)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(graph_steps):
                        keep.append(w.step(sets[i % nsets], ops))
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            self.barrier()
        blocks, phases, total = [], [], 0.0
        with ClockSampler(self.local) as clocks:
            while True:
                marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.barrier()
                t0.record()
                if graph:
                    for _ in range(steps // graph_steps):
                        graph.replay()
                    for i in range(steps % graph_steps):
                        w.step(sets[i % nsets], ops)
                else:
                    for i in range(steps):
                        w.step(sets[i % nsets], ops, marks[i])
                t1.record()
                self.barrier()
                ms = self.max_over_ranks(t0.elapsed_time(t1))
                blocks.append(ms)
                # marks: [0] after the first launch of a step (or before the only one), [1] after the last
                per_step = t0.elapsed_time(t1) / steps
                phases.append((per_step if graph else sum(a.elapsed_time(b) for a, b in marks) / steps, per_step))
                total += ms
                if total >= min_seconds * 1e3 or len(blocks) >= 400:
                    break
        order = sorted(range(len(blocks)), key=lambda i: blocks[i])
        mid = order[len(order) // 2]
        return blocks[mid] / steps, phases[mid][0], blocks, clocks.summary(), graph is not None

    def op_record(self, w, ms_per_step, dominant_ms, blocks, clocks, tokens_all_ranks):
        hbm_peak, tc_peak, kind = measured_peaks()
        rec = {"workload": w.name, "batch_per_gpu": w.B, "ms_per_step": ms_per_step,
               "tokens_per_s": tokens_all_ranks / (ms_per_step * 1e-3), "dtype": w.dtype,
               "blocks": len(blocks), "block_ms_min_med_max": [min(blocks), sorted(blocks)[len(blocks) // 2], max(blocks)],
               "clocks": clocks}
        if hasattr(w, "roofline"):
            rec["roofline"] = w.roofline(ms_per_step if getattr(w, "roofline_of_step", False) else dominant_ms)
            return rec
        alg = w.algorithmic_bytes()
        flops = w.algorithmic_flops()
        step_bytes, step_flops = sum(alg.values()), sum(flops.values())
        t = ms_per_step * 1e-3
        # whole step (all launches) against both roofs; the binding roof is the one with the larger floor time
        hbm_frac = step_bytes / t / 1e9 / hbm_peak
        tc_frac = step_flops / t / 1e12 / tc_peak
        dom_bytes = alg[w.dominant]
        achieved = dom_bytes / (dominant_ms * 1e-3) / 1e9
        rec["roofline"] = {
            "bound": "hbm" if step_bytes / hbm_peak / 1e9 >= step_flops / tc_peak / 1e12 else "tensor",
            "step": {"algorithmic_bytes": step_bytes, "algorithmic_flop": step_flops, "hbm_frac": hbm_frac,
                     "tensor_frac": tc_frac, "hbm_peak_gbs": hbm_peak, "tensor_peak_tflops": tc_peak},
            "kernel": w.dominant, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
            "peak_kind": f"of {kind}", "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dominant_ms,
            "tensor_frac_of_kernel": flops[w.dominant] / (dominant_ms * 1e-3) / 1e12 / tc_peak}
        if w.B == type(w).B:
            rec["roofline"]["traffic"] = w.dominant_traffic_bytes
        return rec

    def run_op(self, cls, batch, steps, warmup, min_seconds, on_device=True, graph=False):
        """Times one workload with device-generated inputs and frees everything afterwards.  ``graph``: replay the
        steps as CUDA graphs (for splits whose step is shorter than the host takes to enqueue it)."""
        w = cls(batch=batch)
        if graph:
            w.use_graph = True
        _, sets, in_bytes = self.input_sets(w, on_device)
        ms, dom_ms, blocks, clocks, graphed = self.time_workload(w, sets, steps, warmup, min_seconds)
        rec = self.op_record(w, ms, dom_ms, blocks, clocks, self.world * w.tokens())
        rec["l2"] = f"{len(sets)} input set(s) rotated, {in_bytes * len(sets) / 1e6:.0f} MB of inputs"
        rec["launch"] = "cuda graph replays of up to 32 steps each" if graphed else "direct"
        if hasattr(w, "variants"):
            rec["variants_ms"] = w.variants(sets[0], self.ops)
        if hasattr(w, "trainer"):
            w.trainer = None
        del sets, w
        torch.cuda.empty_cache()
        return rec


def run_gpu_arm(args):
    hz = Harness(args)
    rank, world, dev, ops = hz.rank, hz.world, hz.dev, hz.ops
    cls = WORKLOADS[args.workload]
    w = cls(batch=args.batch)
    host, sets, in_bytes = hz.input_sets(w, on_device=False)
    nsets = len(sets)
    ms_per_step, dominant_ms, blocks, clock_summary, graphed = hz.time_workload(w, sets, args.steps, args.warmup,
                                                                               args.min_seconds)
    value = world * w.tokens() / (ms_per_step * 1e-3)
    head = hz.op_record(w, ms_per_step, dominant_ms, blocks, clock_summary, world * w.tokens())

    # ---- end to end: host buffers in, host results out, through the same calls ----
    barrier = hz.barrier
    pinned_in = {k: v.pin_memory() for k, v in host.items()}
    # a streaming pipeline is a throughput measurement: 100 steps, so that filling and draining it (one step's
    # copy-in before the first copy-out, one copy-out after the last copy-in) weigh 1 % instead of 5 %
    outs = w.step(to_device(pinned_in, dev), ops)
    pinned_out = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True) for o in outs]
    h2d = sum(v.numel() * v.element_size() for v in pinned_in.values())
    d2h = sum(o.numel() * o.element_size() for o in pinned_out)
    if (args.e2e_mode or getattr(w, "e2e_mode", "plain")) == "stream":
        e2e_steps = 100 if h2d + d2h < (2 << 30) else 12   # a multi-gigabyte step takes a fifth of a second on the wire
    else:
        e2e_steps = max(3, min(args.steps, 20))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from memorax_b200.host import HostPipeline
    nslices = args.e2e_slices or getattr(w, "e2e_slices", 1)
    # "stream": consecutive steps overlap (copy-in of step i+1 under the copy-out of step i, at most three
    # steps in flight: one step of slack between the two copy directions); "graph": one CUDA-graph replay per step; "plain": call by call
    mode = args.e2e_mode or getattr(w, "e2e_mode", "plain")
    pipe = HostPipeline(lambda xs: w.step(xs, ops), w.B, dev, slices=nslices, graph=(mode == "graph"),
                        overlap_calls=3 if mode == "stream" else 1)
    for _ in range(pipe.overlap_calls):      # warm the three streams' allocator pools and every staging set
        pipe.run(pinned_in, pinned_out)
    pipe.wait()
    barrier()
    e0.record()
    host_t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pipe.run(pinned_in, pinned_out)
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / e2e_steps   # the host's share: enqueueing one step
    pipe.join()
    e1.record()
    barrier()
    e2e_ms = hz.max_over_ranks(e0.elapsed_time(e1))
    e2e_value = world * w.tokens() / (e2e_ms / e2e_steps * 1e-3)
    ops.check_status(dev)

    # ---- wire floor: the same bytes over PCIe, both directions at once, no kernels ----
    dev_in = to_device(pinned_in, dev)
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    s_up.wait_event(f0)
    s_down.wait_event(f0)
    for _ in range(e2e_steps):
        with torch.cuda.stream(s_up):
            for k, v in pinned_in.items():
                dev_in[k].copy_(v, non_blocking=True)
        with torch.cuda.stream(s_down):
            for dst, src in zip(pinned_out, outs):
                dst.copy_(src, non_blocking=True)
    torch.cuda.current_stream().wait_stream(s_up)
    torch.cuda.current_stream().wait_stream(s_down)
    f1.record()
    barrier()
    wire_ms = hz.max_over_ranks(f0.elapsed_time(f1)) / e2e_steps
    wire = {"value": world * w.tokens() / (wire_ms * 1e-3), "unit": "tokens/s", "ms_per_step": wire_ms,
            "h2d_gbs_per_gpu": h2d / wire_ms / 1e6, "d2h_gbs_per_gpu": d2h / wire_ms / 1e6,
            "what": "same pinned buffers copied in and out concurrently, no kernels: the PCIe bound of e2e"}
    del dev_in, outs, pipe, sets
    torch.cuda.empty_cache()

    # ---- every other op of the metric, and the strong-scaling split of the configs ----
    per_op, strong = {}, {}
    if args.ops:
        per_op[args.workload] = {k: head[k] for k in ("workload", "batch_per_gpu", "ms_per_step", "tokens_per_s",
                                                      "dtype", "blocks", "clocks", "roofline")}
        for name in ("c1", "c3", "c4", "c5", "a7", "n1", "n1t", "n2", "n3", "n4"):
            if name == args.workload:
                continue
            per_op[name] = hz.run_op(WORKLOADS[name], None, args.steps, args.warmup, args.min_seconds)
        for name in ("c2", "c3", "c4"):
            full = WORKLOADS[name].B
            if full % world:
                continue
            if world == 1:
                src = per_op[name]
                strong[name] = {"batch_per_gpu": full, "ms_per_step": src["ms_per_step"], "tokens_per_s": src["tokens_per_s"],
                                "note": "one GPU: the strong split is the whole config (same measurement as ops)"}
                continue
            # a split c2 step (two launches of a few tens of microseconds) is shorter than its Python enqueue
            rec = hz.run_op(WORKLOADS[name], full // world, args.steps, args.warmup, args.min_seconds, graph=(name == "c2"))
            rec["tokens_per_s"] = WORKLOADS[name].B * WORKLOADS[name].T / (rec["ms_per_step"] * 1e-3)
            strong[name] = {k: rec[k] for k in ("batch_per_gpu", "ms_per_step", "tokens_per_s", "blocks", "clocks", "launch")}
            strong[name]["config_batch"] = full

    if rank == 0:
        roof = head["roofline"]
        if "traffic" not in roof:
            roof["traffic"] = (w.dominant_traffic_bytes if args.batch is None else None)
        line = {
            "metric": "tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name, "batch_per_gpu": w.B, "T": w.T, "tokens_per_step_per_gpu": w.tokens(),
                       "l2": f"{nsets} input set(s) rotated, {in_bytes * nsets / 1e6:.0f} MB of inputs > 126 MB L2",
                       "sharding": "independent sequences per rank, no data-path collective",
                       "launch": "cuda graph replays of up to 32 steps each" if graphed else "direct",
                       "timing": f"{len(blocks)} blocks of {args.steps} steps (>= {args.min_seconds} s of device time), "
                                 "median block reported, max over ranks per block",
                       "block_ms_min_med_max": head["block_ms_min_med_max"]},
            "clocks": clock_summary,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "batch_slices_in_flight": nslices, "host_enqueue_ms_per_step": host_enqueue_ms,
                    "host_binding": hz.binding,
                    "wire_floor": wire,
                    "mode": {"stream": "three streams, copy-in of step i+1 overlaps copy-out of step i (three steps in flight)",
                             "graph": "cuda graph replay of the three-stream schedule",
                             "plain": "three streams, step by step"}[mode]},
            "gpu_launches": w.launches_per_step * args.steps * len(blocks),
            "roofline": roof,
        }
        if per_op:
            line["ops"] = per_op
            line["strong"] = strong
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(cls)
        print(json.dumps(line))
    if hz.dist:
        hz.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=None, help="override sequences per GPU (profiling only)")
    ap.add_argument("--e2e-slices", type=int, default=None, help="override the batch slices of the host pipeline")
    ap.add_argument("--e2e-mode", choices=["stream", "graph", "plain"], default=None, help="host pipeline mode for the e2e figure")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="repeat the block of --steps steps until this much device time has been measured")
    ap.add_argument("--ops", dest="ops", action="store_true", default=None,
                    help="also time every other op of the metric (c1, c3, c4, c5) and the strong-scaling split; "
                         "default: on when --workload and --batch are not given")
    ap.add_argument("--no-ops", dest="ops", action="store_false")
    args = ap.parse_args()
    if args.ops is None:
        args.ops = args.workload is None and args.batch is None
    args.workload = args.workload or "c2"
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
