"""Minimal mirrors of the reference's composition blocks, only as far as the
training-step benchmark needs them: ``GatedResidual`` (x + sigmoid(Dense(x)) *
module(x), blocks/residual.py:33-63), ``PreNorm`` (LayerNorm before the module,
blocks/normalization.py:10-35), ``FFN`` (Dense-gelu-Dense, blocks/ffn.py:11-50)
and ``Stack`` (blocks/stack.py:33-60), with the reference's
``(inputs, done, initial_carry) -> (carry, outputs)`` block signature, plus the
flat-buffer trainer that runs forward, backward, the gradient all-reduce and
the fused Adam kernel."""
from __future__ import annotations

import torch
from torch import nn

from . import ops
from .memoroid import DeltaNetCell, Memoroid


class PreNorm(nn.Module):
    def __init__(self, module, features):
        super().__init__()
        self.module, self.norm = module, nn.LayerNorm(features)

    def forward(self, inputs, done=None, initial_carry=None):
        normed = ops.layer_norm(inputs, self.norm.weight, self.norm.bias, self.norm.eps)
        return self.module(normed, done, initial_carry)


class Dense(nn.Linear):
    """``nn.Linear`` whose bias gradient is this library's fixed-order column sum (``ops.dense``)."""

    def forward(self, x):
        return ops.dense(x, self.weight, self.bias)


class GatedResidual(nn.Module):
    def __init__(self, module, features):
        super().__init__()
        self.module, self.gate = module, Dense(features, features)

    def forward(self, inputs, done=None, initial_carry=None):
        carry, out = self.module(inputs, done, initial_carry)
        return carry, ops.gated_residual(inputs, self.gate(inputs), out)


class FFN(nn.Module):
    def __init__(self, features, expansion_factor=4):
        super().__init__()
        self.up, self.down = Dense(features, features * expansion_factor), Dense(features * expansion_factor, features)

    def forward(self, inputs, done=None, initial_carry=None):
        return None, self.down(ops.gelu(self.up(inputs)))


class Stack(nn.Module):
    def __init__(self, blocks):
        super().__init__()
        self.blocks = nn.ModuleList(blocks)

    def forward(self, inputs, done=None, initial_carry=None):
        carries, x = [], inputs
        initial_carry = initial_carry or (None,) * len(self.blocks)
        for block, carry in zip(self.blocks, initial_carry):
            c, x = block(x, done, carry)
            carries.append(c)
        return tuple(carries), x


class GTrXLStyleValueNet(nn.Module):
    """Dense(obs -> d_model) -> [GatedResidual(PreNorm(mixer)), GatedResidual(PreNorm(FFN))] x layers
    -> Dense(d_model -> 1); the reference's "GTrXL-style" composition
    (README.md:119-124) with the attention block replaced by the delta-rule mixer."""

    def __init__(self, obs_dim=128, d_model=512, num_heads=8, head_dim=64, layers=4):
        super().__init__()
        self.embed = Dense(obs_dim, d_model)
        blocks = []
        for _ in range(layers):
            mixer = Memoroid(DeltaNetCell(features=d_model, head_dim=head_dim, num_heads=num_heads))
            blocks += [GatedResidual(PreNorm(mixer, d_model), d_model), GatedResidual(PreNorm(FFN(d_model), d_model), d_model)]
        self.torso = Stack(blocks)
        self.head = nn.Linear(d_model, 1)

    def forward(self, obs, done):
        _, x = self.torso(self.embed(obs), done)
        return self.head(x).squeeze(-1)


class FlatAdamTrainer:
    """Keeps every parameter (bf16) and gradient as a view into one flat buffer so
    that Adam is one kernel launch and the gradient all-reduce works on contiguous
    ranges.  The update itself is applied to an fp32 master copy (optax.adam on the
    reference's fp32 params); the bf16 buffer the model computes with is its rounding,
    rewritten by the same kernel -- a step of lr = 3e-4 is far below a bf16 ulp at |p| = 1.

    The flat gradient is cut into one bucket per top-level block (embedding, each torso block,
    head).  Parameters enter the backward pass without a ``.grad``, so autograd hands over each
    gradient tensor as it is (no add kernel per parameter, no zeroing of the flat buffer); a
    gradient hook copies a bucket's gradients into the flat buffer with one multi-tensor copy the
    moment the last of them has arrived and, with more than one rank, launches that bucket's
    all-reduce, which runs on NCCL's stream underneath the rest of the backward pass; the step
    waits for all buckets before the Adam kernel."""

    def __init__(self, model, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, process_group=None, world_size=1,
                 overlap_allreduce=True):
        self.model, self.lr, self.betas, self.eps = model, lr, betas, eps
        self.group, self.world = process_group, world_size
        params = [p for p in model.parameters()]
        total = sum(p.numel() for p in params)
        padded = (total + 7) // 8 * 8
        dev = params[0].device
        self.flat = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        self.flat_grad = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        off = 0
        offsets = {}
        for p in params:
            n = p.numel()
            self.flat[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat[off:off + n].view_as(p)
            offsets[p] = (off, off + n)
            off += n
        self.master = self.flat.float()
        self.m = torch.zeros(padded, dtype=torch.float32, device=dev)
        self.v = torch.zeros(padded, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.check_every = 16
        self.num_params = total
        # ---- gradient buckets: contiguous ranges of the flat buffer, one per top-level block
        self.buckets = []          # (lo, hi, number of parameters)
        self._bucket_params = []   # per bucket: (parameters, their views into the flat gradient)
        self._pending, self._handles = [], []
        self._params = params
        self._reduce_in_hooks = world_size > 1 and overlap_allreduce
        for child in self._top_level_blocks(model):
            ps = [p for p in child.parameters()]
            if not ps:
                continue
            lo, hi = min(offsets[p][0] for p in ps), max(offsets[p][1] for p in ps)
            index = len(self.buckets)
            self.buckets.append((lo, hi, len(ps)))
            self._bucket_params.append((ps, [self.flat_grad[offsets[p][0]:offsets[p][1]].view_as(p) for p in ps]))
            for p in ps:
                p.register_post_accumulate_grad_hook(self._make_hook(index))
        covered = sorted((lo, hi) for lo, hi, _ in self.buckets)
        assert covered[0][0] == 0 and covered[-1][1] == total and all(
            a[1] == b[0] for a, b in zip(covered, covered[1:])), "buckets must tile the flat gradient"

    @staticmethod
    def _top_level_blocks(model):
        for child in model.children():
            if isinstance(child, Stack):
                yield from child.blocks
            else:
                yield child

    def _make_hook(self, index):
        def hook(_param):
            self._pending[index] -= 1
            if self._pending[index] == 0:
                ps, views = self._bucket_params[index]
                torch._foreach_copy_(views, [p.grad for p in ps])
                for p in ps:
                    p.grad = None
                if self._reduce_in_hooks:
                    import torch.distributed as dist
                    lo, hi, _ = self.buckets[index]
                    self._handles.append(dist.all_reduce(self.flat_grad[lo:hi], group=self.group, async_op=True))
        return hook

    def step(self, obs, done, target):
        for p in self._params:
            p.grad = None
        self._pending = [n for _, _, n in self.buckets]
        self._handles = []
        value = self.model(obs, done)
        loss = 0.5 * (value.float() - target).square().mean()     # VNetwork.loss, heads.py:114-117
        loss.backward()
        assert not any(self._pending), "a gradient bucket never filled (a parameter received no gradient)"
        if self.world > 1:
            if self._reduce_in_hooks:
                for handle in self._handles:
                    handle.wait()
                assert len(self._handles) == len(self.buckets), "a gradient bucket was never reduced"
            else:
                import torch.distributed as dist
                dist.all_reduce(self.flat_grad, group=self.group)
        self.step_count += 1
        ops.adam_step(self.flat, self.flat_grad, self.m, self.v, self.step_count, self.lr, self.betas, self.eps,
                      grad_scale=1.0 / self.world, master=self.master)
        if self.step_count % self.check_every == 0:
            ops.check_status(self.flat.device)   # a bounded wait that gave up inside the mixer kernels
        return loss.detach()
