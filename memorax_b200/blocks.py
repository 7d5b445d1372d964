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
        return self.module(self.norm(inputs), done, initial_carry)


class GatedResidual(nn.Module):
    def __init__(self, module, features):
        super().__init__()
        self.module, self.gate = module, nn.Linear(features, features)

    def forward(self, inputs, done=None, initial_carry=None):
        carry, out = self.module(inputs, done, initial_carry)
        return carry, inputs + torch.sigmoid(self.gate(inputs)) * out


class FFN(nn.Module):
    def __init__(self, features, expansion_factor=4):
        super().__init__()
        self.up, self.down = nn.Linear(features, features * expansion_factor), nn.Linear(features * expansion_factor, features)

    def forward(self, inputs, done=None, initial_carry=None):
        return None, self.down(torch.nn.functional.gelu(self.up(inputs)))


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

    def __init__(self, obs_dim=128, d_model=512, num_heads=4, head_dim=128, layers=4):
        super().__init__()
        self.embed = nn.Linear(obs_dim, d_model)
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
    that the gradient all-reduce is one NCCL call and Adam one kernel launch."""

    def __init__(self, model, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, process_group=None, world_size=1):
        self.model, self.lr, self.betas, self.eps = model, lr, betas, eps
        self.group, self.world = process_group, world_size
        params = [p for p in model.parameters()]
        total = sum(p.numel() for p in params)
        padded = (total + 7) // 8 * 8
        dev = params[0].device
        self.flat = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        self.flat_grad = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        off = 0
        for p in params:
            n = p.numel()
            self.flat[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat[off:off + n].view_as(p)
            p.grad = self.flat_grad[off:off + n].view_as(p)
            off += n
        self.m = torch.zeros(padded, dtype=torch.float32, device=dev)
        self.v = torch.zeros(padded, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.num_params = total

    def step(self, obs, done, target):
        self.flat_grad.zero_()
        value = self.model(obs, done)
        loss = 0.5 * (value.float() - target).square().mean()     # VNetwork.loss, heads.py:114-117
        loss.backward()
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(self.flat_grad, group=self.group)
        self.step_count += 1
        ops.adam_step(self.flat, self.flat_grad, self.m, self.v, self.step_count, self.lr, self.betas, self.eps,
                      grad_scale=1.0 / self.world)
        return loss.detach()
