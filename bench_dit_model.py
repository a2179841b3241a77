"""Measurement harness only (not part of the package): a DiT-MoE backbone with
the tensor flow of the reference's ``models.py:464-706`` around the dice_b200
MoE blocks, so that ``bench.py`` can report the latency of one sampling step of
the full model next to the MoE-block throughput.

Everything except the MoE block is plain PyTorch in bf16 (patch embedding,
timestep / label embedding, adaLN-Zero modulation, LayerNorm, attention with
q/k LayerNorm through ``scaled_dot_product_attention``, final layer); weights
are random.  The reference's sampler doubles the batch for classifier-free
guidance and takes one Euler step per model call
(``diffusion/rectified_flow.py:107-126``); that is what ``sampling_step`` does.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def _modulate(x, shift, scale):
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class _Attention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.qkv = nn.Linear(dim, 3 * dim, bias=True)
        self.q_norm = nn.LayerNorm(self.head_dim, eps=1e-6)
        self.k_norm = nn.LayerNorm(self.head_dim, eps=1e-6)
        self.proj = nn.Linear(dim, dim, bias=True)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, self.head_dim).unbind(dim=2)
        q, k = self.q_norm(q), self.k_norm(k)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return self.proj(o.transpose(1, 2).reshape(b, s, d))


class _Block(nn.Module):
    def __init__(self, dim, heads, moe):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.attn = _Attention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.moe = moe
        self.ada = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim, bias=True))
        self.fused_glue = True

    def forward(self, x, c):
        s1, c1, g1, s2, c2, g2 = self.ada(c).chunk(6, dim=1)
        x = x + g1.unsqueeze(1) * self.attn(_modulate(self.norm1(x), s1, c1))
        if self.fused_glue:  # LayerNorm + modulation and the gated residual inside the MoE block's kernels
            return self.moe.forward_with_glue(x, s2, c2, g2, eps=self.norm2.eps)
        return x + g2.unsqueeze(1) * self.moe(_modulate(self.norm2(x), s2, c2))


class DiTBackbone(nn.Module):
    """``moe_blocks``: one dice_b200.SparseMoeBlock per layer (kept by reference)."""

    def __init__(self, moe_blocks, hidden, heads=16, latent=32, patch=2, channels=4, classes=1000):
        super().__init__()
        self.patch, self.channels, self.grid = patch, channels, latent // patch
        self.x_embed = nn.Conv2d(channels, hidden, patch, patch)
        self.pos = nn.Parameter(torch.randn(1, self.grid * self.grid, hidden) * 0.02)
        self.t_mlp = nn.Sequential(nn.Linear(256, hidden), nn.SiLU(), nn.Linear(hidden, hidden))
        self.y_embed = nn.Embedding(classes + 1, hidden)
        self.blocks = nn.ModuleList([_Block(hidden, heads, m) for m in moe_blocks])
        self.final_norm = nn.LayerNorm(hidden, elementwise_affine=False, eps=1e-6)
        self.final_ada = nn.Sequential(nn.SiLU(), nn.Linear(hidden, 2 * hidden))
        self.final = nn.Linear(hidden, patch * patch * channels * 2)

    def set_fused_glue(self, flag: bool) -> None:
        for blk in self.blocks:
            blk.fused_glue = flag

    def _t_embed(self, t):
        half = 128
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
        args = t[:, None].float() * freqs[None]
        return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)

    def forward(self, z, t, y):
        dt = self.pos.dtype
        x = self.x_embed(z.to(dt)).flatten(2).transpose(1, 2) + self.pos
        c = self.t_mlp(self._t_embed(t).to(dt)) + self.y_embed(y)
        for blk in self.blocks:
            x = blk(x, c)
        shift, scale = self.final_ada(c).chunk(2, dim=1)
        x = self.final(_modulate(self.final_norm(x), shift, scale))
        b, p, g = x.shape[0], self.patch, self.grid
        x = x.view(b, g, g, p, p, 2 * self.channels).permute(0, 5, 1, 3, 2, 4)
        return x.reshape(b, 2 * self.channels, g * p, g * p)

    @torch.no_grad()
    def sampling_step(self, z, cond, null_cond, t, dt, cfg=1.5):
        """One rectified-flow Euler step with classifier-free guidance (batch doubled)."""
        b = z.shape[0]
        v = self(torch.cat([z, z]), torch.full((2 * b,), t, device=z.device), torch.cat([cond, null_cond]))
        vc, vu = v[:b, : self.channels], v[b:, : self.channels]
        return z - dt * (vu + cfg * (vc - vu)).to(z.dtype)
