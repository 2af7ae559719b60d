"""Vision-Mamba2 "tiny" forward network around the SSD operator (benchmark configuration 4).

A plain stack, as the benchmark definition describes it: patch-16 embedding of a 3 x 1024 x 1024 image into
4096 tokens of width 192, then 12 Mamba-2 blocks, each

    RMSNorm -> in_proj (z, x, B, C, dt) -> depthwise causal conv1d (width 4) + SiLU on (x, B, C)
            -> SSD (expand 2 -> d_inner 384, headdim 64 -> 6 heads, d_state 64, 1 group, chunk 64,
                    D skip, dt_bias, softplus)
            -> gated RMSNorm (y * silu(z)) -> out_proj, with a residual connection,

and a mean-pool + linear head.  The reference's own demo network (mamba_torch/vmamba2_network.py) is a
different, hierarchical four-direction model; what is kept from it is the integration pattern of its
``SsdCore`` (:31-85): the block calls one injectable SSD function with the ``mamba2_ssd_fwd`` signature.
Projections, convolution and norms run on PyTorch / cuBLAS; only the SSD is this library's kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VisionMamba2Config:
    image_size: int = 1024
    patch: int = 16
    d_model: int = 192
    depth: int = 12
    expand: int = 2
    headdim: int = 64
    d_state: int = 64
    ngroups: int = 1
    d_conv: int = 4
    chunk_size: int = 64
    num_classes: int = 1000

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def nheads(self) -> int:
        return self.d_inner // self.headdim

    @property
    def tokens(self) -> int:
        return (self.image_size // self.patch) ** 2


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, gate=None):
        if gate is not None:
            x = x * F.silu(gate)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


class Mamba2Block(nn.Module):
    def __init__(self, cfg: VisionMamba2Config, ssd_fn: Callable):
        super().__init__()
        self.cfg = cfg
        self.ssd_fn = ssd_fn
        d_in, g, n, h = cfg.d_inner, cfg.ngroups, cfg.d_state, cfg.nheads
        self.norm = RMSNorm(cfg.d_model)
        self.in_proj = nn.Linear(cfg.d_model, 2 * d_in + 2 * g * n + h, bias=False)
        conv_dim = d_in + 2 * g * n
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, cfg.d_conv, groups=conv_dim, padding=cfg.d_conv - 1)
        self.A_log = nn.Parameter(torch.log(torch.empty(h).uniform_(1.0, 16.0)))
        self.D = nn.Parameter(torch.ones(h))
        dt = torch.exp(torch.rand(h) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.out_norm = RMSNorm(d_in)
        self.out_proj = nn.Linear(d_in, cfg.d_model, bias=False)

    def forward(self, u):
        cfg = self.cfg
        b, l, _ = u.shape
        d_in, g, n, h, p = cfg.d_inner, cfg.ngroups, cfg.d_state, cfg.nheads, cfg.headdim
        zxbcdt = self.in_proj(self.norm(u))
        z, xbc, dt = torch.split(zxbcdt, [d_in, d_in + 2 * g * n, h], dim=-1)
        xbc = F.silu(self.conv1d(xbc.transpose(1, 2))[..., :l].transpose(1, 2))
        x, bm, cm = torch.split(xbc, [d_in, g * n, g * n], dim=-1)
        y = self.ssd_fn(x.reshape(b, l, h, p).contiguous(), dt.contiguous(), -torch.exp(self.A_log),
                        bm.reshape(b, l, g, n).contiguous(), cm.reshape(b, l, g, n).contiguous(), cfg.chunk_size,
                        D=self.D, dt_bias=self.dt_bias, dt_softplus=True)
        y = self.out_norm(y.reshape(b, l, d_in), gate=z)
        return u + self.out_proj(y)


class VisionMamba2(nn.Module):
    """``ssd_fn`` defaults to this package's ``mamba2_ssd_fwd``; tests pass a checker with the same signature."""

    def __init__(self, cfg: Optional[VisionMamba2Config] = None, ssd_fn: Optional[Callable] = None):
        super().__init__()
        self.cfg = cfg or VisionMamba2Config()
        if ssd_fn is None:
            from .mamba2 import mamba2_ssd_fwd as ssd_fn
        c = self.cfg
        self.patch_embed = nn.Conv2d(3, c.d_model, c.patch, stride=c.patch)
        self.blocks = nn.ModuleList([Mamba2Block(c, ssd_fn) for _ in range(c.depth)])
        self.norm = RMSNorm(c.d_model)
        self.head = nn.Linear(c.d_model, c.num_classes)

    def forward(self, images):
        t = self.patch_embed(images).flatten(2).transpose(1, 2)  # [B, tokens, d_model]
        for blk in self.blocks:
            t = blk(t)
        return self.head(self.norm(t).mean(dim=1))
