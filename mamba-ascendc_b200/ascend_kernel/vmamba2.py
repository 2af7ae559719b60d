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
The projections run on PyTorch / cuBLAS.  In inference on CUDA (no gradients) the norms and the convolution run
as this library's fused forward kernels (``ssd_block_rmsnorm_fwd``, ``ssd_block_conv_silu_fwd``: one pass each,
writing the SSD's inputs in place of the framework's split / transpose / copy chain); with gradients enabled, on
CPU, or when this file is loaded without the package, the same steps run as framework operations.
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


def _kernels():
    """The C-ABI binding, or None when this module was loaded on its own (no package, no CUDA library)."""
    try:
        from . import _capi
    except (ImportError, ValueError):
        return None
    return _capi


def _fast(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.float32 and not torch.is_grad_enabled() and _kernels() is not None


def _rmsnorm_kernel(x2d: torch.Tensor, x_stride: int, z, z_stride: int, weight: torch.Tensor, eps: float, rows: int,
                    d: int) -> torch.Tensor:
    capi = _kernels()
    out = torch.empty(rows, d, device=weight.device, dtype=torch.float32)
    capi.check(capi.lib.ssd_block_rmsnorm_fwd(x2d, x_stride, z, z_stride, weight.data_ptr(), out.data_ptr(), rows, d,
                                              eps, torch.cuda.current_stream().cuda_stream), "vmamba2_rmsnorm")
    return out


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, gate=None):
        if _fast(x) and x.is_contiguous() and gate is None and x.shape[-1] <= 512:
            rows, d = x.numel() // x.shape[-1], x.shape[-1]
            return _rmsnorm_kernel(x.data_ptr(), d, None, 0, self.weight, self.eps, rows, d).view(x.shape)
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
        if _fast(zxbcdt) and zxbcdt.is_contiguous() and cfg.d_conv == 4 and d_in <= 512:
            return u + self.out_proj(self._fused_inner(zxbcdt, b, l))
        z, xbc, dt = torch.split(zxbcdt, [d_in, d_in + 2 * g * n, h], dim=-1)
        xbc = F.silu(self.conv1d(xbc.transpose(1, 2))[..., :l].transpose(1, 2))
        x, bm, cm = torch.split(xbc, [d_in, g * n, g * n], dim=-1)
        y = self.ssd_fn(x.reshape(b, l, h, p).contiguous(), dt.contiguous(), -torch.exp(self.A_log),
                        bm.reshape(b, l, g, n).contiguous(), cm.reshape(b, l, g, n).contiguous(), cfg.chunk_size,
                        D=self.D, dt_bias=self.dt_bias, dt_softplus=True)
        y = self.out_norm(y.reshape(b, l, d_in), gate=z)
        return u + self.out_proj(y)


    def _fused_inner(self, zxbcdt: torch.Tensor, b: int, l: int) -> torch.Tensor:
        """conv1d + SiLU + split, SSD, gated norm on the fused kernels; z, xBC and dt are read as column slices of
        the in_proj output where they lie."""
        cfg, capi = self.cfg, _kernels()
        d_in, g, n, h, p = cfg.d_inner, cfg.ngroups, cfg.d_state, cfg.nheads, cfg.headdim
        width = zxbcdt.shape[-1]
        dev = zxbcdt.device
        x = torch.empty(b, l, h, p, device=dev, dtype=torch.float32)
        bm = torch.empty(b, l, g, n, device=dev, dtype=torch.float32)
        cm = torch.empty(b, l, g, n, device=dev, dtype=torch.float32)
        w = self.conv1d.weight.view(-1, cfg.d_conv)
        bias = self.conv1d.bias
        capi.check(capi.lib.ssd_block_conv_silu_fwd(zxbcdt.data_ptr() + 4 * d_in, width, w.data_ptr(),
                                                    None if bias is None else bias.data_ptr(), x.data_ptr(),
                                                    bm.data_ptr(), cm.data_ptr(), b, l, d_in, g * n,
                                                    torch.cuda.current_stream().cuda_stream), "vmamba2_conv1d")
        dt = zxbcdt[..., d_in + d_in + 2 * g * n:].contiguous()
        y = self.ssd_fn(x, dt, -torch.exp(self.A_log), bm, cm, cfg.chunk_size, D=self.D, dt_bias=self.dt_bias,
                        dt_softplus=True)
        y = y.contiguous()
        return _rmsnorm_kernel(y.data_ptr(), d_in, zxbcdt.data_ptr(), width, self.out_norm.weight, self.out_norm.eps,
                               b * l, d_in).view(b, l, d_in)


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
        # [B, tokens, d_model], token-major in memory (a transposed view would hand its layout on to every
        # residual sum after it)
        t = self.patch_embed(images).flatten(2).transpose(1, 2).contiguous()
        for blk in self.blocks:
            t = blk(t)
        return self.head(self.norm(t).mean(dim=1))
