"""Shapes beyond what the tile kernels take, reduced to calls the kernels do take.

The CUDA tile kernels handle headdim P = 64, state size N = 64 (forward and backward) or N = 128 (forward
only) and a sequence length that is a multiple of 128.  The reference API accepts any shape: its generic
kernel covers what its Cube kernels do not (``mamba2_ssd_fwd.cpp:49-136``; shape matrix
``benchmarks/mamba2_shape_matrix.py:129-190``: P and N from 8 to 128, ragged L).  ``run_general`` maps every
such call onto kernel calls with exact algebra, using differentiable torch operations only, so autograd
returns the gradients of the original tensors:

* sequence: zero-pad to the tile; padded tokens take no step (``valid_len``), as the reference pads to a
  chunk multiple (``ssd_reference.py:250-261``);
* headdim: zero-pad P to a multiple of 64 (zero channels of x give zero channels of out and zero rows of the
  state); a head with P = 64 v is v heads of 64 channels that share dt, A and the head's group;
* state size: zero-pad N to a multiple of 64 (zero columns of B and C change neither C B^T nor the other
  state columns); the SSD is a sum over the state index, so N = 64 m is the sum of m calls on 64-column
  blocks of B and C, and the final state is their concatenation.  Without gradients a 128-column block goes
  to the N = 128 forward kernels in one call.

``core(x, dt, A, B, C, initial_states, dt_bias, valid_len) -> (out, final_state or None)`` is the fixed-shape
call.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.nn.functional as F

TILE = 128  # tokens per kernel tile
LANE = 64   # headdim of the kernels, and their basic state block


def _ceil_to(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def run_general(core: Callable, x, dt, A, B, C, initial_states: Optional[torch.Tensor],
                dt_bias: Optional[torch.Tensor], needs_grad: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out [B,L,H,P], final_state [B,H,P,N]) for arbitrary L, P, N."""
    b, l, h, p = x.shape
    n = B.shape[3]
    init = initial_states

    # ---- sequence
    pad_l = (-l) % TILE
    if pad_l:
        x = F.pad(x, (0, 0, 0, 0, 0, pad_l))
        dt = F.pad(dt, (0, 0, 0, pad_l))
        B = F.pad(B, (0, 0, 0, 0, 0, pad_l))
        C = F.pad(C, (0, 0, 0, 0, 0, pad_l))
    valid = l if pad_l else 0
    lp = l + pad_l

    # ---- headdim: pad to a multiple of 64, then one virtual head per 64 channels
    p2 = _ceil_to(p, LANE)
    if p2 != p:
        x = F.pad(x, (0, p2 - p))
        if init is not None:
            init = F.pad(init, (0, 0, 0, p2 - p))
    v = p2 // LANE
    if v > 1:
        x = x.reshape(b, lp, h * v, LANE)
        dt = dt.repeat_interleave(v, dim=2)
        A = A.repeat_interleave(v)
        if dt_bias is not None:
            dt_bias = dt_bias.repeat_interleave(v)
        if init is not None:
            init = init.reshape(b, h * v, LANE, n)

    # ---- state size: pad to a multiple of 64, then blocks of columns
    n2 = _ceil_to(n, LANE)
    if n2 != n:
        B = F.pad(B, (0, n2 - n))
        C = F.pad(C, (0, n2 - n))
        if init is not None:
            init = F.pad(init, (0, n2 - n))
    block = 2 * LANE if (not needs_grad and n2 % (2 * LANE) == 0) else LANE
    if n2 == block:
        out, final = core(x.contiguous(), dt.contiguous(), A.contiguous(), B.contiguous(), C.contiguous(),
                          None if init is None else init.contiguous(), dt_bias, valid)
    else:
        out, finals = None, []
        for c0 in range(0, n2, block):
            o, f = core(x.contiguous(), dt.contiguous(), A.contiguous(), B[..., c0:c0 + block].contiguous(),
                        C[..., c0:c0 + block].contiguous(),
                        None if init is None else init[..., c0:c0 + block].contiguous(), dt_bias, valid)
            out = o if out is None else out + o
            finals.append(f)
        final = None if finals[0] is None else torch.cat(finals, dim=-1)

    # ---- back to the caller's shapes
    if v > 1:
        out = out.reshape(b, lp, h, p2)
    if pad_l or p2 != p:
        out = out[:, :l, :, :p]
    if final is not None:
        if v > 1:
            final = final.reshape(b, h, p2, n2)
        if p2 != p or n2 != n:
            final = final[:, :, :p, :n]
        final = final.contiguous()
    return out.contiguous(), final
