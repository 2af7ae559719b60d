"""Multi-GPU use of the SSD path: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-device (no distributed code in its tree); these helpers are the B200 additions.

* Head-block sharding (default).  Rank r owns heads ``[r*H/R, (r+1)*H/R)`` and the groups that go with
  them.  out, final state, dx, ddt, dA (per head) and dB, dC (per group) are then rank-local: there is no
  collective on the data path.  ``gather=True`` only assembles full tensors for callers that want them.
* Sequence parallel (optional).  Rank r owns ``L/R`` consecutive tokens.  Only the ``[B,H,P,N]`` boundary
  state crosses ranks, and dA, which sums over the sequence, is all-reduced.  Two forms of the exchange:
  "chain" -- forward the state travels r -> r+1 (send / recv), backward its gradient travels r+1 -> r, each
  rank waiting for its neighbour; "allgather" -- the recurrence is linear, so every rank first computes
  what it would hand on from a zero start together with its total decay, ONE all_gather makes these known
  everywhere, and each rank folds its predecessors' (backward: successors') contributions locally; no rank
  waits for another's recurrence.  Either way the state is received into this rank's own memory before any
  kernel reads it.

``op`` is the local SSD call (default: ``ascend_kernel.mamba2_ssd_fwd``); the CPU tests pass a checker
implementation so that the exchange logic runs under the gloo backend without a GPU.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_block(rank: int, world: int, nheads: int, ngroups: int) -> Tuple[int, int, int, int]:
    """(h0, h1, g0, g1): the heads and groups rank ``rank`` owns.  Blocks are aligned to groups."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of size {world}")
    if nheads % ngroups != 0:
        raise ValueError("nheads must be divisible by ngroups")
    if ngroups % world != 0:
        raise ValueError(f"head-block sharding needs ngroups ({ngroups}) divisible by the number of ranks ({world})")
    gper = ngroups // world
    hper = nheads // world
    return rank * hper, (rank + 1) * hper, rank * gper, (rank + 1) * gper


def shard_by_heads(x, dt, A, B, C, rank: int, world: int):
    """Contiguous local slices of the five inputs for ``rank``."""
    h0, h1, g0, g1 = head_block(rank, world, x.shape[2], B.shape[2])
    return (x[:, :, h0:h1].contiguous(), dt[:, :, h0:h1].contiguous(), A[h0:h1].contiguous(),
            B[:, :, g0:g1].contiguous(), C[:, :, g0:g1].contiguous())


def _default_op() -> Callable:
    from .mamba2 import mamba2_ssd_fwd

    return mamba2_ssd_fwd


def mamba2_ssd_fwd_head_sharded(x, dt, A, B, C, chunk_size: int, *, dt_softplus: bool = False,
                                group: Optional[dist.ProcessGroup] = None, gather: bool = False,
                                op: Optional[Callable] = None):
    """Run this rank's head block of the full problem.  Returns (out, final_state): local blocks, or with
    ``gather=True`` the full tensors assembled with all_gather (not differentiable; for inspection)."""
    op = op or _default_op()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    xs, dts, As, Bs, Cs = shard_by_heads(x, dt, A, B, C, rank, world)
    out, final = op(xs, dts, As, Bs, Cs, chunk_size, dt_softplus=dt_softplus, return_final_state=True)
    if not gather:
        return out, final
    outs = [torch.empty_like(out) for _ in range(world)]
    finals = [torch.empty_like(final) for _ in range(world)]
    dist.all_gather(outs, out.detach().contiguous(), group=group)
    dist.all_gather(finals, final.detach().contiguous(), group=group)
    return torch.cat(outs, dim=2), torch.cat(finals, dim=1)


# ----------------------------------------------------------------------------- sequence parallel
class _RecvState(torch.autograd.Function):
    """Forward: receive the boundary state from the previous rank.  Backward: send its gradient back."""

    @staticmethod
    def forward(ctx, anchor, shape, dtype, device, group, prev):
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, src=dist.get_global_rank(group, prev) if group is not None else prev, group=group)
        ctx.group, ctx.prev = group, prev
        return buf

    @staticmethod
    def backward(ctx, grad):
        dst = dist.get_global_rank(ctx.group, ctx.prev) if ctx.group is not None else ctx.prev
        dist.send(grad.contiguous(), dst=dst, group=ctx.group)
        return torch.zeros(()), None, None, None, None, None


class _SendState(torch.autograd.Function):
    """Forward: send this rank's final state to the next rank.  Backward: receive its gradient."""

    @staticmethod
    def forward(ctx, state, group, nxt):
        dst = dist.get_global_rank(group, nxt) if group is not None else nxt
        dist.send(state.detach().contiguous(), dst=dst, group=group)
        ctx.group, ctx.nxt = group, nxt
        ctx.meta = (state.shape, state.dtype, state.device)
        return state.new_zeros(())

    @staticmethod
    def backward(ctx, _grad_token):
        shape, dtype, device = ctx.meta
        buf = torch.empty(shape, dtype=dtype, device=device)
        src = dist.get_global_rank(ctx.group, ctx.nxt) if ctx.group is not None else ctx.nxt
        dist.recv(buf, src=src, group=ctx.group)
        return buf, None, None


class _Attach(torch.autograd.Function):
    """Identity on ``out`` that also makes the backward pass visit ``token`` (the send above)."""

    @staticmethod
    def forward(ctx, out, token):
        return out.view_as(out)

    @staticmethod
    def backward(ctx, grad):
        return grad, torch.zeros((), dtype=grad.dtype, device=grad.device)


class _SumGradAcrossRanks(torch.autograd.Function):
    """Identity whose gradient is summed over the ranks (A is shared by every token block)."""

    @staticmethod
    def forward(ctx, a, group):
        ctx.group = group
        return a.view_as(a)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous().clone()
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return grad, None


# ---- the all-gather form
def _all_gather(t: torch.Tensor, group) -> list:
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return parts


def fold_inflow(rank: int, finals, log_decays):
    """State entering rank ``rank``: s_0 = 0, s_{j+1} = exp(log_decay_j) * s_j + final0_j over the ranks before
    it (``finals[j]`` [B,H,P,N] = what rank j hands on from a zero start, ``log_decays[j]`` [B,H])."""
    s = None
    for j in range(rank):
        s = finals[j] if s is None else torch.exp(log_decays[j])[..., None, None] * s + finals[j]
    return s


def fold_outflow(rank: int, world: int, d_initials, log_decays):
    """Gradient arriving at rank ``rank``'s final state from the ranks after it: g_{R-1} = 0,
    g_{j-1} = d_initial0_j + exp(log_decay_j) * g_j (``d_initials[j]`` = what rank j hands back when nothing
    comes in from its own successors)."""
    g = None
    for j in range(world - 1, rank, -1):
        g = d_initials[j] if g is None else d_initials[j] + torch.exp(log_decays[j])[..., None, None] * g
    return g


class _SequenceParallelAllGatherKernels(torch.autograd.Function):
    """The all-gather form on the CUDA stages: the zero-start outflow comes from a read-only fold over the
    per-tile states (``ssd_state_fold``), so the exchange costs one extra read of them and no second pass."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, dt_softplus, group):
        from . import mamba2 as M

        rank = dist.get_rank(group)
        decays = []

        def inflow(final0, log_decay):
            decays.extend(_all_gather(log_decay, group))
            return fold_inflow(rank, _all_gather(final0, group), decays)

        with M._device_guard(x.device):
            out, final, q, cs, states = M.forward_stages(x, dt, A, B, C, bool(dt_softplus), want_final=True,
                                                         inflow=inflow)
        ctx.save_for_backward(x, dt, A, B, C, out, q, cs, states, *decays)
        ctx.dt_softplus, ctx.group = bool(dt_softplus), group
        return out, final

    @staticmethod
    def backward(ctx, dout, dfinal):
        from . import mamba2 as M

        x, dt, A, B, C, out, q, cs, states, *decays = ctx.saved_tensors
        rank, world = dist.get_rank(ctx.group), dist.get_world_size(ctx.group)
        dout = torch.zeros_like(x) if dout is None else dout.contiguous().float()
        dfinal = None if dfinal is None else dfinal.contiguous().float()

        def outflow(d0):
            return fold_outflow(rank, world, _all_gather(d0, ctx.group), decays)

        with M._device_guard(x.device):
            dx, ddt, dA, dB, dC, _ = M.backward_stages(x, dt, A, B, C, out, q, cs, states, dout, dfinal,
                                                       ctx.dt_softplus, outflow=outflow)
        dist.all_reduce(dA, op=dist.ReduceOp.SUM, group=ctx.group)
        return dx, ddt, dA, dB, dC, None, None


class _SequenceParallelAllGatherGeneric(torch.autograd.Function):
    """The all-gather form around any differentiable local call with the ``mamba2_ssd_fwd`` signature (the CPU
    tests pass the checker): the zero-start outflow is a call without initial state, the hand-back gradient a
    gradient with respect to the initial state alone."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, chunk_size, dt_softplus, group, op):
        rank = dist.get_rank(group)
        with torch.no_grad():
            _, final0 = op(x, dt, A, B, C, chunk_size, dt_softplus=dt_softplus, return_final_state=True)
            q = torch.nn.functional.softplus(dt) if dt_softplus else dt
            log_decay = (q * A.view(1, 1, -1)).sum(dim=1)
        decays = _all_gather(log_decay, group)
        s_in = fold_inflow(rank, _all_gather(final0, group), decays)
        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(True) for t in (x, dt, A, B, C)]
            init = None if s_in is None else s_in.detach().requires_grad_(True)
            out, final = op(*leaves, chunk_size, dt_softplus=dt_softplus, initial_states=init,
                            return_final_state=True)
        ctx.graph = (leaves, init, out, final, decays, group)
        return out.detach(), final.detach()

    @staticmethod
    def backward(ctx, dout, dfinal):
        leaves, init, out, final, decays, group = ctx.graph
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        dout = torch.zeros_like(out) if dout is None else dout
        dfinal = torch.zeros_like(final) if dfinal is None else dfinal
        if init is not None:
            d0 = torch.autograd.grad([out, final], [init], [dout, dfinal], retain_graph=True)[0]
        else:
            d0 = torch.zeros_like(final)
        g = fold_outflow(rank, world, _all_gather(d0, group), decays)
        grads = list(torch.autograd.grad([out, final], leaves, [dout, dfinal if g is None else dfinal + g]))
        grads[2] = grads[2].contiguous().clone()
        dist.all_reduce(grads[2], op=dist.ReduceOp.SUM, group=group)
        return (*grads, None, None, None, None)


def mamba2_ssd_fwd_sequence_parallel(x, dt, A, B, C, chunk_size: int, *, dt_softplus: bool = False,
                                     group: Optional[dist.ProcessGroup] = None, op: Optional[Callable] = None,
                                     exchange: str = "chain"):
    """Sequence-parallel SSD: ``x, dt, B, C`` hold this rank's block of consecutive tokens, ``A`` is replicated.

    Returns ``(out_local, final_state)``; ``final_state`` is the state after this rank's last token (the state
    of the whole sequence on the last rank).  Differentiable: backward returns the local dx, ddt, dB, dC and
    the dA summed over all ranks.  Every rank must run forward and backward.  ``exchange`` = "chain" (send /
    recv, r -> r+1 forward, r+1 -> r backward) or "allgather" (see the module docstring); with "allgather" and
    the default local call the sequence length per rank must be a multiple of 128 and headdim = dstate = 64.
    """
    if exchange not in ("chain", "allgather"):
        raise ValueError('exchange must be "chain" or "allgather"')
    if exchange == "allgather" and dist.get_world_size(group) > 1:
        if op is None:
            from .mamba2 import _validate
            _validate(x, dt, A, B, C, chunk_size, None, None, None, (0.0, float("inf")), None)
            return _SequenceParallelAllGatherKernels.apply(x, dt, A, B, C, dt_softplus, group)
        return _SequenceParallelAllGatherGeneric.apply(x, dt, A, B, C, chunk_size, dt_softplus, group, op)
    op = op or _default_op()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, _l, h, p = x.shape
    n = B.shape[3]
    a_shared = _SumGradAcrossRanks.apply(A, group) if world > 1 else A
    init = None
    if rank > 0:
        anchor = torch.zeros((), requires_grad=True)
        init = _RecvState.apply(anchor, (b, h, p, n), x.dtype, x.device, group, rank - 1)
    out, final = op(x, dt, a_shared, B, C, chunk_size, dt_softplus=dt_softplus, initial_states=init,
                    return_final_state=True)
    if rank < world - 1:
        token = _SendState.apply(final, group, rank + 1)
        out = _Attach.apply(out, token)
    return out, final
