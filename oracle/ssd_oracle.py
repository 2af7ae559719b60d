"""CPU restatement of the reference's Mamba-2 SSD algorithm.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared with.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import it; the product (``ascend_kernel``) never does and has no CPU path.

Parity status: PINNED.  ``tests/golden/make_golden.py`` ran the reference's own
``mamba_torch/ssd_reference.py`` on seeded inputs and stored its outputs and
fp64 autograd gradients; ``tests/test_oracle.py`` checks every function here
against those files.

What follows the reference, line by line (paths inside So-cean/mamba-ascendc):

* ``ssd_sequential``  — token-by-token recurrence, dtype preserving
  (mamba_torch/ssd_reference.py:10-77).
* ``segsum``          — masked segment sums (mamba_torch/ssd_reference.py:80-110).
* ``ssd_chunked``     — dt bias / softplus / clamp, dA = dt*A, x*dt
  (ssd_reference.py:236-248), padding to a chunk multiple (:250-261), the
  chunked core (:113-189: intra-chunk term, chunk states, inter-chunk
  recurrence, state-to-output term), D skip and z gate (:300-318), final state
  layout [B,H,P,N] (:320-326).  ``compute_dtype=torch.float32`` reproduces the
  reference's internal fp32 casts (:229-234); ``None`` keeps the input dtype,
  which is what an fp64 oracle needs (the reference's chunked entry point
  computes in fp32 even for fp64 inputs).

The chunked core here is written as an explicit loop over chunks instead of
the reference's (K+1)x(K+1) decay matrix; both evaluate the same recurrence
S_{k+1} = exp(sum of dA over chunk k) * S_k + U_k.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

# [B, L, H, P, N, chunk, G] of the five benchmark configurations; index 4 is the
# SSD call inside the Vision-Mamba2 network (per-GPU batch 4).
CONFIG_SHAPES = {
    0: (1, 128, 2, 64, 128, 128, 1),
    1: (1, 128, 2, 64, 64, 64, 1),
    2: (4, 2048, 16, 64, 128, 128, 4),
    3: (8, 4096, 256, 64, 64, 64, 64),
    4: (4, 4096, 6, 64, 64, 64, 1),
}
BASE_SEED = 20260806  # benchmarks/mamba2_backward_bench.py:219


def make_inputs(shape, seed: int, dtype=torch.float32):
    """Seeded inputs with the distributions the benchmark configurations name.

    Draw order x, dt, A, B, C from one CPU generator: x ~ N(0,1), dt ~ U[0,1),
    A = -U[0,1), B, C ~ N(0,1) (the README recipe, README.md:108-112).
    """
    b, l, h, p, n, _chunk, g = shape
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(b, l, h, p, generator=gen)
    dt = torch.rand(b, l, h, generator=gen)
    a = -torch.rand(h, generator=gen)
    bm = torch.randn(b, l, g, n, generator=gen)
    cm = torch.randn(b, l, g, n, generator=gen)
    return tuple(t.to(dtype) for t in (x, dt, a, bm, cm))


def config_inputs(index: int, dtype=torch.float32):
    return make_inputs(CONFIG_SHAPES[index], BASE_SEED + index, dtype)


# --------------------------------------------------------------------------- metrics
def rel_l2(a: torch.Tensor, ref: torch.Tensor) -> float:
    """||a - ref||_2 / ||ref||_2, the NRMSE of mamba_ascendc/tests/test_mamba2_ssd_bwd_m1.py:89-106."""
    ref = ref.double()
    denom = ref.norm().item()
    num = (a.double() - ref).norm().item()
    return num / denom if denom > 0 else num


def max_abs(a: torch.Tensor, ref: torch.Tensor) -> float:
    return (a.double() - ref.double()).abs().max().item()


def cosine(a: torch.Tensor, ref: torch.Tensor) -> float:
    a, ref = a.double().flatten(), ref.double().flatten()
    return (a @ ref / (a.norm() * ref.norm()).clamp_min(1e-300)).item()


# --------------------------------------------------------------------------- dt handling
def _discretise(dt, dt_bias, dt_softplus, dt_limit):
    """q = clamp(softplus(dt + bias)) (ssd_reference.py:236-240)."""
    q = dt
    if dt_bias is not None:
        q = q + dt_bias.view(1, 1, -1)
    if dt_softplus:
        q = F.softplus(q)
    return q.clamp(min=dt_limit[0], max=dt_limit[1])


# --------------------------------------------------------------------------- sequential form
def ssd_sequential(x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False,
                   dt_limit=(0.0, math.inf), initial_states=None, return_final_state=False):
    """h_t = exp(q_t A) h_{t-1} + (q_t x_t) B_t^T ; y_t = h_t C_t (+ D x_t) (* silu(z_t))."""
    b, l, h, p = x.shape
    g, n = B.shape[2:]
    if h % g:
        raise ValueError("nheads must be divisible by ngroups")
    q = _discretise(dt, dt_bias, dt_softplus, dt_limit)
    rep = h // g
    bh = B.repeat_interleave(rep, dim=2)
    ch = C.repeat_interleave(rep, dim=2)
    state = x.new_zeros(b, h, p, n) if initial_states is None else initial_states
    ys = []
    for t in range(l):
        alpha = torch.exp(q[:, t] * A.view(1, h))  # [B,H]
        inject = (x[:, t] * q[:, t, :, None])[..., None] * bh[:, t, :, None, :]  # [B,H,P,N]
        state = alpha[..., None, None] * state + inject
        y = torch.einsum("bhpn,bhn->bhp", state, ch[:, t])
        if D is not None:
            y = y + x[:, t] * (D.view(1, h, 1) if D.ndim == 1 else D[None])
        if z is not None:
            y = y * F.silu(z[:, t])
        ys.append(y)
    out = torch.stack(ys, dim=1)
    return (out, state) if return_final_state else out


# --------------------------------------------------------------------------- chunked form
def segsum(a: torch.Tensor) -> torch.Tensor:
    """out[..., i, j] = sum_{k=j+1..i} a[..., k] for i >= j, -inf above the diagonal."""
    t = a.shape[-1]
    cs = torch.cumsum(a, dim=-1)
    diff = cs[..., :, None] - cs[..., None, :]
    keep = torch.ones(t, t, dtype=torch.bool, device=a.device).tril()
    return diff.masked_fill(~keep, -math.inf)


def chunk_terms(xdt, dA, Bh, Ch, chunk):
    """Per-chunk quantities of the chunked core for per-head B/C.

    xdt [B,L,H,P], dA [B,L,H], Bh/Ch [B,L,H,N]  ->  dict with
    cs [B,H,K,T] (in-chunk inclusive cumsum of dA), y_diag [B,K,T,H,P],
    chunk_state [B,K,H,P,N] (contribution U_k of chunk k with zero inflow).
    """
    b, l, h, p = xdt.shape
    n = Bh.shape[-1]
    k = l // chunk
    xc = xdt.reshape(b, k, chunk, h, p)
    bc = Bh.reshape(b, k, chunk, h, n)
    cc = Ch.reshape(b, k, chunk, h, n)
    ac = dA.reshape(b, k, chunk, h).permute(0, 3, 1, 2)  # [B,H,K,T]
    cs = torch.cumsum(ac, dim=-1)
    decay = torch.exp(segsum(ac))  # [B,H,K,T,T], zero above the diagonal
    cb = torch.einsum("bkihn,bkjhn->bhkij", cc, bc)
    y_diag = torch.einsum("bhkij,bkjhp->bkihp", cb * decay, xc)
    to_end = torch.exp(cs[..., -1:] - cs)  # [B,H,K,T]
    chunk_state = torch.einsum("bhkt,bkthp,bkthn->bkhpn", to_end, xc, bc)
    return {"cs": cs, "y_diag": y_diag, "chunk_state": chunk_state, "cc": cc}


def ssd_core(xdt, dA, Bh, Ch, chunk, initial_states=None):
    """Chunked SSD core on discretised per-head inputs; returns (y [B,L,H,P], final [B,H,P,N], states_start)."""
    b, l, h, p = xdt.shape
    n = Bh.shape[-1]
    assert l % chunk == 0, "seqlen must be a multiple of the chunk size"
    k = l // chunk
    terms = chunk_terms(xdt, dA, Bh, Ch, chunk)
    cs, cc = terms["cs"], terms["cc"]
    state = xdt.new_zeros(b, h, p, n) if initial_states is None else initial_states
    starts = []
    for ci in range(k):
        starts.append(state)
        alpha = torch.exp(cs[:, :, ci, -1])  # [B,H]
        state = alpha[..., None, None] * state + terms["chunk_state"][:, ci]
    states_start = torch.stack(starts, dim=1)  # [B,K,H,P,N]
    y_off = torch.einsum("bkthn,bkhpn,bhkt->bkthp", cc, states_start, torch.exp(cs))
    y = (terms["y_diag"] + y_off).reshape(b, l, h, p)
    return y, state, states_start


def ssd_chunked(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False,
                dt_limit=(0.0, math.inf), initial_states=None, return_final_state=False,
                compute_dtype: Optional[torch.dtype] = torch.float32):
    """The reference's public chunked entry point; see the module docstring for ``compute_dtype``."""
    b, l, h, p = x.shape
    g, n = B.shape[2:]
    assert h % g == 0, f"nheads={h} not divisible by ngroups={g}"
    rep = h // g
    dtype_in = x.dtype
    cast = (lambda t: t) if compute_dtype is None else (lambda t: t.to(compute_dtype))
    xf, dtf, Af, Bf, Cf = (cast(t) for t in (x, dt, A, B, C))
    q = _discretise(dtf, None if dt_bias is None else cast(dt_bias), dt_softplus, dt_limit)
    dA = q * Af.view(1, 1, h)
    xdt = xf * q[..., None]
    pad = (-l) % chunk_size
    if pad:
        xdt = F.pad(xdt, (0, 0, 0, 0, 0, pad))
        dA = F.pad(dA, (0, 0, 0, pad))
        Bf = F.pad(Bf, (0, 0, 0, 0, 0, pad))
        Cf = F.pad(Cf, (0, 0, 0, 0, 0, pad))
    init = None if initial_states is None else cast(initial_states)
    y, final, _ = ssd_core(xdt, dA, Bf.repeat_interleave(rep, dim=2), Cf.repeat_interleave(rep, dim=2),
                           chunk_size, init)
    y = y[:, :l]
    if D is not None:
        Df = cast(D)
        y = y + xf * (Df.view(1, 1, h, 1) if Df.ndim == 1 else Df[None, None])
    if z is not None:
        y = y * F.silu(cast(z))
    y = y.to(dtype_in)
    return (y, final) if return_final_state else y


# --------------------------------------------------------------------------- loss and gradients
def loss_fn(out: torch.Tensor, final_state: Optional[torch.Tensor]) -> torch.Tensor:
    """mean(out^2) + mean(final_state^2), the loss of benchmark configurations 1 and 3."""
    loss = out.pow(2).mean()
    if final_state is not None:
        loss = loss + final_state.pow(2).mean()
    return loss


def fp64_forward_backward(x, dt, A, B, C, chunk_size, dt_softplus=True, sequential=False,
                          dout=None, dfinal=None) -> Tuple[torch.Tensor, ...]:
    """fp64 out, final state and gradients (dx, ddt, dA, dB, dC).

    With ``dout``/``dfinal`` given the gradients are those of
    sum(out*dout) + sum(final*dfinal); otherwise of ``loss_fn``.
    """
    leaves = [t.detach().double().requires_grad_(True) for t in (x, dt, A, B, C)]
    if sequential:
        out, final = ssd_sequential(*leaves, dt_softplus=dt_softplus, return_final_state=True)
    else:
        out, final = ssd_chunked(*leaves, chunk_size, dt_softplus=dt_softplus, return_final_state=True,
                                 compute_dtype=None)
    if dout is None and dfinal is None:
        loss = loss_fn(out, final)
    else:
        loss = out.new_zeros(())
        if dout is not None:
            loss = loss + (out * dout.double()).sum()
        if dfinal is not None:
            loss = loss + (final * dfinal.double()).sum()
    grads = torch.autograd.grad(loss, leaves)
    return (out.detach(), final.detach(), *[g_.detach() for g_ in grads])
