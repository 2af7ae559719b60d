"""Mamba-2 SSD forward and backward on B200 behind the reference's public API.

``mamba2_ssd_fwd`` keeps the signature, argument meaning, return convention and
error style of ``ascend_kernel.mamba2_ssd_fwd`` in So-cean/mamba-ascendc
(mamba_ascendc/python/ascend_kernel/ascend_kernel/mamba2.py:1923-2017; alias
``mamba_chunk_scan_combined`` :2020).  Where the reference picks between several
device routes and torch glue, this layer has one route: a ``torch.autograd.Function``
that allocates outputs and scratch tensors with torch and enqueues the C-ABI stages
of libssd_b200.so on the current CUDA stream.  There is no CPU path.

Stages (see include/ssd_b200.h): dt softplus + in-tile cumulative decay, chunk
states (tcgen05) and inter-tile state scan (one fused launch when batch * ngroups
fills the GPU, two tile-parallel launches otherwise), output kernel (tcgen05);
backward: local state gradient (tcgen05) and reverse state scan (fused likewise),
dx + dt stage (tcgen05), dB/dC (tcgen05), ddt/dA finalisation.

``chunk_size`` is validated like the reference does, but the kernels always tile the
sequence by 128 tokens: the SSD result does not depend on the chunk length.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
from typing import Dict, Optional, Tuple, Union

import torch

from . import _capi
from .shapes import run_general

TILE = 128

_status_words: Dict[int, torch.Tensor] = {}


def _status(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels set when a bounded wait gives up (see ``check_status``)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = word
    return word


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a TMA / MMA wait that ran out.

    A kernel whose bounded wait gives up writes no results, and every kernel launched after it returns at
    once, so tensors produced since the last check are not valid until this has been called and returned.
    Raising clears the word: the next call starts clean."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    word = _status(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        kind = {1: "a TMA load did not arrive", 2: "a tensor-core product or its hand-off did not complete",
                3: "shared memory misaligned"}.get(code & 15, "unknown")
        raise RuntimeError(f"mamba2_ssd: a device-side wait gave up (status {code}: {kind}; source file "
                           f"{code >> 12}, wait {(code >> 4) & 255}); results are invalid")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def make_shape(x: torch.Tensor, B: torch.Tensor, dt_softplus: bool,
               dt_limit: Tuple[float, float] = (0.0, float("inf")), valid_len: int = 0) -> _capi.SsdShape:
    b, l, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    return _capi.SsdShape(b, l, h, p, n, TILE, g, _capi.SSD_FLAG_DT_SOFTPLUS if dt_softplus else 0,
                          float(dt_limit[0]), float(dt_limit[1]), int(valid_len))


# ----------------------------------------------------------------------------- validation
def _check_tensor(t: torch.Tensor, name: str) -> None:
    # mamba_ascendc/csrc/ops/mamba2_ssd_fwd/op_host/mamba2_ssd_fwd.cpp:15-23
    if not t.is_cuda:
        raise RuntimeError(f"mamba2_ssd_fwd: {name} must be a CUDA tensor")
    if t.dtype != torch.float32:
        raise RuntimeError(f"mamba2_ssd_fwd: {name} must be float32")
    if not t.is_contiguous():
        raise RuntimeError(f"mamba2_ssd_fwd: {name} must be contiguous")


def _validate(x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_limit, initial_states) -> None:
    for t, name in ((x, "x"), (dt, "dt"), (A, "A"), (B, "B"), (C, "C")):
        _check_tensor(t, name)
    # mamba2_ssd_fwd.cpp:59-85
    if x.dim() != 4:
        raise RuntimeError("mamba2_ssd_fwd: x must have shape [B,L,H,P]")
    if dt.dim() != 3:
        raise RuntimeError("mamba2_ssd_fwd: dt must have shape [B,L,H]")
    if A.dim() != 1:
        raise RuntimeError("mamba2_ssd_fwd: A must have shape [H]")
    if B.dim() != 4 or C.dim() != 4:
        raise RuntimeError("mamba2_ssd_fwd: B and C must have shape [B,L,G,N]")
    b, l, h, _p = x.shape
    if tuple(dt.shape) != (b, l, h):
        raise RuntimeError("mamba2_ssd_fwd: dt shape must equal [B,L,H]")
    if A.shape[0] != h:
        raise RuntimeError("mamba2_ssd_fwd: A shape must equal [H]")
    if B.shape != C.shape:
        raise RuntimeError("mamba2_ssd_fwd: B and C shapes must match")
    if B.shape[0] != b or B.shape[1] != l:
        raise RuntimeError("mamba2_ssd_fwd: B/C batch and sequence dimensions must match x")
    if h % B.shape[2] != 0:
        raise RuntimeError("mamba2_ssd_fwd: nheads must be divisible by ngroups")
    if int(chunk_size) <= 0:
        raise RuntimeError("mamba2_ssd_fwd: chunk_size must be positive")
    if float(dt_limit[0]) > float(dt_limit[1]):
        raise RuntimeError("mamba2_ssd_fwd: dt_limit min must not exceed max")
    if initial_states is not None:
        _check_tensor(initial_states, "initial_states")
        # mamba2_ssd_fwd.cpp:108-112
        if tuple(initial_states.shape) != (b, h, x.shape[3], B.shape[3]):
            raise RuntimeError("mamba2_ssd_fwd: initial_states shape must equal [B,H,P,N]")
    # mamba2_ssd_fwd.cpp:88-106
    if D is not None:
        _check_tensor(D, "D")
        if not ((D.dim() == 1 and D.shape[0] == h) or (D.dim() == 2 and tuple(D.shape) == (h, x.shape[3]))):
            raise RuntimeError("mamba2_ssd_fwd: D shape must equal [H] or [H,P]")
    if z is not None:
        _check_tensor(z, "z")
        if z.shape != x.shape:
            raise RuntimeError("mamba2_ssd_fwd: z shape must match x")
    if dt_bias is not None:
        _check_tensor(dt_bias, "dt_bias")
        if dt_bias.dim() != 1 or dt_bias.shape[0] != h:
            raise RuntimeError("mamba2_ssd_fwd: dt_bias shape must equal [H]")


# ----------------------------------------------------------------------------- route of the state stages
# The per-tile state products and the inter-tile recurrence run either as two tile-parallel launches
# (ssd_chunk_state + ssd_state_passing_*) or as one launch that walks each (batch, group) in tile order with
# the running state on chip (ssd_chunk_state_scan).  The second moves 2 GiB less per pass at the H256 shape
# but has only batch * ngroups CTAs; "auto" takes it when that is at least 1.5 x the SM count.
_state_scan = "auto"
_sm_counts: Dict[int, int] = {}


def set_state_scan(mode: str) -> str:
    """Choose "auto" (default), "on" (whenever the kernel takes the shape) or "off"; returns the previous mode."""
    global _state_scan
    if mode not in ("auto", "on", "off"):
        raise ValueError('state scan mode must be "auto", "on" or "off"')
    previous, _state_scan = _state_scan, mode
    return previous


def _use_state_scan(shape: "_capi.SsdShape", device: torch.device) -> bool:
    if _state_scan == "off" or not _capi.lib.ssd_chunk_state_scan_supported(ctypes.byref(shape)):
        return False
    if _state_scan == "on":
        return True
    idx = device.index if device.index is not None else torch.cuda.current_device()
    sms = _sm_counts.get(idx)
    if sms is None:
        sms = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return 2 * shape.batch * shape.ngroups >= 3 * sms


# ----------------------------------------------------------------------------- stage drivers
# When set to a list, every stage launch is bracketed by CUDA events on the launching stream and
# (name, start, end) is appended; used by bench.py to time individual kernels inside a step.
stage_events = None


def _call(name: str, fn, *args) -> None:
    events = stage_events
    if events is None:
        _capi.check(fn(*args), name)
        return
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _capi.check(fn(*args), name)
    end.record()
    events.append((name, start, end))


def forward_stages(x, dt, A, B, C, dt_softplus: bool, want_final: bool = True, initial_states=None, dt_bias=None,
                   dt_limit=(0.0, float("inf")), valid_len: int = 0, inflow=None):
    """Run the four forward stages; returns (out, final_state, q, cs, states_start).

    ``inflow(final0, log_decay) -> initial_states`` (sequence-parallel mode): called once the per-tile states
    exist, with the state this block of tokens would hand on from a zero start ([B,H,P,N]) and the logarithm
    of its total decay ([B,H]); what it returns seeds the recurrence."""
    shape = make_shape(x, B, dt_softplus, dt_limit, valid_len)
    _capi.check(_capi.lib.ssd_check_shape(ctypes.byref(shape)), "mamba2_ssd_fwd")
    b, l, h, p = x.shape
    n = B.shape[3]
    k = l // TILE
    dev = x.device
    status = _status(dev)
    st = _stream()
    q = torch.empty(b, h, l, device=dev, dtype=torch.float32)
    cs = torch.empty_like(q)
    states = torch.empty(b, h, k, p, n, device=dev, dtype=torch.float32)
    out = torch.empty_like(x)
    final = torch.empty(b, h, p, n, device=dev, dtype=torch.float32) if want_final else None
    lib = _capi.lib
    sp = ctypes.byref(shape)
    _call("mamba2_ssd_dt_cumsum", lib.ssd_dt_cumsum, sp, _ptr(dt), _ptr(dt_bias), _ptr(A), _ptr(q), _ptr(cs), st)
    if inflow is None and _use_state_scan(shape, dev):
        _call("mamba2_ssd_chunk_state_scan", lib.ssd_chunk_state_scan, sp, _ptr(x), _ptr(B), _ptr(q), _ptr(cs),
              _ptr(initial_states), _ptr(states), _ptr(final), 0, _ptr(status), st)
        _call("mamba2_ssd_chunk_scan", lib.ssd_chunk_scan_fwd, sp, _ptr(x), _ptr(B), _ptr(C), _ptr(states), _ptr(q), _ptr(cs),
              _ptr(out), _ptr(status), st)
        return out, final, q, cs, states
    _call("mamba2_ssd_chunk_state", lib.ssd_chunk_state, sp, _ptr(x), _ptr(B), _ptr(q), _ptr(cs), _ptr(states), 0, _ptr(status), st)
    if inflow is not None:
        final0 = torch.empty(b, h, p, n, device=dev, dtype=torch.float32)
        _call("mamba2_ssd_state_fold", lib.ssd_state_fold, sp, _ptr(states), _ptr(cs), None, _ptr(final0), 0, st)
        initial_states = inflow(final0, cs.view(b, h, k, TILE)[..., -1].sum(-1))
    _call("mamba2_ssd_state_passing", lib.ssd_state_passing_fwd, sp, _ptr(states), _ptr(cs), _ptr(initial_states),
          _ptr(final), st)
    _call("mamba2_ssd_chunk_scan", lib.ssd_chunk_scan_fwd, sp, _ptr(x), _ptr(B), _ptr(C), _ptr(states), _ptr(q), _ptr(cs), _ptr(out),
                                       _ptr(status), st)
    return out, final, q, cs, states


def backward_stages(x, dt, A, B, C, out, q, cs, states, dout, dfinal, dt_softplus: bool, want_dinitial: bool = False,
                    dt_bias=None, dt_limit=(0.0, float("inf")), valid_len: int = 0, outflow=None, D=None):
    """Run the backward stages; returns (dx, ddt, dA, dB, dC, d_initial_states or None).

    ``outflow(d_initial0) -> extra dfinal or None`` (sequence-parallel mode): called once the local state
    gradients exist, with the gradient this block hands back to its predecessor when nothing comes in from
    its successors; what it returns is added to ``dfinal`` before the reverse recurrence runs.

    ``D``: the skip connection of the gated node; then ``dout`` / ``out`` are the gradient / value of the SSD
    output before skip and gate, and ``D * dout`` is added to dx by the dx kernel."""
    shape = make_shape(x, B, dt_softplus, dt_limit, valid_len)
    b, l, h, p = x.shape
    n = B.shape[3]
    k = l // TILE
    dev = x.device
    status = _status(dev)
    st = _stream()
    lib = _capi.lib
    sp = ctypes.byref(shape)
    dstates = torch.empty(b, h, k, p, n, device=dev, dtype=torch.float32)
    g_last = torch.empty(b, h, k, device=dev, dtype=torch.float32)
    ddt_t = torch.empty(b, h, l, device=dev, dtype=torch.float32)
    dA_part = torch.empty(b, h, k, device=dev, dtype=torch.float64)
    dx = torch.empty_like(x)
    ddt = torch.empty_like(dt)
    dA = torch.empty_like(A)
    dB = torch.empty_like(B)
    dC = torch.empty_like(C)
    d_initial = torch.empty(b, h, p, n, device=dev, dtype=torch.float32) if want_dinitial else None
    # g_last (the gradient of each tile's total decay through the state recurrence) comes out of the dB/dC
    # kernel, which streams the forward's states and dU anyway; the reverse scan then never reads the states.
    fused = outflow is None and _use_state_scan(shape, dev)
    if fused:
        _call("mamba2_ssd_chunk_state_scan_bwd", lib.ssd_chunk_state_scan, sp, _ptr(dout), _ptr(C), _ptr(q), _ptr(cs),
              _ptr(dfinal), _ptr(dstates), _ptr(d_initial), 1, _ptr(status), st)
    else:
        _call("mamba2_ssd_chunk_state_bwd", lib.ssd_chunk_state, sp, _ptr(dout), _ptr(C), _ptr(q), _ptr(cs), _ptr(dstates), 1, _ptr(status), st)
    if outflow is not None:
        d0 = torch.empty(b, h, p, n, device=dev, dtype=torch.float32)
        _call("mamba2_ssd_state_fold", lib.ssd_state_fold, sp, _ptr(dstates), _ptr(cs), _ptr(dfinal), _ptr(d0), 1, st)
        extra = outflow(d0)
        if extra is not None:
            dfinal = extra if dfinal is None else dfinal + extra
    if not fused:
        _call("mamba2_ssd_state_passing_bwd", lib.ssd_state_passing_bwd, sp, _ptr(dstates), None, _ptr(cs), _ptr(dfinal),
              None, _ptr(d_initial), st)
    _call("mamba2_ssd_chunk_dbc_bwd", lib.ssd_chunk_dbc_bwd, sp, _ptr(x), _ptr(B), _ptr(C), _ptr(dout), _ptr(states), _ptr(dstates),
                                      _ptr(q), _ptr(cs), _ptr(dB), _ptr(dC), _ptr(g_last), _ptr(status), st)
    _call("mamba2_ssd_chunk_dx_bwd", lib.ssd_chunk_dx_bwd, sp, _ptr(x), _ptr(B), _ptr(C), _ptr(dout), _ptr(out), _ptr(dstates), _ptr(q),
                                     _ptr(cs), _ptr(dt), _ptr(dt_bias), _ptr(A), _ptr(g_last), _ptr(dx), _ptr(ddt_t),
                                     _ptr(dA_part), _ptr(D), _d_mode(D), _ptr(status), st)
    _call("mamba2_ssd_dt_bwd", lib.ssd_dt_finalize_bwd, sp, _ptr(ddt_t), _ptr(dA_part), _ptr(ddt), _ptr(dA), st)
    return dx, ddt, dA, dB, dC, d_initial


# ----------------------------------------------------------------------------- autograd
class _Mamba2SsdAutograd(torch.autograd.Function):
    """Counterpart of ``_Mamba2SsdAutogradM1`` (mamba2.py:1661-1838): saves the inputs plus, under the
    default policy, q, cs, the tile-start states and the output; backward returns gradients for x, dt, A, B, C, the initial states and
    dt_bias, and None for the non-tensor arguments."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, dt_softplus, initial_states, dt_bias, dt_min, dt_max, valid_len):
        out, final, q, cs, states = forward_stages(x, dt, A, B, C, dt_softplus, want_final=True,
                                                   initial_states=initial_states, dt_bias=dt_bias,
                                                   dt_limit=(dt_min, dt_max), valid_len=valid_len)
        ctx.valid_len = valid_len
        ctx.recompute = _save_policy == "recompute"
        if ctx.recompute:  # inputs only; out, q, cs and the tile-start states are rebuilt in backward
            ctx.save_for_backward(x, dt, A, B, C, dt_bias, initial_states)
        else:
            ctx.save_for_backward(x, dt, A, B, C, dt_bias, out, q, cs, states)
        ctx.dt_softplus = dt_softplus
        ctx.has_initial = initial_states is not None
        ctx.dt_limit = (dt_min, dt_max)
        return out, final

    @staticmethod
    def backward(ctx, dout, dfinal):
        if ctx.recompute:
            x, dt, A, B, C, dt_bias, initial_states = ctx.saved_tensors
        else:
            x, dt, A, B, C, dt_bias, out, q, cs, states = ctx.saved_tensors
        if dout is None:  # loss depends on the final state only (mamba2.py:1801-1802)
            dout = torch.zeros_like(x)
        dout = dout.contiguous().float()
        if dfinal is not None:
            dfinal = dfinal.contiguous().float()
        with _device_guard(x.device):
            if ctx.recompute:
                out, _, q, cs, states = forward_stages(x, dt, A, B, C, ctx.dt_softplus, want_final=False,
                                                       initial_states=initial_states, dt_bias=dt_bias,
                                                       dt_limit=ctx.dt_limit, valid_len=ctx.valid_len)
            dx, ddt, dA, dB, dC, dinit = backward_stages(x, dt, A, B, C, out, q, cs, states, dout, dfinal,
                                                         ctx.dt_softplus, want_dinitial=ctx.has_initial,
                                                         dt_bias=dt_bias, dt_limit=ctx.dt_limit,
                                                         valid_len=ctx.valid_len)
        dbias = ddt.sum(dim=(0, 1)) if dt_bias is not None else None  # mamba2_ssd_dt_bwd/design.md:63-77
        return dx, ddt, dA, dB, dC, None, dinit, dbias, None, None, None


# ----------------------------------------------------------------------------- D skip and z gate
def _d_mode(D: Optional[torch.Tensor]) -> int:
    return 0 if D is None else D.dim()  # 1: [H], 2: [H,P]


def gate_forward(y, x, B, D, z):
    """out = (y + D .* x) .* silu(z) in one pass (ssd_gate_skip_fwd)."""
    shape = make_shape(x, B, False)
    out = torch.empty_like(y)
    _call("mamba2_ssd_gate", _capi.lib.ssd_gate_skip_fwd, ctypes.byref(shape), _ptr(y), _ptr(x), _ptr(D), _d_mode(D),
          _ptr(z), _ptr(out), _stream())
    return out


def gate_backward(dout, y, x, B, D, z):
    """(dy, dz, dD) of the gate / skip epilogue in one pass; without z, dy is dout itself."""
    shape = make_shape(x, B, False)
    sp = ctypes.byref(shape)
    dy = torch.empty_like(dout) if z is not None else dout
    dz = torch.empty_like(dout) if z is not None else None
    dD = part = None
    if D is not None:
        dD = torch.empty_like(D)
        part = torch.empty(_capi.lib.ssd_gate_partial_floats(sp), device=dout.device, dtype=torch.float32)
    _call("mamba2_ssd_bwd_gate", _capi.lib.ssd_gate_skip_bwd, sp, _ptr(dout), _ptr(y), _ptr(x), _ptr(D), _d_mode(D),
          _ptr(z), _ptr(dy) if z is not None else None, _ptr(dz), _ptr(part), _ptr(dD), _stream())
    return dy, dz, dD


class _Mamba2SsdGatedAutograd(torch.autograd.Function):
    """The SSD with its D skip connection and z gate as one autograd node: the epilogue runs as one fused pass
    forward and one backward (the reference fuses them into its state-epilogue and gate kernels,
    mamba2_ssd_state_epilogue.cpp:413-482, bwd_gate/design.md:8-13), and the skip connection's share of dx is
    added in the epilogue of the dx kernel."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, D, z, dt_softplus, initial_states, dt_bias, dt_min, dt_max):
        y, final, q, cs, states = forward_stages(x, dt, A, B, C, dt_softplus, want_final=True,
                                                 initial_states=initial_states, dt_bias=dt_bias,
                                                 dt_limit=(dt_min, dt_max))
        out = gate_forward(y, x, B, D, z)
        ctx.recompute = _save_policy == "recompute"
        if ctx.recompute:
            ctx.save_for_backward(x, dt, A, B, C, dt_bias, D, z, initial_states)
        else:
            ctx.save_for_backward(x, dt, A, B, C, dt_bias, D, z, y, q, cs, states)
        ctx.dt_softplus = dt_softplus
        ctx.has_initial = initial_states is not None
        ctx.dt_limit = (dt_min, dt_max)
        return out, final

    @staticmethod
    def backward(ctx, dout, dfinal):
        if ctx.recompute:
            x, dt, A, B, C, dt_bias, D, z, initial_states = ctx.saved_tensors
        else:
            x, dt, A, B, C, dt_bias, D, z, y, q, cs, states = ctx.saved_tensors
        if dout is None:
            dout = torch.zeros_like(x)
        dout = dout.contiguous().float()
        if dfinal is not None:
            dfinal = dfinal.contiguous().float()
        with _device_guard(x.device):
            if ctx.recompute:
                y, _, q, cs, states = forward_stages(x, dt, A, B, C, ctx.dt_softplus, want_final=False,
                                                     initial_states=initial_states, dt_bias=dt_bias,
                                                     dt_limit=ctx.dt_limit)
            dy, dz, dD = gate_backward(dout, y, x, B, D, z)
            dx, ddt, dA, dB, dC, dinit = backward_stages(x, dt, A, B, C, y, q, cs, states, dy, dfinal,
                                                         ctx.dt_softplus, want_dinitial=ctx.has_initial,
                                                         dt_bias=dt_bias, dt_limit=ctx.dt_limit, D=D)
        dbias = ddt.sum(dim=(0, 1)) if dt_bias is not None else None
        return dx, ddt, dA, dB, dC, dD, dz, None, dinit, dbias, None, None


# What the autograd function keeps between forward and backward (mamba2_ssd_bwd/design.md:207-223 lists the
# reference's save / recompute choices).  "save": inputs plus out, q, cs and the tile-start states (at the
# H256 shape 3.1 GiB on top of the inputs); "recompute": inputs only, the forward stages run again in backward.
_save_policy = "save"


def set_save_policy(policy: str) -> str:
    """Choose "save" (default) or "recompute"; returns the previous policy."""
    global _save_policy
    if policy not in ("save", "recompute"):
        raise ValueError('save policy must be "save" or "recompute"')
    previous, _save_policy = _save_policy, policy
    return previous


class SavedTensorStats:
    """Bytes autograd holds for backward, counted with saved-tensor hooks (the reference's benchmark counts
    the same way, benchmarks/mamba2_backward_bench.py:168-209): ``logical_bytes`` adds every saved tensor,
    ``unique_bytes`` counts each backing storage once.  Use as ``with stats.hooks(): out = fn(...)``."""

    def __init__(self):
        self.logical_bytes = 0
        self._storages: Dict[Tuple[str, Optional[int], int], int] = {}

    def _pack(self, t: torch.Tensor) -> torch.Tensor:
        self.logical_bytes += t.numel() * t.element_size()
        st = t.untyped_storage()
        key = (t.device.type, t.device.index, st.data_ptr())
        self._storages[key] = max(self._storages.get(key, 0), st.nbytes())
        return t

    def hooks(self):
        return torch.autograd.graph.saved_tensors_hooks(self._pack, lambda t: t)

    @property
    def unique_bytes(self) -> int:
        return sum(self._storages.values())


def _device_guard(device: torch.device):
    """Launches go to the current stream of the tensors' device; a context switch only when that is not the
    current device already (the switch costs several microseconds per call)."""
    if torch.cuda.current_device() == device.index:
        return contextlib.nullcontext()
    return torch.cuda.device(device)


def _requires_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def mamba2_ssd_fwd(
    x: torch.Tensor,
    dt: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    chunk_size: int,
    D: Optional[torch.Tensor] = None,
    z: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    dt_softplus: bool = False,
    dt_limit: Tuple[float, float] = (0.0, float("inf")),
    initial_states: Optional[torch.Tensor] = None,
    return_final_state: bool = False,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Mamba-2 SSD chunk scan: ``out[B,L,H,P]`` and optionally ``final_state[B,H,P,N]``.

    x [B,L,H,P], dt [B,L,H], A [H] (the negative decay value, not its log), B and C [B,L,G,N] with
    head h reading group h // (H/G); all contiguous fp32 CUDA tensors.
    """
    _validate(x, dt, A, B, C, chunk_size, D, z, dt_bias, dt_limit, initial_states)
    lim = (float(dt_limit[0]), float(dt_limit[1]))
    needs_grad = _requires_grad(x, dt, A, B, C, initial_states, dt_bias)

    def core(xk, dtk, Ak, Bk, Ck, init, bias, valid):
        # the fixed-shape call: headdim 64, state size 64 (128 without gradients), whole tiles
        if needs_grad:
            return _Mamba2SsdAutograd.apply(xk, dtk, Ak, Bk, Ck, bool(dt_softplus), init, bias, lim[0], lim[1], valid)
        out_k, final_k, *_ = forward_stages(xk, dtk, Ak, Bk, Ck, bool(dt_softplus), want_final=return_final_state,
                                            initial_states=init, dt_bias=bias, dt_limit=lim, valid_len=valid)
        return out_k, final_k

    with _device_guard(x.device):
        p, n = x.shape[3], B.shape[3]
        native = p == 64 and x.shape[1] % TILE == 0
        if native and n == 64 and (D is not None or z is not None) and _requires_grad(
                x, dt, A, B, C, initial_states, dt_bias, D, z):
            # the kernels' own shapes with a D skip or z gate under autograd: one node, fused epilogue
            out, final = _Mamba2SsdGatedAutograd.apply(x, dt, A, B, C, D, z, bool(dt_softplus), initial_states,
                                                       dt_bias, lim[0], lim[1])
            return (out, final) if return_final_state else out
        if native and (n == 64 or (n == 128 and not needs_grad)):
            out, final = core(x, dt, A, B, C, initial_states, dt_bias, 0)  # the kernels' own shapes
            if not _requires_grad(D, z, out):
                if D is not None or z is not None:  # no gradients anywhere: the fused epilogue pass
                    out = gate_forward(out, x, B, D, z)
                return (out, final) if return_final_state else out
        else:
            # any sequence length, headdim and state size: see shapes.py
            out, final = run_general(core, x, dt, A, B, C, initial_states, dt_bias, needs_grad)
        # D skip connection and z gate (ssd_reference.py:300-318) as element-wise epilogue; under autograd
        # their gradients (dD, dz and the extra term of dx) come from these same operations
        if D is not None:
            out = out + x * (D.view(1, 1, -1, 1) if D.dim() == 1 else D.view(1, 1, *D.shape))
        if z is not None:
            out = out * torch.nn.functional.silu(z)
    if return_final_state:
        return out, final
    return out


mamba_chunk_scan_combined = mamba2_ssd_fwd
