"""The reference's own precision case tables, restated: shapes, feature modes, seeds, input recipes, gates.

Backward table: mamba_ascendc/tests/bwd_m1_precision_common.py:15-96 (8 shapes x 5 modes + one larger case
that crosses the reference's hybrid-route threshold = 41 cases; inputs :62-96; upstream gradients :161-163;
gate :195-198).  Forward table: mamba_ascendc/csrc/ops/mamba2_ssd_fwd/test/precision_common.py:11-69
(30 regular + 15 boundary cases; inputs :83-150; metrics and gate :170-228).

Only the data is restated here (what each case feeds the operator and what it demands of the result); the
checker the GPU tests compare with is this repository's fp64 oracle, and a few cases carry outputs of the
reference itself as golden fixtures (tests/golden/make_golden.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

# ----------------------------------------------------------------------------- backward table
BWD_SHAPES = (  # name, (batch, seqlen, heads, groups); headdim = dstate = chunk = 64
    ("single", (1, 64, 1, 1)),
    ("heads", (1, 64, 2, 1)),
    ("groups", (1, 128, 2, 2)),
    ("shared", (1, 128, 4, 1)),
    ("multi_group", (1, 128, 4, 2)),
    ("batch", (2, 64, 4, 4)),
    ("chunks", (1, 256, 8, 2)),
    ("occupancy", (2, 128, 8, 8)),
)
BWD_MODES = ("output_only", "output_final", "final_only", "full_channel_D", "full_head_D")
BWD_NRMSE_GATE = 8.0e-3
BWD_COSINE_GATE = 0.999


@dataclass(frozen=True)
class BwdCase:
    case_id: int
    category: str
    shape: Tuple[int, int, int, int]
    mode: str

    @property
    def name(self) -> str:
        return f"{self.case_id:02d}-{self.category}-{self.mode}"


def bwd_cases() -> List[BwdCase]:
    cases, cid = [], 0
    for category, shape in BWD_SHAPES:
        for mode in BWD_MODES:
            cid += 1
            cases.append(BwdCase(cid, category, shape, mode))
    cases.append(BwdCase(cid + 1, "hybrid_threshold", (1, 1024, 64, 16), "full_head_D"))
    return cases


def _pos(gen, *dims, scale):
    return scale + scale * torch.rand(*dims, generator=gen)


def bwd_inputs(case: BwdCase) -> Dict[str, object]:
    """Tensors and flags of one backward case; draw order as in the reference (one CPU generator, seed
    20260810 + case id): x, dt, A, B, C, then for the full modes D, z, dt_bias, initial_states."""
    b, l, h, g = case.shape
    gen = torch.Generator(device="cpu").manual_seed(20260810 + case.case_id)
    v: Dict[str, object] = {
        "x": _pos(gen, b, l, h, 64, scale=0.1),
        "dt": _pos(gen, b, l, h, scale=0.03),
        "A": -(0.1 + 0.2 * torch.rand(h, generator=gen)),
        "B": _pos(gen, b, l, g, 64, scale=0.05),
        "C": _pos(gen, b, l, g, 64, scale=0.05),
        "D": None, "z": None, "dt_bias": None, "initial_states": None,
        "dt_softplus": False, "dt_limit": (0.0, math.inf), "chunk_size": 64,
    }
    if case.mode.startswith("full"):
        v["D"] = _pos(gen, h, scale=0.03) if case.mode == "full_head_D" else _pos(gen, h, 64, scale=0.03)
        v["z"] = _pos(gen, b, l, h, 64, scale=0.2)
        v["dt_bias"] = 0.02 * torch.randn(h, generator=gen)
        v["initial_states"] = _pos(gen, b, h, 64, 64, scale=0.02)
        v["dt_softplus"] = True
        v["dt_limit"] = (0.02, 1.0)
    return v


def bwd_upstream(case: BwdCase, out_shape, final_shape):
    """(dout, dfinal) of the case: 0.1 + 0.1 U[0,1) from seed 20260811 + case id, dout drawn first."""
    gen = torch.Generator(device="cpu").manual_seed(20260811 + case.case_id)
    dout = 0.1 + 0.1 * torch.rand(out_shape, generator=gen)
    dfinal = 0.1 + 0.1 * torch.rand(final_shape, generator=gen)
    return dout, dfinal


def bwd_selected(case: BwdCase, out, final, dout, dfinal):
    """Which outputs carry an upstream gradient in this mode."""
    if case.mode == "output_only":
        return (out,), (dout,)
    if case.mode == "final_only":
        return (final,), (dfinal,)
    return (out, final), (dout, dfinal)


TENSOR_NAMES = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias", "initial_states")


def leaf_names(values) -> List[str]:
    return [n for n in TENSOR_NAMES if values[n] is not None]


def call_kwargs(values, leaves) -> Dict[str, object]:
    """Keyword arguments of the public API call for a case, given its leaf tensors by name."""
    return dict(D=leaves.get("D"), z=leaves.get("z"), dt_bias=leaves.get("dt_bias"), dt_softplus=values["dt_softplus"],
                dt_limit=values["dt_limit"], initial_states=leaves.get("initial_states"), return_final_state=True)


# ----------------------------------------------------------------------------- forward table
FWD_THRESHOLD = 2.0 ** -13  # mean relative error; the maximum relative error may be ten times that
FWD_FEATURES = ("basic", "d_only", "z_only", "initial", "softplus", "all")
_FWD_SIX = (
    ("small", (1, 32, 2, 8, 8, 16, 1)),
    ("tail", (1, 65, 4, 16, 16, 32, 2)),
    ("multi_group", (2, 128, 8, 32, 32, 64, 2)),
)
_FWD_PAIRS = (  # category, [B,L,H,P,N,chunk,G], feature
    ("chunk128", (1, 256, 8, 32, 64, 128, 2), "basic"), ("chunk128", (1, 256, 8, 32, 64, 128, 2), "all"),
    ("aligned", (1, 128, 2, 64, 64, 64, 1), "basic"), ("aligned", (1, 128, 2, 64, 64, 64, 1), "all"),
    ("aligned128", (1, 128, 2, 64, 64, 128, 1), "basic"), ("aligned128", (1, 128, 2, 64, 64, 128, 1), "all"),
    ("dstate128", (1, 128, 2, 64, 128, 128, 1), "basic"), ("dstate128", (1, 128, 2, 64, 128, 128, 1), "all"),
    ("single_token", (1, 1, 1, 8, 8, 16, 1), "basic"),
    ("odd_l", (1, 31, 2, 16, 16, 16, 1), "all"),
    ("head_group_ratio", (1, 96, 16, 16, 32, 32, 1), "basic"),
    ("many_groups", (1, 96, 16, 16, 32, 32, 8), "all"),
)
FWD_BOUNDARIES = ("x_zero", "b_zero", "c_zero", "a_near_zero", "a_strong", "dt_softplus_negative",
                  "dt_softplus_positive", "dt_limit_fixed", "z_negative", "z_zero", "z_positive", "initial_zero",
                  "initial_one", "d_per_head", "d_per_channel")
FWD_BOUNDARY_SHAPE = (1, 32, 2, 8, 8, 16, 1)


@dataclass(frozen=True)
class FwdCase:
    case_id: int
    category: str
    shape: Tuple[int, int, int, int, int, int, int]
    feature: str
    boundary: Optional[str]

    @property
    def name(self) -> str:
        return f"{self.case_id:02d}-{self.category}-{self.boundary or self.feature}"


def fwd_cases() -> List[FwdCase]:
    cases, cid = [], 0
    for category, shape in _FWD_SIX:
        for feature in FWD_FEATURES:
            cid += 1
            cases.append(FwdCase(cid, category, shape, feature, None))
    for category, shape, feature in _FWD_PAIRS:
        cid += 1
        cases.append(FwdCase(cid, category, shape, feature, None))
    for boundary in FWD_BOUNDARIES:
        cid += 1
        cases.append(FwdCase(cid, "boundary", FWD_BOUNDARY_SHAPE, "basic", boundary))
    return cases


def fwd_inputs(case: FwdCase) -> Dict[str, object]:
    """Positive-domain inputs of one forward case (seed 20260801 + case id; draw order x, dt, A, B, C, then
    the optional tensors the feature switches on: D [H,P], z, dt_bias, initial_states), followed by the
    boundary override of the case, if any."""
    b, l, h, p, n, chunk, g = case.shape
    gen = torch.Generator().manual_seed(20260801 + case.case_id)
    x = 0.1 + 0.9 * torch.rand(b, l, h, p, generator=gen)
    dt = 0.01 + 0.1 * torch.rand(b, l, h, generator=gen)
    A = -(0.1 + 0.4 * torch.rand(h, generator=gen))
    B = 0.02 + 0.18 * torch.rand(b, l, g, n, generator=gen)
    C = 0.02 + 0.18 * torch.rand(b, l, g, n, generator=gen)
    f = case.feature
    has_d, has_z = f in ("d_only", "all"), f in ("z_only", "all")
    has_bias = softplus = f in ("softplus", "all")
    has_init = f in ("initial", "all")
    D = 0.1 + torch.rand(h, p, generator=gen) if has_d else None
    z = 0.1 + torch.rand(b, l, h, p, generator=gen) if has_z else None
    dt_bias = 0.01 * torch.rand(h, generator=gen) if has_bias else None
    init = 0.1 + torch.rand(b, h, p, n, generator=gen) if has_init else None
    limit = (0.005, 0.2) if softplus else (0.0, math.inf)
    bd = case.boundary
    if bd == "x_zero":
        x.zero_()
    elif bd == "b_zero":
        B.zero_()
    elif bd == "c_zero":
        C.zero_()
    elif bd == "a_near_zero":
        A.fill_(-1e-4)
    elif bd == "a_strong":
        A.fill_(-10.0)
    elif bd in ("dt_softplus_negative", "dt_softplus_positive"):
        dt.fill_(-20.0 if bd.endswith("negative") else 20.0)
        softplus, limit = True, (0.0, 0.2)
    elif bd == "dt_limit_fixed":
        softplus, limit = True, (0.05, 0.05)
    elif bd in ("z_negative", "z_zero", "z_positive"):
        z = torch.full_like(x, {"z_negative": -20.0, "z_zero": 0.0, "z_positive": 20.0}[bd])
    elif bd == "initial_zero":
        init = torch.zeros(b, h, p, n)
    elif bd == "initial_one":
        init = torch.ones(b, h, p, n)
    elif bd == "d_per_head":
        D = 0.1 + torch.rand(h, generator=gen)
    elif bd == "d_per_channel":
        D = 0.1 + torch.rand(h, p, generator=gen)
    return {"x": x, "dt": dt, "A": A, "B": B, "C": C, "D": D, "z": z, "dt_bias": dt_bias, "initial_states": init,
            "dt_softplus": softplus, "dt_limit": limit, "chunk_size": chunk}


def fwd_metrics(actual: torch.Tensor, reference: torch.Tensor) -> Dict[str, float]:
    """Mean and maximum relative error with the table's fixed 1e-7 floor in the denominator, and non-finite count."""
    a, r = actual.detach().cpu().double(), reference.detach().cpu().double()
    err = (a - r).abs()
    rel = err / (r.abs() + 1e-7)
    return {"MERE": rel.mean().item(), "MARE": rel.max().item(), "max_abs": err.max().item(),
            "nan_inf": int((~torch.isfinite(a)).sum().item())}


def bwd_metrics(actual: torch.Tensor, expected: torch.Tensor) -> Dict[str, float]:
    """NRMSE (error norm over reference norm, floor 1e-12) and cosine similarity (1 when both are all zero)."""
    a, e = actual.detach().cpu().double().flatten(), expected.detach().cpu().double().flatten()
    err = a - e
    both_zero = int(torch.count_nonzero(a)) == 0 and int(torch.count_nonzero(e)) == 0
    cos = 1.0 if both_zero else (a @ e / (a.norm() * e.norm()).clamp_min(1e-300)).item()
    return {"nrmse": (err.norm() / e.norm().clamp_min(1e-12)).item(), "cosine": cos, "max_abs": err.abs().max().item()}
