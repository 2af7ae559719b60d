"""The restated case tables of the reference (tests/reference_cases.py) and the oracle on them, on CPU.

The tables must have the reference's sizes (41 backward, 45 forward cases); for the cases whose reference
outputs are stored (tests/golden/table_cases.npz, written by tests/golden/make_golden.py from the reference's
``ssd_chunk_scan_ref`` and autograd through it) the oracle's fp32 path must reproduce them -- this is what
pins the checker the GPU table tests use, including its gradients of D, z, dt_bias and initial_states.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import reference_cases as R
from oracle import ssd_oracle as O

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "table_cases.npz")
CORE = ("x", "dt", "A", "B", "C")


def test_table_sizes_and_ids():
    bwd, fwd = R.bwd_cases(), R.fwd_cases()
    assert len(bwd) == 41 and len(fwd) == 45
    assert [c.case_id for c in bwd] == list(range(1, 42)) and [c.case_id for c in fwd] == list(range(1, 46))
    assert bwd[-1].shape == (1, 1024, 64, 16) and bwd[-1].mode == "full_head_D"
    assert sum(c.boundary is not None for c in fwd) == 15
    assert {c.name for c in fwd if c.boundary} >= {"31-boundary-x_zero", "45-boundary-d_per_channel"}


def test_input_recipes_are_in_the_tables_domains():
    v = R.bwd_inputs(R.bwd_cases()[3])  # single / full_channel_D
    assert v["D"].shape == (1, 64) and v["dt_softplus"] and v["dt_limit"] == (0.02, 1.0)
    assert float(v["x"].min()) >= 0.1 and float(v["x"].max()) < 0.2
    assert float(v["dt"].min()) >= 0.03 and float(v["A"].max()) <= -0.1
    f = R.fwd_inputs(R.fwd_cases()[34])  # boundary a_strong
    assert bool((f["A"] == -10.0).all()) and f["D"] is None
    f = R.fwd_inputs(R.fwd_cases()[39])  # boundary z_zero
    assert bool((f["z"] == 0).all())


@pytest.mark.parametrize("case_id", [4, 13, 30])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_oracle_gradients_reproduce_the_reference_on_table_cases(case_id, dtype):
    case = R.bwd_cases()[case_id - 1]
    values = R.bwd_inputs(case)
    names = R.leaf_names(values)
    leaves = {n: values[n].to(dtype).requires_grad_(True) for n in names}
    out, final = O.ssd_chunked(*(leaves[n] for n in CORE), values["chunk_size"],
                               compute_dtype=None if dtype == torch.float64 else torch.float32,
                               **R.call_kwargs(values, leaves))
    dout, dfinal = R.bwd_upstream(case, out.shape, final.shape)
    outs, ups = R.bwd_selected(case, out, final, dout.to(dtype), dfinal.to(dtype))
    grads = torch.autograd.grad(outs, [leaves[n] for n in names], ups, allow_unused=True)
    for n, g in zip(names, grads):
        want = torch.from_numpy(GOLDEN[f"bwd{case_id:02d}_d{n}"])
        g = torch.zeros_like(leaves[n]) if g is None else g
        m = R.bwd_metrics(g, want)
        assert m["nrmse"] <= 2e-5 and m["cosine"] >= 1 - 1e-9, f"d{n}: {m}"  # fp32 rounding of the reference
    assert O.rel_l2(out.detach(), torch.from_numpy(GOLDEN[f"bwd{case_id:02d}_out"])) <= 2e-6
    assert O.rel_l2(final.detach(), torch.from_numpy(GOLDEN[f"bwd{case_id:02d}_final"])) <= 2e-6


@pytest.mark.parametrize("case_id", [12, 27, 35, 40])
def test_oracle_forward_reproduces_the_reference_on_table_cases(case_id):
    case = R.fwd_cases()[case_id - 1]
    values = R.fwd_inputs(case)
    v64 = {n: values[n].double() for n in R.leaf_names(values)}
    out, final = O.ssd_chunked(*(v64[n] for n in CORE), values["chunk_size"], compute_dtype=None,
                               **R.call_kwargs(values, v64))
    for name, got in (("out", out), ("final", final)):
        m = R.fwd_metrics(got, torch.from_numpy(GOLDEN[f"fwd{case_id:02d}_{name}"]))
        assert m["MERE"] < 1e-5 and m["MARE"] < 1e-3 and m["nan_inf"] == 0, f"{name}: {m}"
