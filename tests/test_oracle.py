"""The oracle (oracle/ssd_oracle.py) against the fixtures the reference produced (tests/golden/*.npz).

Mirrors the reference's CPU tier (tests/mamba2/test_reference.py): segsum known answers, chunked form
against the sequential form, groups, ragged lengths, optional inputs, final-state layout.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import ssd_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["config0", "config1", "two_tiles_grouped", "ragged_len", "optional_inputs"]


def _load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    shape = tuple(int(v) for v in z["shape"])
    inputs = O.make_inputs(shape, int(z["seed"]))
    extra, limit = {}, (0.0, float("inf"))
    if bool(z["optional"]):
        b, l, h, p, n, _c, _g = shape
        gen = torch.Generator().manual_seed(int(z["seed"]) + 1000)
        extra = dict(D=torch.randn(h, generator=gen), z=torch.randn(b, l, h, p, generator=gen),
                     dt_bias=0.1 * torch.randn(h, generator=gen),
                     initial_states=torch.randn(b, h, p, n, generator=gen))
        limit = (1e-3, 1.0)
    return z, shape, inputs, extra, limit


def test_segsum_known_answer():
    z = np.load(GOLDEN / "segsum.npz")
    got = O.segsum(torch.from_numpy(z["x"]))
    want = torch.from_numpy(z["segsum"])
    assert torch.equal(torch.isinf(got), torch.isinf(want))
    finite = ~torch.isinf(want)
    assert torch.allclose(got[finite], want[finite], atol=1e-6)
    # tests/mamba2/test_reference.py:13-23: unit diagonal, zero above it after exp
    e = torch.exp(got)
    assert torch.allclose(torch.diagonal(e), torch.ones(4))
    assert e[0, 1] == 0 and e[0, 2] == 0 and e[1, 0] > 1


@pytest.mark.parametrize("name", CASES)
def test_sequential_fp64_matches_reference(name):
    z, shape, (x, dt, a, b, c), extra, limit = _load(name)
    e64 = {k: v.double() for k, v in extra.items()}
    out, final = O.ssd_sequential(x.double(), dt.double(), a.double(), b.double(), c.double(), dt_softplus=True,
                                  dt_limit=limit, return_final_state=True, **e64)
    assert O.max_abs(out, torch.from_numpy(z["seq64_out"])) < 1e-11
    assert O.max_abs(final, torch.from_numpy(z["seq64_final"])) < 1e-11
    assert final.shape == (shape[0], shape[2], shape[3], shape[4])  # [B,H,P,N]


@pytest.mark.parametrize("name", CASES)
def test_chunked_fp64_matches_sequential_reference(name):
    z, shape, (x, dt, a, b, c), extra, limit = _load(name)
    e64 = {k: v.double() for k, v in extra.items()}
    out, final = O.ssd_chunked(x.double(), dt.double(), a.double(), b.double(), c.double(), shape[5],
                               dt_softplus=True, dt_limit=limit, return_final_state=True, compute_dtype=None, **e64)
    assert out.dtype == torch.float64
    assert O.rel_l2(out, torch.from_numpy(z["seq64_out"])) < 1e-12
    assert O.rel_l2(final, torch.from_numpy(z["seq64_final"])) < 1e-12


@pytest.mark.parametrize("name", CASES)
def test_chunked_fp32_matches_reference_chunked(name):
    """compute_dtype=float32 is the reference's own public path (fp32 inside); same rounding regime."""
    z, shape, (x, dt, a, b, c), extra, limit = _load(name)
    out, final = O.ssd_chunked(x, dt, a, b, c, shape[5], dt_softplus=True, dt_limit=limit,
                               return_final_state=True, **extra)
    assert out.dtype == torch.float32
    assert O.rel_l2(out, torch.from_numpy(z["chunk32_out"])) < 2e-6
    assert O.rel_l2(final, torch.from_numpy(z["chunk32_final"])) < 2e-6
    # and the fp32 path stays within the reference's own cross-check bound (test_reference.py:45-80: 1e-3)
    assert O.max_abs(out, torch.from_numpy(z["seq64_out"])) < 1e-3 * max(1.0, float(np.abs(z["seq64_out"]).max()))


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("sequential", [False, True])
def test_fp64_gradients_match_reference_autograd(name, sequential):
    """Gradients of mean(out^2) + mean(final^2) against the reference's fp64 autograd; the case with optional
    inputs also pins dD, dz, d(dt_bias) and d(initial_states)."""
    z, shape, (x, dt, a, b, c), extra, limit = _load(name)
    core = [t.double().requires_grad_(True) for t in (x, dt, a, b, c)]
    e64 = {k: v.double().requires_grad_(True) for k, v in extra.items()}
    if sequential:
        out, final = O.ssd_sequential(*core, dt_softplus=True, dt_limit=limit, return_final_state=True, **e64)
    else:
        out, final = O.ssd_chunked(*core, shape[5], dt_softplus=True, dt_limit=limit, return_final_state=True,
                                   compute_dtype=None, **e64)
    grads = torch.autograd.grad(O.loss_fn(out, final), core + list(e64.values()))
    keys = ["dx", "ddt", "dA", "dB", "dC"] + [f"d{k}" for k in e64]
    assert len(keys) == (9 if extra else 5)
    for got, key in zip(grads, keys):
        assert O.rel_l2(got, torch.from_numpy(z[f"seq64_{key}"])) < 1e-11, key
    if not extra:  # the helper the GPU tests call gives the same numbers
        res = O.fp64_forward_backward(x, dt, a, b, c, shape[5], dt_softplus=True, sequential=sequential)
        for got, ref in zip(res[2:], grads):
            assert torch.equal(got, ref)


def test_chunk_size_does_not_change_the_result():
    """The chunk length is a blocking parameter only; the CUDA path relies on this to tile by 128 tokens."""
    x, dt, a, b, c = (t.double() for t in O.make_inputs((1, 256, 2, 8, 8, 64, 1), 5))
    outs = [O.ssd_chunked(x, dt, a, b, c, cs, dt_softplus=True, return_final_state=True, compute_dtype=None)
            for cs in (32, 64, 128, 256)]
    for o, f in outs[1:]:
        assert O.rel_l2(o, outs[0][0]) < 1e-12 and O.rel_l2(f, outs[0][1]) < 1e-12


def test_config_shapes_and_distributions():
    x, dt, a, b, c = O.config_inputs(1)
    assert x.shape == (1, 128, 2, 64) and dt.shape == (1, 128, 2) and a.shape == (2,)
    assert b.shape == c.shape == (1, 128, 1, 64)
    assert (dt >= 0).all() and (dt < 1).all() and (a <= 0).all() and (a > -1).all()
