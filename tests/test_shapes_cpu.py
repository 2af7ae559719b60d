"""Host-side shape reduction (ascend_kernel/shapes.py) on CPU: the fixed-shape call is played by the checker.

``run_general`` must turn any (L, P, N) into calls with headdim 64, state size 64 (or 128 without gradients)
and whole tiles of 128 tokens, and give the result and the gradients of the original problem.  Shapes follow
the reference's matrix (benchmarks/mamba2_shape_matrix.py:129-190).
"""
import importlib.util
import pathlib

import pytest
import torch

from oracle import ssd_oracle as O

_spec = importlib.util.spec_from_file_location(
    "ssd_shapes", pathlib.Path(__file__).resolve().parents[1] / "mamba-ascendc_b200" / "ascend_kernel" / "shapes.py")
shapes = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(shapes)


def _core_factory(needs_grad, calls):
    def core(x, dt, A, B, C, init, dt_bias, valid):
        # what the CUDA entry points accept
        assert x.shape[3] == 64 and x.shape[1] % 128 == 0
        assert B.shape[3] == 64 or (B.shape[3] == 128 and not needs_grad)
        for t in (x, dt, A, B, C):
            assert t.is_contiguous()
        calls.append((tuple(x.shape), B.shape[3], valid))
        if valid:  # padded tokens take no step: the kernel sets q = 0 there
            keep = (torch.arange(x.shape[1]) < valid).to(dt.dtype).view(1, -1, 1)
            q = O._discretise(dt, dt_bias, True, (0.0, float("inf"))) * keep
            return O.ssd_chunked(x, q, A, B, C, 128, dt_softplus=False, initial_states=init,
                                 return_final_state=True, compute_dtype=None)
        return O.ssd_chunked(x, dt, A, B, C, 128, dt_bias=dt_bias, dt_softplus=True, initial_states=init,
                             return_final_state=True, compute_dtype=None)

    return core


CASES = [
    # B, L, H, P, N, G
    (1, 16, 1, 8, 8, 1),       # generic_tiny
    (1, 65, 4, 16, 16, 2),     # generic_tail_l65
    (1, 256, 8, 32, 64, 2),    # aligned_p32_n64
    (2, 128, 4, 128, 64, 2),   # headdim_128: two virtual heads per head
    (1, 128, 2, 64, 128, 1),   # state size 128: two column blocks under autograd
    (1, 200, 4, 96, 160, 2),   # everything at once (P -> 128, N -> 192, ragged L)
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("with_grad", [False, True])
def test_run_general_matches_direct(case, with_grad):
    b, l, h, p, n, g = case
    gen = torch.Generator().manual_seed(7 + l + p + n)
    x = torch.randn(b, l, h, p, generator=gen, dtype=torch.float64)
    dt = torch.rand(b, l, h, generator=gen, dtype=torch.float64)
    A = -torch.rand(h, generator=gen, dtype=torch.float64)
    B = torch.randn(b, l, g, n, generator=gen, dtype=torch.float64)
    C = torch.randn(b, l, g, n, generator=gen, dtype=torch.float64)
    init = torch.randn(b, h, p, n, generator=gen, dtype=torch.float64)
    bias = torch.randn(h, generator=gen, dtype=torch.float64) * 0.1
    leaves = [x, dt, A, B, C, init, bias]
    if with_grad:
        for t in leaves:
            t.requires_grad_(True)
    calls = []
    out, final = shapes.run_general(_core_factory(with_grad, calls), x, dt, A, B, C, init, bias, with_grad)
    ref_out, ref_final = O.ssd_sequential(x, dt, A, B, C, dt_bias=bias, dt_softplus=True, initial_states=init,
                                          return_final_state=True)
    assert out.shape == ref_out.shape and final.shape == ref_final.shape
    assert out.is_contiguous() and final.is_contiguous()
    assert O.rel_l2(out, ref_out) < 1e-12 and O.rel_l2(final, ref_final) < 1e-12
    n_blocks = -(-n // 64)
    expected_calls = 1 if (n_blocks == 1 or (not with_grad and n_blocks == 2)) else n_blocks
    assert len(calls) == expected_calls
    if with_grad:
        w_out = torch.randn(ref_out.shape, generator=gen, dtype=torch.float64)
        w_fin = torch.randn(ref_final.shape, generator=gen, dtype=torch.float64)
        got = torch.autograd.grad((out * w_out).sum() + (final * w_fin).sum(), leaves)
        want = torch.autograd.grad((ref_out * w_out).sum() + (ref_final * w_fin).sum(), leaves)
        for a, r, name in zip(got, want, ("x", "dt", "A", "B", "C", "initial_states", "dt_bias")):
            assert a.shape == r.shape
            assert O.rel_l2(a, r) < 1e-10, name
