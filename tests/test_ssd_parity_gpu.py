"""Parity of the CUDA path with the fp64 oracle, through the public API (which calls the C ABI).

Tolerance (stated by the benchmark definition): relative L2 <= 2e-3 and max-abs <= 1e-2 for out, final
state and every gradient.  The split-bf16 tensor-core operands land two orders of magnitude inside it.
Shapes: the CPU-sized benchmark configurations, the reference's backward case table flavours
(mamba_ascendc/tests/bwd_m1_precision_common.py:15-59: one tile, several tiles, groups, odd head
counts, batch > 1), the golden fixtures, and full-size properties at the H256 shape.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

REL_L2_TOL = 2e-3
MAX_ABS_TOL = 1e-2
GOLDEN = Path(__file__).resolve().parent / "golden"


def _dev():
    return torch.device("cuda:0")


def _assert_close(got, want, name):
    r, m = O.rel_l2(got.cpu(), want), O.max_abs(got.cpu(), want)
    if float(want.abs().max()) == 0.0:  # an exactly-zero gradient: only the absolute bound applies
        r = 0.0 if m <= 1e-12 else float("inf")
    assert r <= REL_L2_TOL and m <= MAX_ABS_TOL, f"{name}: rel-L2 {r:.3e}, max-abs {m:.3e}"
    return r, m


def _run_fwd_bwd(inputs, chunk):
    from ascend_kernel import check_status, mamba2_ssd_fwd

    leaves = [t.to(_dev()).requires_grad_(True) for t in inputs]
    out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
    loss = O.loss_fn(out, final)
    loss.backward()
    check_status()
    return out.detach(), final.detach(), [t.grad for t in leaves]


# [B, L, H, P, N, chunk, G], seed
BWD_CASES = [
    (O.CONFIG_SHAPES[1], O.BASE_SEED + 1),      # benchmark configuration 1
    ((1, 256, 4, 64, 64, 64, 2), 11),           # two tiles, two groups (the golden fixture's inputs)
    ((2, 384, 6, 64, 64, 64, 2), 21),           # three tiles, three heads per group (odd), batch 2
    ((1, 512, 3, 64, 64, 128, 3), 22),          # one head per group
    ((3, 128, 8, 64, 64, 64, 1), 23),           # one tile, eight heads in one group
]


@pytest.mark.parametrize("shape,seed", BWD_CASES)
def test_forward_backward_matches_fp64_oracle(shape, seed):
    inputs = O.make_inputs(shape, seed)
    want = O.fp64_forward_backward(*inputs, shape[5], dt_softplus=True)
    out, final, grads = _run_fwd_bwd(inputs, shape[5])
    _assert_close(out, want[0], "out")
    _assert_close(final, want[1], "final_state")
    for g, w, name in zip(grads, want[2:], ["dx", "ddt", "dA", "dB", "dC"]):
        _assert_close(g, w, name)


FWD_CASES = [
    (O.CONFIG_SHAPES[0], O.BASE_SEED + 0),      # benchmark configuration 0 (N = 128)
    ((2, 256, 8, 64, 128, 128, 4), 31),
    ((1, 384, 5, 64, 128, 64, 1), 32),
]


@pytest.mark.parametrize("shape,seed", FWD_CASES)
def test_forward_dstate128_matches_fp64_oracle(shape, seed):
    from ascend_kernel import check_status, mamba2_ssd_fwd

    x, dt, a, b, c = O.make_inputs(shape, seed)
    want_out, want_final = O.ssd_chunked(x.double(), dt.double(), a.double(), b.double(), c.double(), shape[5],
                                         dt_softplus=True, return_final_state=True, compute_dtype=None)
    dev = _dev()
    out, final = mamba2_ssd_fwd(x.to(dev), dt.to(dev), a.to(dev), b.to(dev), c.to(dev), shape[5], dt_softplus=True,
                                return_final_state=True)
    check_status()
    _assert_close(out, want_out, "out")
    _assert_close(final, want_final, "final_state")
    only_out = mamba2_ssd_fwd(x.to(dev), dt.to(dev), a.to(dev), b.to(dev), c.to(dev), shape[5], dt_softplus=True)
    assert isinstance(only_out, torch.Tensor) and torch.equal(only_out, out)


@pytest.mark.parametrize("name", ["config0", "config1", "two_tiles_grouped"])
def test_against_reference_generated_golden(name):
    """Outputs of the reference's own ssd_sequential_ref (fp64) stored by tests/golden/make_golden.py."""
    z = np.load(GOLDEN / f"{name}.npz")
    shape = tuple(int(v) for v in z["shape"])
    inputs = O.make_inputs(shape, int(z["seed"]))
    if shape[4] == 64:
        out, final, grads = _run_fwd_bwd(inputs, shape[5])
        for g, key in zip(grads, ["dx", "ddt", "dA", "dB", "dC"]):
            _assert_close(g, torch.from_numpy(z[f"seq64_{key}"]), key)
    else:
        from ascend_kernel import mamba2_ssd_fwd

        dev = _dev()
        out, final = mamba2_ssd_fwd(*[t.to(dev) for t in inputs], shape[5], dt_softplus=True, return_final_state=True)
    _assert_close(out, torch.from_numpy(z["seq64_out"]), "out")
    _assert_close(final, torch.from_numpy(z["seq64_final"]), "final_state")


def test_configuration2_forward():
    """[4,2048,16,64,128,128,4], forward only, no final state requested."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    shape = O.CONFIG_SHAPES[2]
    x, dt, a, b, c = O.config_inputs(2)
    dev = _dev()
    out = mamba2_ssd_fwd(x.to(dev), dt.to(dev), a.to(dev), b.to(dev), c.to(dev), shape[5], dt_softplus=True,
                         return_final_state=False)
    check_status()
    assert isinstance(out, torch.Tensor)
    # fp64 oracle on the device the test runs on (the oracle is device agnostic), one batch at a time
    for bi in range(shape[0]):
        sl = slice(bi, bi + 1)
        want = O.ssd_chunked(x[sl].double().to(dev), dt[sl].double().to(dev), a.double().to(dev),
                             b[sl].double().to(dev), c[sl].double().to(dev), shape[5], dt_softplus=True,
                             compute_dtype=None)
        _assert_close(out[sl], want.cpu(), f"out[batch {bi}]")


def test_gradient_only_through_final_state_and_only_through_out():
    """Both gradient entry points work alone (mamba_ascendc/tests/test_mamba2_ssd_bwd_m1.py:121-133)."""
    from ascend_kernel import mamba2_ssd_fwd

    shape = (1, 256, 2, 64, 64, 64, 1)
    inputs = O.make_inputs(shape, 41)
    dev = _dev()
    for which in ("final", "out"):
        leaves = [t.to(dev).requires_grad_(True) for t in inputs]
        out, final = mamba2_ssd_fwd(*leaves, 64, dt_softplus=True, return_final_state=True)
        (final.pow(2).mean() if which == "final" else out.pow(2).mean()).backward()
        l64 = [t.double().requires_grad_(True) for t in inputs]
        o64, f64 = O.ssd_chunked(*l64, 64, dt_softplus=True, return_final_state=True, compute_dtype=None)
        g64 = torch.autograd.grad(f64.pow(2).mean() if which == "final" else o64.pow(2).mean(), l64,
                                  allow_unused=True)  # the final state does not depend on C
        g64 = [torch.zeros_like(t) if g is None else g for g, t in zip(g64, l64)]
        for leaf, w, nm in zip(leaves, g64, ["dx", "ddt", "dA", "dB", "dC"]):
            _assert_close(leaf.grad, w, f"{nm} ({which} only)")


def test_initial_states_forward_and_gradient():
    """initial_states [B,H,P,N] seeds the recurrence and receives a gradient (ssd_reference.py:43-53)."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    shape = (2, 384, 4, 64, 64, 64, 2)
    x, dt, a, b, c = O.make_inputs(shape, 44)
    init = torch.randn(2, 4, 64, 64, generator=torch.Generator().manual_seed(45))
    dev = _dev()
    leaves = [t.to(dev).requires_grad_(True) for t in (x, dt, a, b, c, init)]
    out, final = mamba2_ssd_fwd(*leaves[:5], 64, dt_softplus=True, initial_states=leaves[5], return_final_state=True)
    O.loss_fn(out, final).backward()
    check_status()
    l64 = [t.double().requires_grad_(True) for t in (x, dt, a, b, c, init)]
    o64, f64 = O.ssd_chunked(*l64[:5], 64, dt_softplus=True, initial_states=l64[5], return_final_state=True,
                             compute_dtype=None)
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    _assert_close(out.detach(), o64.detach(), "out")
    _assert_close(final.detach(), f64.detach(), "final_state")
    for leaf, w, nm in zip(leaves, g64, ["dx", "ddt", "dA", "dB", "dC", "dinitial"]):
        _assert_close(leaf.grad, w, nm)


@pytest.mark.parametrize("d_dims", [1, 2])
def test_full_feature_set_matches_fp64_oracle(d_dims):
    """D + z + dt_bias + softplus + initial_states + dt_limit (1e-3, 1.0): the reference benchmark's `full` mode
    (benchmarks/mamba2_backward_bench.py:159-165) and the feature modes of its backward case table
    (mamba_ascendc/tests/bwd_m1_precision_common.py:84-96)."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    shape = (2, 256, 4, 64, 64, 64, 2)
    b_, l_, h_, p_, n_ = shape[:5]
    x, dt, a, bm, cm = O.make_inputs(shape, 46)
    gen = torch.Generator().manual_seed(47)
    D = torch.randn(h_, generator=gen) if d_dims == 1 else torch.randn(h_, p_, generator=gen)
    z = torch.randn(b_, l_, h_, p_, generator=gen)
    bias = 0.5 * torch.randn(h_, generator=gen)
    init = torch.randn(b_, h_, p_, n_, generator=gen)
    limit = (1e-3, 1.0)
    dev = _dev()
    names = ["dx", "ddt", "dA", "dB", "dC", "dD", "dz", "d_dt_bias", "dinitial"]
    cpu = [x, dt, a, bm, cm, D, z, bias, init]
    leaves = [t.to(dev).requires_grad_(True) for t in cpu]
    out, final = mamba2_ssd_fwd(*leaves[:5], 64, D=leaves[5], z=leaves[6], dt_bias=leaves[7], dt_softplus=True,
                                dt_limit=limit, initial_states=leaves[8], return_final_state=True)
    O.loss_fn(out, final).backward()
    check_status()
    l64 = [t.double().requires_grad_(True) for t in cpu]
    o64, f64 = O.ssd_chunked(*l64[:5], 64, D=l64[5], z=l64[6], dt_bias=l64[7], dt_softplus=True, dt_limit=limit,
                             initial_states=l64[8], return_final_state=True, compute_dtype=None)
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    _assert_close(out.detach(), o64.detach(), "out")
    _assert_close(final.detach(), f64.detach(), "final_state")
    for leaf, w, nm in zip(leaves, g64, names):
        _assert_close(leaf.grad, w, nm)
    # forward-only path gives the same numbers
    with torch.no_grad():
        o2 = mamba2_ssd_fwd(*[t.detach() for t in leaves[:5]], 64, D=leaves[5].detach(), z=leaves[6].detach(),
                            dt_bias=leaves[7].detach(), dt_softplus=True, dt_limit=limit,
                            initial_states=leaves[8].detach())
    assert torch.equal(o2, out.detach())


@pytest.mark.parametrize("seqlen", [100, 300])
def test_ragged_sequence_length(seqlen):
    """L not a multiple of the tile: padded internally, like the reference's own padding to a chunk multiple
    (tests/mamba2/test_reference.py:202-216).  dt_limit with a positive minimum checks that padding takes no step."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    shape = (2, seqlen, 4, 64, 64, 64, 2)
    inputs = O.make_inputs(shape, 48)
    limit = (1e-2, 1.0)
    dev = _dev()
    leaves = [t.to(dev).requires_grad_(True) for t in inputs]
    out, final = mamba2_ssd_fwd(*leaves, 64, dt_softplus=True, dt_limit=limit, return_final_state=True)
    assert out.shape == inputs[0].shape
    O.loss_fn(out, final).backward()
    check_status()
    l64 = [t.double().requires_grad_(True) for t in inputs]
    o64, f64 = O.ssd_chunked(*l64, 64, dt_softplus=True, dt_limit=limit, return_final_state=True, compute_dtype=None)
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    _assert_close(out.detach(), o64.detach(), "out")
    _assert_close(final.detach(), f64.detach(), "final_state")
    for leaf, w, nm in zip(leaves, g64, ["dx", "ddt", "dA", "dB", "dC"]):
        assert leaf.grad.shape == w.shape
        _assert_close(leaf.grad, w, nm)


@pytest.mark.parametrize("seqlen,headdim", [(100, 64), (300, 64), (300, 128)])
def test_ragged_length_with_dt_bias_and_final_state_loss(seqlen, headdim):
    """Padding tokens take no step, so they must not feed d(dt_bias) either: with a loss on the final state the
    recurrence hands a gradient to every token of the last tile, padded ones included, and the dt stage has to
    drop it there.  headdim 128 runs as two virtual heads of 64 channels that share dt, A and the bias."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    shape = (2, seqlen, 4, headdim, 64, 64, 2)
    x, dt, a, bm, cm = O.make_inputs(shape, 49)
    bias = 0.5 * torch.randn(4, generator=torch.Generator().manual_seed(50))
    limit = (1e-2, 1.0)
    dev = _dev()
    cpu = [x, dt, a, bm, cm, bias]
    leaves = [t.to(dev).requires_grad_(True) for t in cpu]
    out, final = mamba2_ssd_fwd(*leaves[:5], 64, dt_bias=leaves[5], dt_softplus=True, dt_limit=limit,
                                return_final_state=True)
    O.loss_fn(out, final).backward()
    check_status()
    l64 = [t.double().requires_grad_(True) for t in cpu]
    o64, f64 = O.ssd_chunked(*l64[:5], 64, dt_bias=l64[5], dt_softplus=True, dt_limit=limit, return_final_state=True,
                             compute_dtype=None)
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    _assert_close(out.detach(), o64.detach(), "out")
    _assert_close(final.detach(), f64.detach(), "final_state")
    for leaf, w, nm in zip(leaves, g64, ["dx", "ddt", "dA", "dB", "dC", "d_dt_bias"]):
        _assert_close(leaf.grad, w, nm)


def test_no_softplus_path():
    from ascend_kernel import mamba2_ssd_fwd

    shape = (1, 256, 2, 64, 64, 64, 1)
    x, dt, a, b, c = O.make_inputs(shape, 42)
    dt = 0.01 + 0.1 * dt  # the reference benchmark's positive step sizes (mamba2_backward_bench.py:224-233)
    dev = _dev()
    leaves = [t.to(dev).requires_grad_(True) for t in (x, dt, a, b, c)]
    out, final = mamba2_ssd_fwd(*leaves, 64, dt_softplus=False, return_final_state=True)
    O.loss_fn(out, final).backward()
    want = O.fp64_forward_backward(x, dt, a, b, c, 64, dt_softplus=False)
    _assert_close(out, want[0], "out")
    for leaf, w, nm in zip(leaves, want[2:], ["dx", "ddt", "dA", "dB", "dC"]):
        _assert_close(leaf.grad, w, nm)


def test_run_to_run_bitwise_identical():
    """Fixed-order reductions: two runs give identical bits (the reference's determinism gate,
    mamba_ascendc/csrc/ops/mamba2_ssd_bwd/design.md:232-233)."""
    shape = (2, 256, 4, 64, 64, 64, 2)
    inputs = O.make_inputs(shape, 43)
    a = _run_fwd_bwd(inputs, 64)
    b = _run_fwd_bwd(inputs, 64)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    for ga, gb in zip(a[2], b[2]):
        assert torch.equal(ga, gb)


# ------------------------------------------------------------------ full-size checks at the H256 shape
def _h256_inputs(dev):
    """The configuration's own seeded inputs (CPU generator, seed 20260806 + 3), copied to the device."""
    return tuple(t.to(dev) for t in O.config_inputs(3))


def test_h256_full_size_slices_and_linearity():
    """Configuration 3 at full size, every element of every result.  Groups are independent, so the fp64
    oracle runs on the device one group at a time (all 8 batch rows of the group's 4 heads, which is what
    dA sums over) and each of the 64 group slices of out, final state, dx, ddt, dA, dB and dC is compared with
    it.  Size-independent property on top: the SSD map is linear in x for fixed dt, A, B, C."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    dev = _dev()
    b, l, h, p, n, chunk, g = O.CONFIG_SHAPES[3]
    r = h // g
    x, dt, a, bm, cm = _h256_inputs(dev)
    leaves = [t.requires_grad_(True) for t in (x, dt, a, bm, cm)]
    out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
    O.loss_fn(out, final).backward()
    check_status()
    n_out, n_fin = out.numel(), final.numel()
    for gi in range(g):
        hs = slice(gi * r, (gi + 1) * r)
        l64 = [x[:, :, hs].detach().double().requires_grad_(True), dt[:, :, hs].detach().double().requires_grad_(True),
               a[hs].detach().double().requires_grad_(True), bm[:, :, gi:gi + 1].detach().double().requires_grad_(True),
               cm[:, :, gi:gi + 1].detach().double().requires_grad_(True)]
        o64, f64 = O.ssd_chunked(*l64, chunk, dt_softplus=True, return_final_state=True, compute_dtype=None)
        loss = o64.pow(2).sum() / n_out + f64.pow(2).sum() / n_fin
        g64 = torch.autograd.grad(loss, l64)
        _assert_close(out[:, :, hs].detach(), o64.detach().cpu(), f"out[group {gi}]")
        _assert_close(final[:, hs].detach(), f64.detach().cpu(), f"final[group {gi}]")
        got = [x.grad[:, :, hs], dt.grad[:, :, hs], a.grad[hs], bm.grad[:, :, gi:gi + 1], cm.grad[:, :, gi:gi + 1]]
        for gg, w, nm in zip(got, g64, ["dx", "ddt", "dA", "dB", "dC"]):
            _assert_close(gg, w.cpu(), f"{nm}[group {gi}]")
    del leaves
    # linearity in x at full size
    with torch.no_grad():
        x0, dt0, a0, b0, c0 = (t.detach() for t in (x, dt, a, bm, cm))
        x2 = torch.randn_like(x0)
        o1 = mamba2_ssd_fwd(x0, dt0, a0, b0, c0, chunk, dt_softplus=True)
        o2 = mamba2_ssd_fwd(x2, dt0, a0, b0, c0, chunk, dt_softplus=True)
        o12 = mamba2_ssd_fwd(x0 + 0.5 * x2, dt0, a0, b0, c0, chunk, dt_softplus=True)
        check_status()
        lin = o1 + 0.5 * o2
        err = (o12 - lin).abs().max().item()
        rel = ((o12 - lin).norm() / lin.norm()).item()
        assert rel <= 1e-4 and err <= MAX_ABS_TOL, f"linearity: rel {rel:.3e}, max-abs {err:.3e}"


# Shapes outside the tile kernels' own (headdim 64, state 64): rows of the reference's shape matrix
# (benchmarks/mamba2_shape_matrix.py:129-190), reduced to kernel calls by ascend_kernel/shapes.py.
GENERAL_CASES = [
    ((1, 16, 1, 8, 8, 8, 1), 41),          # generic_tiny
    ((1, 65, 4, 16, 16, 32, 2), 42),       # generic_tail_l65
    ((1, 256, 8, 16, 32, 64, 2), 43),      # aligned_p16_n32
    ((1, 256, 8, 32, 64, 64, 2), 44),      # aligned_p32_n64
    ((2, 256, 4, 128, 64, 64, 2), 45),     # headdim_128 (smaller batch / length)
    ((1, 512, 8, 64, 128, 128, 2), 46),    # cube_n128_c128: backward at state size 128
    ((1, 1024, 4, 64, 128, 256, 4), 47),   # logical_chunk256
]


@pytest.mark.parametrize("shape,seed", GENERAL_CASES)
def test_general_shapes_forward_backward(shape, seed):
    inputs = O.make_inputs(shape, seed)
    want = O.fp64_forward_backward(*inputs, shape[5], dt_softplus=True)
    out, final, grads = _run_fwd_bwd(inputs, shape[5])
    assert out.shape == want[0].shape and final.shape == want[1].shape
    _assert_close(out, want[0], "out")
    _assert_close(final, want[1], "final_state")
    for g, w, name in zip(grads, want[2:], ["dx", "ddt", "dA", "dB", "dC"]):
        assert g.shape == w.shape
        _assert_close(g, w, name)


def test_recompute_policy_same_gradients_less_saved():
    """Saving only the inputs and re-running the forward stages in backward gives bitwise the same
    gradients and keeps less memory alive (mamba2_ssd_bwd/design.md:207-223 for the reference's policy)."""
    from ascend_kernel import SavedTensorStats, check_status, mamba2_ssd_fwd, set_save_policy

    shape = (2, 512, 8, 64, 64, 64, 2)
    inputs = O.make_inputs(shape, 51)
    results = {}
    for policy in ("save", "recompute"):
        previous = set_save_policy(policy)
        try:
            leaves = [t.to(_dev()).requires_grad_(True) for t in inputs]
            stats = SavedTensorStats()
            with stats.hooks():
                out, final = mamba2_ssd_fwd(*leaves, shape[5], dt_softplus=True, return_final_state=True)
            O.loss_fn(out, final).backward()
            check_status()
            results[policy] = ([t.grad.clone() for t in leaves], stats.unique_bytes)
        finally:
            set_save_policy(previous)
    for a, b in zip(results["save"][0], results["recompute"][0]):
        assert torch.equal(a, b)
    input_bytes = sum(t.numel() * 4 for t in inputs)
    assert results["recompute"][1] <= input_bytes + 4096
    assert results["save"][1] > results["recompute"][1] + inputs[0].numel() * 4  # out alone is as large as x


@pytest.mark.parametrize("shape", [
    (2, 4096, 48, 64, 64, 64, 12),   # 32 x 12 x 2 = 768 tiles of 128 tokens, four heads per group
    (2, 1408, 14, 64, 64, 128, 14),  # 11 x 14 x 2 = 308 tiles, one head per group: every carry of the tile walk
])
def test_persistent_kernels_walk_several_tiles_per_cta(shape):
    """More work items than SMs, so the persistent kernels (output kernel, dB/dC kernel) cross tile
    boundaries inside a CTA (positions are advanced incrementally, with carries from token tile to group to
    batch): sampled groups against the fp64 oracle (run on the device), and the whole result bitwise equal over
    repeated runs (a race would show as run-to-run differences)."""
    from ascend_kernel import check_status, mamba2_ssd_fwd

    dev = _dev()
    b, l, h, p, n, chunk, g = shape
    r = h // g
    inputs = [t.to(dev) for t in O.make_inputs(shape, 61)]
    results = []
    for _ in range(3):
        leaves = [t.clone().requires_grad_(True) for t in inputs]
        out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
        O.loss_fn(out, final).backward()
        check_status()
        results.append([out.detach(), final.detach()] + [t.grad for t in leaves])
    for other in results[1:]:
        for a_, b_ in zip(results[0], other):
            assert torch.equal(a_, b_)
    out, final, dx, ddt, da, db, dc = results[0]
    x, dt, a, bm, cm = inputs
    for gi in (0, g // 2 - 1, g - 1):
        hs = slice(gi * r, (gi + 1) * r)
        l64 = [x[:, :, hs].double().requires_grad_(True), dt[:, :, hs].double().requires_grad_(True),
               a[hs].double().requires_grad_(True), bm[:, :, gi:gi + 1].double().requires_grad_(True),
               cm[:, :, gi:gi + 1].double().requires_grad_(True)]
        o64, f64 = O.ssd_chunked(*l64, chunk, dt_softplus=True, return_final_state=True, compute_dtype=None)
        loss = o64.pow(2).sum() / out.numel() + f64.pow(2).sum() / final.numel()
        g64 = torch.autograd.grad(loss, l64)
        _assert_close(out[:, :, hs], o64.detach().cpu(), f"out[group {gi}]")
        _assert_close(final[:, hs], f64.detach().cpu(), f"final[group {gi}]")
        got = [dx[:, :, hs], ddt[:, :, hs], da[hs], db[:, :, gi:gi + 1], dc[:, :, gi:gi + 1]]
        for gg, w, nm in zip(got, g64, ["dx", "ddt", "dA", "dB", "dC"]):
            _assert_close(gg, w.cpu(), f"{nm}[group {gi}]")


@pytest.mark.parametrize("scale", [8.0, 40.0])
def test_strong_decay_takes_the_exact_paths(scale):
    """Decay far beyond the table fast path of the decay passes (more than e^60 across 32 tokens): the
    diagonal blocks fall back to one exp per element, off-diagonal factors underflow to zero.  Mixed heads:
    some weak, some strong, one with A = 0 (no decay at all)."""
    shape = (2, 384, 8, 64, 64, 64, 2)
    x, dt, a, bm, cm = O.make_inputs(shape, 71)
    a = a * torch.tensor([0.0, 0.1, 1.0, scale, scale, 0.5 * scale, 1.0, 2.0 * scale])
    want = O.fp64_forward_backward(x, dt, a, bm, cm, shape[5], dt_softplus=True)
    out, final, grads = _run_fwd_bwd((x, dt, a, bm, cm), shape[5])
    _assert_close(out, want[0], "out")
    _assert_close(final, want[1], "final_state")
    for g, w, name in zip(grads, want[2:], ["dx", "ddt", "dA", "dB", "dC"]):
        assert torch.isfinite(g).all(), name
        # the head with A = 0 has |dA| ~ 1e5 here: the absolute bound is taken relative to the largest entry
        r, m = O.rel_l2(g.cpu(), w), O.max_abs(g.cpu(), w)
        assert r <= REL_L2_TOL and m <= MAX_ABS_TOL * max(1.0, float(w.abs().max())), f"{name}: {r:.3e}, {m:.3e}"


@pytest.mark.parametrize("which", ["D", "z"])
@pytest.mark.parametrize("policy", ["save", "recompute"])
def test_skip_or_gate_alone(which, policy):
    """Only the D skip connection, or only the z gate, through the fused epilogue, under both save policies."""
    from ascend_kernel import check_status, mamba2_ssd_fwd, set_save_policy

    shape = (1, 384, 6, 64, 64, 64, 3)
    b_, l_, h_, p_ = shape[:4]
    x, dt, a, bm, cm = O.make_inputs(shape, 81)
    gen = torch.Generator().manual_seed(82)
    extra = torch.randn(h_, generator=gen) if which == "D" else torch.randn(b_, l_, h_, p_, generator=gen)
    dev = _dev()
    cpu = [x, dt, a, bm, cm, extra]
    leaves = [t.to(dev).requires_grad_(True) for t in cpu]
    previous = set_save_policy(policy)
    try:
        out, final = mamba2_ssd_fwd(*leaves[:5], 64, dt_softplus=True, return_final_state=True, **{which: leaves[5]})
        O.loss_fn(out, final).backward()
        check_status()
    finally:
        set_save_policy(previous)
    l64 = [t.double().requires_grad_(True) for t in cpu]
    o64, f64 = O.ssd_chunked(*l64[:5], 64, dt_softplus=True, return_final_state=True, compute_dtype=None,
                             **{which: l64[5]})
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    _assert_close(out.detach(), o64.detach(), "out")
    _assert_close(final.detach(), f64.detach(), "final_state")
    for leaf, w, nm in zip(leaves, g64, ["dx", "ddt", "dA", "dB", "dC", "d" + which]):
        _assert_close(leaf.grad, w, nm)


# ------------------------------------------------------------------ the two routes of the state stages
SCAN_CASES = [
    ((2, 256, 4, 64, 64, 64, 2), 101),    # two pairs per group
    ((2, 384, 6, 64, 64, 64, 2), 102),    # three heads per group: a full pair and a single head
    ((1, 512, 3, 64, 64, 128, 3), 103),   # one head per group
    ((3, 128, 12, 64, 64, 64, 2), 104),   # one tile, three pairs per group (the most the kernel keeps on chip)
]


@pytest.mark.parametrize("shape,seed", SCAN_CASES)
def test_fused_state_scan_route_matches_oracle_and_the_tile_parallel_route(shape, seed):
    """The state products fused with the inter-tile recurrence (one CTA per (batch, group) walking the tiles,
    running state in tensor memory) against the fp64 oracle, with an initial state and a gradient on the final
    state so that both ends of the recurrence matter; the tile-parallel route on the same inputs must agree
    to rounding, and the fused route must repeat bit for bit."""
    from ascend_kernel import check_status, mamba2_ssd_fwd, set_state_scan

    b_, l_, h_, p_, n_ = shape[:5]
    x, dt, a, bm, cm = O.make_inputs(shape, seed)
    init = torch.randn(b_, h_, p_, n_, generator=torch.Generator().manual_seed(seed + 1))
    cpu = [x, dt, a, bm, cm, init]
    dev = _dev()
    results = {}
    for mode in ("on", "on", "off"):
        previous = set_state_scan(mode)
        try:
            leaves = [t.to(dev).requires_grad_(True) for t in cpu]
            out, final = mamba2_ssd_fwd(*leaves[:5], shape[5], dt_softplus=True, initial_states=leaves[5],
                                        return_final_state=True)
            O.loss_fn(out, final).backward()
            check_status()
        finally:
            set_state_scan(previous)
        results.setdefault(mode, []).append([out.detach(), final.detach()] + [t.grad for t in leaves])
    l64 = [t.double().requires_grad_(True) for t in cpu]
    o64, f64 = O.ssd_chunked(*l64[:5], shape[5], dt_softplus=True, initial_states=l64[5], return_final_state=True,
                             compute_dtype=None)
    g64 = torch.autograd.grad(O.loss_fn(o64, f64), l64)
    names = ["out", "final_state", "dx", "ddt", "dA", "dB", "dC", "dinitial"]
    want = [o64.detach(), f64.detach()] + list(g64)
    for got, w, nm in zip(results["on"][0], want, names):
        _assert_close(got, w, f"{nm} (fused)")
    for got, w, nm in zip(results["off"][0], want, names):
        _assert_close(got, w, f"{nm} (tile-parallel)")
    for a_, b_t in zip(results["on"][0], results["on"][1]):
        assert torch.equal(a_, b_t)
    for a_, b_t, nm in zip(results["on"][0], results["off"][0], names):
        assert O.rel_l2(a_.cpu(), b_t.cpu()) <= 1e-5, nm


def test_state_scan_route_is_chosen_by_the_number_of_chains():
    from ascend_kernel import mamba2 as M

    dev = _dev()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    x = torch.empty(8, 4096, 256, 64, device="meta")
    bm = torch.empty(8, 4096, 64, 64, device="meta")
    assert M._use_state_scan(M.make_shape(x, bm, True), dev) == (2 * 8 * 64 >= 3 * sms)   # the H256 shape
    few = M.make_shape(torch.empty(4, 4096, 6, 64, device="meta"), torch.empty(4, 4096, 1, 64, device="meta"), True)
    assert not M._use_state_scan(few, dev)                                               # configuration 4
    wide = M.make_shape(torch.empty(8, 128, 16, 64, device="meta"), torch.empty(8, 128, 1, 64, device="meta"), True)
    previous = M.set_state_scan("on")
    try:
        assert not M._use_state_scan(wide, dev)   # 16 heads per group: more pair states than fit on chip
    finally:
        M.set_state_scan(previous)


def test_long_sequence_backward_walks_the_reverse_scan_in_blocks():
    """More than 384 tiles (49152 tokens): the tile-parallel reverse state scan keeps its per-tile partial sums
    in shared memory and walks longer sequences in blocks."""
    from ascend_kernel import set_state_scan

    shape = (1, 128 * 390, 1, 64, 64, 64, 1)
    x, dt, a, bm, cm = O.make_inputs(shape, 111)
    dt = 0.05 * dt  # slow decay, so that early tiles still reach the final state
    want = O.fp64_forward_backward(x, dt, a, bm, cm, shape[5], dt_softplus=False)
    previous = set_state_scan("off")
    try:
        from ascend_kernel import check_status, mamba2_ssd_fwd

        leaves = [t.to(_dev()).requires_grad_(True) for t in (x, dt, a, bm, cm)]
        out, final = mamba2_ssd_fwd(*leaves, shape[5], dt_softplus=False, return_final_state=True)
        O.loss_fn(out, final).backward()
        check_status()
    finally:
        set_state_scan(previous)
    _assert_close(out.detach(), want[0], "out")
    _assert_close(final.detach(), want[1], "final_state")
    for leaf, w, nm in zip(leaves, want[2:], ["dx", "ddt", "dA", "dB", "dC"]):
        r, m = O.rel_l2(leaf.grad.cpu(), w), O.max_abs(leaf.grad.cpu(), w)
        assert r <= REL_L2_TOL and m <= MAX_ABS_TOL * max(1.0, float(w.abs().max())), f"{nm}: {r:.3e}, {m:.3e}"


@pytest.mark.parametrize("d_dims,with_z", [(1, True), (2, True), (1, False), (0, True)])
def test_forward_without_gradients_with_skip_and_gate(d_dims, with_z):
    """Forward without gradients: D and z are applied by the element-wise epilogue pass (ssd_gate_skip_fwd), through
    the public API and called directly on a plain SSD output."""
    from ascend_kernel import check_status, mamba2 as M, mamba2_ssd_fwd

    shape = (2, 256, 6, 64, 64, 64, 3)
    b_, l_, h_, p_ = shape[:4]
    x, dt, a, bm, cm = (t.to(_dev()) for t in O.make_inputs(shape, 121))
    gen = torch.Generator().manual_seed(122)
    D = None if d_dims == 0 else (torch.randn(h_, generator=gen) if d_dims == 1 else torch.randn(h_, p_, generator=gen)).to(_dev())
    z = torch.randn(b_, l_, h_, p_, generator=gen).to(_dev()) if with_z else None
    out, final = mamba2_ssd_fwd(x, dt, a, bm, cm, 64, D=D, z=z, dt_softplus=True, return_final_state=True)
    y = mamba2_ssd_fwd(x, dt, a, bm, cm, 64, dt_softplus=True)
    staged = M.gate_forward(y, x, bm, D, z)
    check_status()
    want = O.ssd_chunked(*(t.double().cpu() for t in (x, dt, a, bm, cm)), 64, D=None if D is None else D.double().cpu(),
                         z=None if z is None else z.double().cpu(), dt_softplus=True, compute_dtype=None)
    _assert_close(out, want, "out (public API)")
    _assert_close(staged, want, "out (direct call)")
    assert torch.equal(out, staged)
