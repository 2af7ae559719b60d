"""Host-side multi-GPU logic on CPU: two gloo ranks, the checker (oracle) as the local SSD call.

Covers the head-block partition (no collective on the data path) and the sequence-parallel mode (boundary
state sent r -> r+1, its gradient r+1 -> r, dA all-reduced; and the all-gather form of the same exchange),
each against the single-process result; the fold of the all-gather form also on four simulated ranks.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O

WORLD = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_op(x, dt, A, B, C, chunk_size, dt_softplus=False, initial_states=None, return_final_state=False):
    return O.ssd_chunked(x, dt, A, B, C, chunk_size, dt_softplus=dt_softplus, initial_states=initial_states,
                         return_final_state=return_final_state, compute_dtype=None)


def _worker(rank, port, mode, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "mamba-ascendc_b200"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        # import the module file directly: the package __init__ loads the CUDA library, which a CPU rank need not
        import importlib.util
        spec = importlib.util.spec_from_file_location("ssd_parallel", root / "mamba-ascendc_b200/ascend_kernel/parallel.py")
        par = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(par)
        shape = (2, 256, 4, 8, 8, 64, 2)
        x, dt, a, b, c = (t.double() for t in O.make_inputs(shape, 77))
        full = [t.clone().requires_grad_(True) for t in (x, dt, a, b, c)]
        o_full, f_full = _oracle_op(*full, 64, dt_softplus=True, return_final_state=True)
        O.loss_fn(o_full, f_full).backward()
        if mode == "heads":
            h0, h1, g0, g1 = par.head_block(rank, WORLD, shape[2], shape[6])
            local = [t.clone().requires_grad_(True) for t in par.shard_by_heads(x, dt, a, b, c, rank, WORLD)]
            out, final = _oracle_op(*local, 64, dt_softplus=True, return_final_state=True)
            # the loss of the full problem restricted to this block, with the full problem's normalisation
            (out.pow(2).sum() / o_full.numel() + final.pow(2).sum() / f_full.numel()).backward()
            want = [full[0].grad[:, :, h0:h1], full[1].grad[:, :, h0:h1], full[2].grad[h0:h1],
                    full[3].grad[:, :, g0:g1], full[4].grad[:, :, g0:g1]]
            errs = [O.rel_l2(l.grad, w) for l, w in zip(local, want)]
            errs += [O.rel_l2(out, o_full[:, :, h0:h1]), O.rel_l2(final, f_full[:, h0:h1])]
            og, fg = par.mamba2_ssd_fwd_head_sharded(x, dt, a, b, c, 64, dt_softplus=True, gather=True, op=_oracle_op)
            errs += [O.rel_l2(og, o_full), O.rel_l2(fg, f_full)]
        else:
            l = shape[1] // WORLD
            sl = slice(rank * l, (rank + 1) * l)
            local = [x[:, sl].clone().requires_grad_(True), dt[:, sl].clone().requires_grad_(True),
                     a.clone().requires_grad_(True), b[:, sl].clone().requires_grad_(True),
                     c[:, sl].clone().requires_grad_(True)]
            out, final = par.mamba2_ssd_fwd_sequence_parallel(*local, 64, dt_softplus=True, op=_oracle_op,
                                                              exchange="allgather" if mode == "sequence_allgather"
                                                              else "chain")
            loss = out.pow(2).sum() / o_full.numel()
            if rank == WORLD - 1:
                loss = loss + final.pow(2).sum() / f_full.numel()
            loss.backward()
            want = [full[0].grad[:, sl], full[1].grad[:, sl], full[2].grad, full[3].grad[:, sl], full[4].grad[:, sl]]
            errs = [O.rel_l2(t.grad, w) for t, w in zip(local, want)]
            errs.append(O.rel_l2(out, o_full[:, sl]))
            if rank == WORLD - 1:
                errs.append(O.rel_l2(final, f_full))
        q.put((rank, max(errs)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["heads", "sequence", "sequence_allgather"])
def test_two_gloo_ranks_match_single_process(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, mode, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(WORLD)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 1e-10, f"rank {rank}: {err}"


def test_all_gather_fold_equals_the_chain_on_four_blocks():
    """fold_inflow / fold_outflow against the plain chain, with random per-block outflows and decays."""
    import importlib.util
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("ssd_parallel", root / "mamba-ascendc_b200/ascend_kernel/parallel.py")
    par = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(par)
    world = 4
    gen = torch.Generator().manual_seed(3)
    finals = [torch.randn(2, 3, 4, 5, generator=gen, dtype=torch.float64) for _ in range(world)]
    d0s = [torch.randn(2, 3, 4, 5, generator=gen, dtype=torch.float64) for _ in range(world)]
    logs = [-torch.rand(2, 3, generator=gen, dtype=torch.float64) for _ in range(world)]
    state = torch.zeros(2, 3, 4, 5, dtype=torch.float64)
    for r in range(world):
        got = par.fold_inflow(r, finals, logs)
        assert (got is None and r == 0) or torch.allclose(got, state, atol=1e-14)
        state = torch.exp(logs[r])[..., None, None] * state + finals[r]
    grad = torch.zeros(2, 3, 4, 5, dtype=torch.float64)  # arriving at the last rank's final state
    for r in range(world - 1, -1, -1):
        got = par.fold_outflow(r, world, d0s, logs)
        assert (got is None and r == world - 1) or torch.allclose(got, grad, atol=1e-14)
        grad = d0s[r] + torch.exp(logs[r])[..., None, None] * grad  # what rank r hands back in the chain


def test_head_block_partition():
    import importlib.util
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("ssd_parallel", root / "mamba-ascendc_b200/ascend_kernel/parallel.py")
    par = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(par)
    assert par.head_block(3, 8, 256, 64) == (96, 128, 24, 32)
    blocks = [par.head_block(r, 4, 16, 4) for r in range(4)]
    assert [b[:2] for b in blocks] == [(0, 4), (4, 8), (8, 12), (12, 16)]
    with pytest.raises(ValueError):
        par.head_block(0, 3, 16, 4)  # groups do not divide over the ranks
    with pytest.raises(ValueError):
        par.head_block(4, 4, 16, 4)


def _failing_worker(rank, port, q):
    """Sequence-parallel exchange in which rank 0 fails before it sends its boundary state."""
    import datetime
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "mamba-ascendc_b200"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=datetime.timedelta(seconds=5))
    import importlib.util
    spec = importlib.util.spec_from_file_location("ssd_parallel", root / "mamba-ascendc_b200/ascend_kernel/parallel.py")
    par = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(par)
    shape = (1, 128, 2, 8, 8, 64, 1)
    x, dt, a, b, c = (t.double() for t in O.make_inputs(shape, 78))
    l = shape[1] // WORLD
    sl = slice(rank * l, (rank + 1) * l)
    if rank == 0:
        q.put((rank, "left"))  # the failure: this rank leaves between steps, with nothing in flight
        return
    try:
        par.mamba2_ssd_fwd_sequence_parallel(x[:, sl], dt[:, sl], a, b[:, sl], c[:, sl], 64, dt_softplus=True,
                                             op=_oracle_op)
        q.put((rank, "no error"))
    except Exception as e:  # noqa: BLE001  (the process-group timeout or a closed connection)
        q.put((rank, "error: " + type(e).__name__))


def test_sequence_parallel_peer_failure_surfaces_on_the_host():
    """A rank that never sends its boundary state: the waiting rank gets a host-side error within the
    process-group timeout instead of hanging (no device-side wait on a peer exists anywhere)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(WORLD))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    assert results[0] == "left"
    assert results[1].startswith("error"), results[1]
