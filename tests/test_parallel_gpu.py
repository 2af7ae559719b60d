"""Sequence-parallel and head-sharded SSD on two GPUs (NCCL), against the fp64 oracle of the full problem.

Needs two visible GPUs; skipped otherwise.  NVLS is switched off for the test processes: a rank that dies while
its memory is bound to an NVLink multicast object can disturb the other ranks' GPUs, and nothing here needs it.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu
WORLD = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "mamba-ascendc_b200"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev)
    try:
        from ascend_kernel import check_status, parallel as par

        shape = (2, 512, 4, 64, 64, 64, 2)
        x, dt, a, b, c = O.make_inputs(shape, 91)
        want = O.fp64_forward_backward(x, dt, a, b, c, 64, dt_softplus=True)
        n_out, n_fin = want[0].numel(), want[1].numel()
        errs = {}
        # ---- sequence parallel: this rank's half of the tokens, both forms of the boundary exchange
        l = shape[1] // WORLD
        sl = slice(rank * l, (rank + 1) * l)
        ref = [want[2][:, sl], want[3][:, sl], want[4], want[5][:, sl], want[6][:, sl]]
        for exchange, tag in (("chain", "sp"), ("allgather", "spag")):
            local = [x[:, sl].contiguous().to(dev).requires_grad_(True), dt[:, sl].contiguous().to(dev).requires_grad_(True),
                     a.to(dev).requires_grad_(True), b[:, sl].contiguous().to(dev).requires_grad_(True),
                     c[:, sl].contiguous().to(dev).requires_grad_(True)]
            out, final = par.mamba2_ssd_fwd_sequence_parallel(*local, 64, dt_softplus=True, exchange=exchange)
            loss = out.pow(2).sum() / n_out
            if rank == WORLD - 1:
                loss = loss + final.pow(2).sum() / n_fin
            loss.backward()
            check_status(dev)
            for t, w, nm in zip(local, ref, ["dx", "ddt", "dA", "dB", "dC"]):
                errs[f"{tag}_{nm}"] = (O.rel_l2(t.grad.cpu(), w), O.max_abs(t.grad.cpu(), w))
            errs[f"{tag}_out"] = (O.rel_l2(out.detach().cpu(), want[0][:, sl]), O.max_abs(out.detach().cpu(), want[0][:, sl]))
            if rank == WORLD - 1:
                errs[f"{tag}_final"] = (O.rel_l2(final.detach().cpu(), want[1]), O.max_abs(final.detach().cpu(), want[1]))
        # ---- head blocks: this rank's half of the heads, gathered
        og, fg = par.mamba2_ssd_fwd_head_sharded(*(t.to(dev) for t in (x, dt, a, b, c)), 64, dt_softplus=True, gather=True)
        check_status(dev)
        errs["heads_out"] = (O.rel_l2(og.cpu(), want[0]), O.max_abs(og.cpu(), want[0]))
        errs["heads_final"] = (O.rel_l2(fg.cpu(), want[1]), O.max_abs(fg.cpu(), want[1]))
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < WORLD, reason="needs two GPUs")
def test_two_gpu_ranks_match_fp64_oracle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(WORLD)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, errs in results:
        for name, (rel, mabs) in errs.items():
            assert rel <= 2e-3 and mabs <= 1e-2, f"rank {rank} {name}: rel-L2 {rel:.3e} max-abs {mabs:.3e}"
