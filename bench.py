"""Benchmark of the Mamba-2 SSD forward + backward path at the H256 training shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling strong|weak]
                    [--mode heads|sp] [--heads H] [--workload h256|vmamba2]

One step = one forward + backward of ``[B,L,H,P,N,chunk,G] = [8,4096,256,64,64,64,64]`` (fp32 public tensors,
dt_softplus, final state returned, gradients for x, dt, A, B, C).  With N > 1 (launched by
``torch.distributed.run``) the ONE problem is sharded by group-aligned head blocks -- rank r owns heads
``[r*256/N, (r+1)*256/N)`` and their groups -- which needs no collective, so ``scaling`` is "strong" and
``value`` is the whole problem's flops over the slowest rank's time.  ``--scaling weak`` gives every rank the
full shape instead (an N x 256-head problem); at N > 1 its number is also reported under ``secondary``.
``--mode sp`` times the optional sequence-parallel mode (tokens sharded, boundary state exchanged over NCCL).
Rank 0 prints ONE JSON line.

``value`` is algorithmic TFLOP/s (6.7001e11 flop per step, dense tiles, forward x 3) with inputs resident in
HBM, timed with CUDA events over exactly K steps, max over ranks; the upstream gradients of the loss
mean(out^2) + mean(final^2) are precomputed, so the loss itself is outside ``value`` and inside ``e2e``.
``e2e`` repeats the step with the inputs in pinned host memory and the gradients returned to pinned host
memory inside the timed region, as an upload / compute / download pipeline over the same K steps.
``roofline`` describes the slowest kernel of the step, timed live with CUDA events on the launching stream.
``cpu_baseline`` / ``--impl reference`` time the reference's own CPU function (``ssd_chunk_scan_ref`` from the
file the build step places under oracle/_ref, fp32, all host threads; the pinned port oracle/ssd_oracle.py
where that file is absent) on a bounded sample of the same workload.  ``secondary`` (one GPU only) carries
the other configurations' numbers.  Inputs are synthetic (seeded).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "mamba-ascendc_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

H256 = (8, 4096, 256, 64, 64, 64, 64)  # benchmark configuration 3
CONFIG2 = (4, 2048, 16, 64, 128, 128, 4)
WORKLOAD = "config3 H256 fwd+bwd [B,L,H,P,N,chunk,G]=[8,4096,256,64,64,64,64], dt_softplus, final state"
METRIC = "ssd_fwd_bwd_tflops_h256"
TILE = 128
SEED = 20260806 + 3  # the reference benchmark's seed (benchmarks/mamba2_backward_bench.py:219) + configuration index


def bench_config(world: int, scaling: str, mode: str) -> dict:
    """The ``config`` object; both arms print the same one for the same command line."""
    if mode == "sp":
        par = f"{world} x token-block shard (sequence parallel), boundary state over NCCL"
    elif scaling == "strong":
        par = (f"{world} x head-block shard of the one problem ({H256[2] // world} heads / {H256[6] // world} groups "
               "per GPU), no collective")
    else:
        par = f"{world} x the full shape (head blocks of an {world}x256-head problem), no collective"
    return {"workload": WORKLOAD, "l2": "inputs (3.2 GB in total) are larger than the 126 MB L2",
            "parallelism": par, "tile_tokens": TILE, "loss": "excluded from value, included in e2e"}


def forward_flops(shape) -> float:
    """Dense-tile GEMM work of the chunked algorithm at the configuration's own chunk length:
    B*K*[G*2T^2N + H*(2T^2P + 4TNP)]; backward = 2x forward."""
    b, l, h, p, n, t, g = shape
    k = l // t
    return float(b * k * (g * 2 * t * t * n + h * (2 * t * t * p + 4 * t * n * p)))


def step_flops(shape) -> float:
    return 3.0 * forward_flops(shape)


def path_bytes(shape) -> float:
    """Compulsory HBM bytes of forward + backward: every input read once per pass, every output written once."""
    b, l, h, p, n, _t, g = shape
    x, dt, bc, fin = b * l * h * p, b * l * h, b * l * g * n, b * h * p * n
    fwd = x + dt + h + 2 * bc + x + fin
    bwd = x + dt + h + 2 * bc + x + fin + x + dt + h + 2 * bc
    return 4.0 * (fwd + bwd)


def forward_bytes(shape, final: bool) -> float:
    b, l, h, p, n, _t, g = shape
    return 4.0 * (2 * b * l * h * p + b * l * h + h + 2 * b * l * g * n + (b * h * p * n if final else 0))


def stage_bytes(shape) -> dict:
    """Algorithmic bytes of each kernel launch: its own inputs read once and outputs written once (fp32)."""
    b, l, h, p, n, _t, g = shape
    k = l // TILE
    x, dt, bc, st, fin = b * l * h * p, b * l * h, b * l * g * n, b * h * k * p * n, b * h * p * n
    words = {
        "mamba2_ssd_dt_cumsum": dt + h + 2 * dt,
        "mamba2_ssd_chunk_state": x + bc + 2 * dt + st,
        "mamba2_ssd_state_passing": 2 * st + fin + dt // TILE,
        "mamba2_ssd_chunk_state_scan": x + bc + 2 * dt + st + fin,
        "mamba2_ssd_chunk_scan": x + 2 * bc + st + 2 * dt + x,
        "mamba2_ssd_chunk_state_bwd": x + bc + 2 * dt + st,
        "mamba2_ssd_state_passing_bwd": 2 * st + fin,
        "mamba2_ssd_chunk_state_scan_bwd": x + bc + 2 * dt + st + fin,
        "mamba2_ssd_chunk_dx_bwd": 3 * x + 2 * bc + st + 3 * dt + x + dt,
        "mamba2_ssd_chunk_dbc_bwd": 2 * x + 2 * bc + 2 * st + 2 * dt + 2 * bc + b * h * k,
        "mamba2_ssd_dt_bwd": 2 * dt + 2 * b * h * k,
    }
    return {name: 4.0 * w for name, w in words.items()}


def measured_peaks() -> dict:
    """Roofline denominators: the pool's measured copy bandwidth and bf16 GEMM rate if the file is present,
    else the recorded fallback (6650 GB/s, 1590 TFLOP/s)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


# DRAM bytes per launch at the H256 shape from ncu (dram__bytes_read.sum + dram__bytes_write.sum), captured on
# the reduced cases ``--heads 32`` (1/8 of the heads) and, for the fused state kernels, ``--seqlen 512`` (1/8 of
# the tokens), where traffic is proportional to the head count / the length, and scaled by 8.  Each entry names
# the kernel source it was captured from and that file's sha256 prefix at capture time:
# when the source has changed since, the figure is stale and ``roofline.traffic`` is reported as null.
TRAFFIC = {
    "mamba2_ssd_chunk_scan": (8 * (546.0e6 + 230.9e6), "ssd_chunk_scan.cu", "8d8320f7bc1f"),
    "mamba2_ssd_chunk_state_scan": (8 * (344.0e6 + 133.3e6), "ssd_state_scan.cu", "0a31a50df5b1"),
    "mamba2_ssd_chunk_state_scan_bwd": (8 * (373.3e6 + 107.0e6), "ssd_state_scan.cu", "0a31a50df5b1"),
    "mamba2_ssd_chunk_state": (8 * (344.0e6 + 106.4e6), "ssd_chunk_state.cu", "732394ea328c"),
    "mamba2_ssd_chunk_state_bwd": (8 * (344.0e6 + 107.9e6), "ssd_chunk_state.cu", "732394ea328c"),
    "mamba2_ssd_state_passing": (8 * (135.3e6 + 80.2e6), "ssd_scan.cu", "87477650b721"),
    "mamba2_ssd_state_passing_bwd": (8 * (139.5e6 + 77.2e6), "ssd_scan.cu", "87477650b721"),
    "mamba2_ssd_chunk_dx_bwd": (8 * (1088.7e6 + 254.1e6), "ssd_bwd_dx.cu", "19a67c9b991b"),
    "mamba2_ssd_chunk_dbc_bwd": (8 * (949.3e6 + 119.1e6), "ssd_bwd_dbc.cu", "b042aaed86e7"),
}


def traffic_of(stage: str):
    entry = TRAFFIC.get(stage)
    if entry is None:
        return None
    nbytes, source, sha = entry
    path = ROOT / "mamba-ascendc_b200" / "csrc" / source
    if not sha or not path.exists() or hashlib.sha256(path.read_bytes()).hexdigest()[:12] != sha:
        return None
    return nbytes


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (reading only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        """Start sampling and wait (at most 3 s) for the first sample, so that the tool's start-up time does
        not eat a short timed region."""
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
            return
        t0 = time.time()
        while time.time() - t0 < 3.0 and self._rows() == 0:
            time.sleep(0.02)

    def _rows(self) -> int:
        try:
            return sum(1 for _ in open(self.file.name))
        except OSError:
            return 0

    def mark(self) -> None:
        """The timed region starts here: earlier samples (warm-up) are not counted."""
        self.first = self._rows()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        first = getattr(self, "first", 0)
        if len(rows) > first:  # a region shorter than one sampling interval keeps the sample just before it
            rows = rows[max(first - 1, 0):]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.strip().lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- the reference's CPU path
CPU_SAMPLE_SHAPE = (1, 4096, 32, 64, 64, 64, 8)  # 1/64 of the workload: one batch row, 8 of the 64 groups
CPU_SAMPLE_TEXT = "one forward+backward of a [1,4096,32,64,64,64,8] slice (1/64 of the workload: 1 batch row, 8 groups)"


def cpu_inputs(shape, seed: int):
    b, l, h, p, n, _t, g = shape
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(b, l, h, p, generator=gen)
    dt = torch.rand(b, l, h, generator=gen)
    a = -torch.rand(h, generator=gen)
    bm = torch.randn(b, l, g, n, generator=gen)
    cm = torch.randn(b, l, g, n, generator=gen)
    return [x, dt, a, bm, cm]


def reference_cpu_function():
    """(callable, kind): the reference's ``ssd_chunk_scan_ref`` from the unmodified file under oracle/_ref
    ("reference"), or the pinned port of it ("port") where that file is absent."""
    ref_file = ROOT / "oracle" / "_ref" / "ssd_reference.py"
    if ref_file.exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location("ssd_reference_unmodified", ref_file)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        return mod.ssd_chunk_scan_ref, "reference"
    from oracle import ssd_oracle as O

    return O.ssd_chunked, "port"


def time_cpu_reference(repeats: int, warmup: int):
    fn, kind = reference_cpu_function()
    inputs = cpu_inputs(CPU_SAMPLE_SHAPE, SEED)

    def step():
        leaves = [t.detach().requires_grad_(True) for t in inputs]
        out, final = fn(*leaves, CPU_SAMPLE_SHAPE[5], dt_softplus=True, return_final_state=True)
        (out.pow(2).mean() + final.pow(2).mean()).backward()

    for _ in range(warmup):
        step()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return times, kind


def run_reference_arm(args) -> None:
    """--impl reference: the reference's CPU implementation of the path on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)  # torch.distributed.run pins OMP_NUM_THREADS to 1
    times, kind = time_cpu_reference(args.steps, args.warmup)
    total = sum(times)
    tflops = step_flops(CPU_SAMPLE_SHAPE) * len(times) / total / 1e12
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.gpus, args.scaling, args.mode),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": CPU_SAMPLE_TEXT, "host_cpus": os.cpu_count()},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def device_inputs(dev, shape, seed: int):
    """Seeded synthetic inputs with the configuration's distributions, drawn on the device."""
    b, l, h, p, n, _t, g = shape
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(b, l, h, p, device=dev, generator=gen)
    dt = torch.rand(b, l, h, device=dev, generator=gen)
    a = -torch.rand(h, device=dev, generator=gen)
    bm = torch.randn(b, l, g, n, device=dev, generator=gen)
    cm = torch.randn(b, l, g, n, device=dev, generator=gen)
    return [x, dt, a, bm, cm]


class Timer:
    """K steps between two CUDA events on the current stream, with a barrier and a synchronize on both sides."""

    def __init__(self, barrier):
        self.barrier = barrier

    def run(self, fn, steps: int) -> float:
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return e0.elapsed_time(e1)


def make_step(inputs, chunk, op, **kwargs):
    """(step function, its fixed upstream gradients): forward + backward with gradients for every input."""
    with torch.no_grad():
        out0, fin0 = op(*inputs, chunk, dt_softplus=True, return_final_state=True, **kwargs)
        dout = (2.0 / out0.numel()) * out0
        dfin = (2.0 / fin0.numel()) * fin0
        del out0, fin0

    def step():
        leaves = [t.detach().requires_grad_(True) for t in inputs]
        extra = {k: (v.detach().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in kwargs.items()}
        out, final = op(*leaves, chunk, dt_softplus=True, return_final_state=True, **extra)
        torch.autograd.backward([out, final], [dout, dfin])
        return leaves

    return step


def secondary_measurements(dev, timer, peaks) -> dict:
    """The other configurations, a few steps each, outside the headline's timed region (one GPU only)."""
    from ascend_kernel import SavedTensorStats, check_status, mamba2 as M, mamba2_ssd_fwd, set_save_policy
    from ascend_kernel.vmamba2 import VisionMamba2, VisionMamba2Config

    sec = {}
    # configuration 2: forward only, no final state.  Its 100 MB fit the L2, so four input sets are rotated.
    sets = [device_inputs(dev, CONFIG2, SEED + 10 + i) for i in range(4)]
    it = [0]

    def c2():
        s = sets[it[0] % 4]
        it[0] += 1
        mamba2_ssd_fwd(*s, CONFIG2[5], dt_softplus=True)

    with torch.no_grad():
        for _ in range(8):
            c2()
        ms = timer.run(c2, 40) / 40
    sec["config2_forward"] = {"shape": list(CONFIG2), "ms": ms,
                              "hbm_frac": forward_bytes(CONFIG2, False) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              "algorithmic_bytes": forward_bytes(CONFIG2, False),
                              "l2": "four input sets in rotation (400 MB)"}
    del sets

    inputs = device_inputs(dev, H256, SEED)
    b, l, h, p, n, chunk, g = H256
    # the reference benchmark's own `full` mode: D, z, dt_bias, dt_limit, initial_states, all with gradients
    gen = torch.Generator(device=dev).manual_seed(SEED + 20)
    full = dict(D=torch.randn(h, device=dev, generator=gen), z=torch.randn(b, l, h, p, device=dev, generator=gen),
                dt_bias=0.1 * torch.randn(h, device=dev, generator=gen), dt_limit=(1e-3, 1.0),
                initial_states=torch.randn(b, h, p, n, device=dev, generator=gen))
    step = make_step(inputs, chunk, mamba2_ssd_fwd, **full)
    for _ in range(3):
        step()
    sec["full_feature_h256"] = {"ms_per_step": timer.run(step, 5) / 5,
                                "features": "D, z, dt_bias, dt_limit (1e-3, 1), initial_states"}
    del full, step
    # save-vs-recompute policy
    previous = set_save_policy("recompute")
    try:
        step = make_step(inputs, chunk, mamba2_ssd_fwd)
        for _ in range(3):
            step()
        ms = timer.run(step, 5) / 5
        stats = SavedTensorStats()
        leaves = [t.detach().requires_grad_(True) for t in inputs]
        with stats.hooks():
            out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
        saved_recompute = stats.unique_bytes
        del out, final, leaves
    finally:
        set_save_policy(previous)
    stats = SavedTensorStats()
    leaves = [t.detach().requires_grad_(True) for t in inputs]
    with stats.hooks():
        out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
    sec["recompute_policy_h256"] = {"ms_per_step": ms, "saved_bytes": saved_recompute,
                                    "saved_bytes_default_policy": stats.unique_bytes}
    del out, final, leaves, inputs, step
    # shapes outside the native kernels (reduced to them by padding and column blocks in the Python layer), each
    # beside the native shape it is reduced to: what the reduction costs
    general = {}
    for name, shape, native in (
            ("dstate128_fwd_bwd", (4, 2048, 16, 64, 128, 128, 4), (4, 2048, 16, 64, 64, 128, 4)),
            ("headdim32_ragged_fwd_bwd", (4, 2000, 32, 32, 64, 64, 4), (4, 2048, 16, 64, 64, 64, 4))):
        row = {"shape": list(shape), "native_shape": list(native)}
        for key, shp in (("ms_per_step", shape), ("native_ms_per_step", native)):
            gi = device_inputs(dev, shp, SEED + 30)
            gstep = make_step(gi, shp[5], mamba2_ssd_fwd)
            for _ in range(3):
                gstep()
            row[key] = timer.run(gstep, 10) / 10
            del gi, gstep
        general[name] = row
    sec["general_shapes"] = general
    # configuration 4: Vision-Mamba2 tiny forward, 4 images per GPU
    torch.manual_seed(1234)
    net = VisionMamba2(VisionMamba2Config()).to(dev).eval()
    images = torch.randn(4, 3, 1024, 1024, device=dev)
    with torch.no_grad():
        for _ in range(3):
            net(images)
        M.stage_events = []
        ms = timer.run(lambda: net(images), 5) / 5
        events, M.stage_events = M.stage_events, None
    sec["config4_vmamba2_forward"] = {"images_per_s": 4 / (ms * 1e-3), "ms_per_step": ms,
                                      "ssd_ms_per_step": sum(a.elapsed_time(b_) for _n, a, b_ in events) / 5,
                                      "images_per_gpu": 4}
    check_status(dev)
    return sec


def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    from ascend_kernel import check_status, mamba2 as M, mamba2_ssd_fwd, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the SSD path has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    timer = Timer(barrier)
    full_shape = H256
    if args.heads is not None:
        full_shape = (H256[0], H256[1], args.heads, 64, 64, 64, args.heads // 4)
    if args.seqlen is not None:
        full_shape = (full_shape[0], args.seqlen) + full_shape[2:]
    reduced = args.heads is not None or args.seqlen is not None
    chunk = full_shape[5]
    sp = args.mode == "sp"

    def local_inputs(scaling: str):
        if sp:  # this rank's block of consecutive tokens of the one problem
            t = device_inputs(dev, full_shape, SEED)
            lr = full_shape[1] // world
            sl = slice(rank * lr, (rank + 1) * lr)
            return [t[0][:, sl].contiguous(), t[1][:, sl].contiguous(), t[2], t[3][:, sl].contiguous(),
                    t[4][:, sl].contiguous()]
        if scaling == "strong" and world > 1:  # this rank's head block of the one problem
            return list(parallel.shard_by_heads(*device_inputs(dev, full_shape, SEED), rank, world))
        return device_inputs(dev, full_shape, SEED + 1000 * rank)

    inputs = local_inputs(args.scaling)
    if sp:
        def op(x, dt, a, bm, cm, chunk_size, **kw):
            kw.pop("return_final_state", None)
            return parallel.mamba2_ssd_fwd_sequence_parallel(x, dt, a, bm, cm, chunk_size, exchange=args.sp_exchange,
                                                             **kw)
    else:
        op = mamba2_ssd_fwd
    step = make_step(inputs, chunk, op)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    check_status(dev)

    # ---- timed region: exactly K steps, CUDA events, per-stage events inside
    if rank == 0:
        sampler.mark()
    M.stage_events = []
    total_ms = timer.run(step, args.steps)
    events, M.stage_events = M.stage_events, None
    clocks = sampler.stop() if rank == 0 else None
    check_status(dev)
    stage_ms = {}
    for name, s0, s1 in events:
        stage_ms.setdefault(name, []).append(s0.elapsed_time(s1))
    stage_avg = {k: sum(v) / len(v) for k, v in stage_ms.items()}
    launches = len(events) + args.steps  # the finalisation stage launches two kernels

    # ---- end to end: pinned host inputs -> device -> forward + backward -> gradients to pinned host.
    # A three-stage pipeline over steps, as a host-side caller of the API would run it: the upload of
    # step i+1 (copy stream) and the download of step i-1 (second copy stream) overlap the compute of
    # step i; device input and gradient buffers are double buffered.  Every step uploads all five
    # inputs and downloads the loss and all five gradients.
    e2e_ms, e2e_steps, h2d, d2h = None, 0, 0, 0
    if not args.no_e2e:
        host_in = [t.cpu().pin_memory() for t in inputs]
        dev_in = [[torch.empty_like(t) for t in inputs] for _ in range(2)]
        dev_grads = [None, None]
        host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in inputs]
        host_loss = torch.empty((), dtype=torch.float32).pin_memory()
        h2d = sum(t.numel() * 4 for t in host_in)
        d2h = sum(t.numel() * 4 for t in host_out) + 4
        s_main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_down = [torch.cuda.Event() for _ in range(2)]

        def upload(i):
            buf = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[buf])  # the compute that last read this buffer has finished
                for d, src in zip(dev_in[buf], host_in):
                    d.copy_(src, non_blocking=True)
                ev_in[buf].record(s_in)

        def compute(i):
            buf = i & 1
            s_main.wait_event(ev_in[buf])
            s_main.wait_event(ev_down[buf])  # the gradients of step i-2 have left this buffer
            leaves = [d.detach().requires_grad_(True) for d in dev_in[buf]]
            out, final = op(*leaves, chunk, dt_softplus=True, return_final_state=True)
            loss = out.pow(2).mean() + final.pow(2).mean()
            loss.backward()
            dev_grads[buf] = ([leaf.grad for leaf in leaves], loss.detach())
            ev_done[buf].record(s_main)
            ev_free[buf].record(s_main)

        def download(i):
            buf = i & 1
            grads, loss = dev_grads[buf]
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[buf])
                for hbuf, gten in zip(host_out, grads):
                    hbuf.copy_(gten, non_blocking=True)
                host_loss.copy_(loss, non_blocking=True)
                ev_down[buf].record(s_out)

        def run_pipeline(n):
            for e in ev_free + ev_down:
                e.record(s_main)
            upload(0)
            for i in range(n):
                if i + 1 < n:
                    upload(i + 1)
                compute(i)
                download(i)
            s_main.wait_stream(s_out)
            s_main.wait_stream(s_in)

        e2e_steps = args.steps
        run_pipeline(2)
        e2e_ms = timer.run(lambda: run_pipeline(e2e_steps), 1)
        check_status(dev)
        del host_in, dev_in, dev_grads, host_out

    # ---- at N > 1 under strong scaling: the weak-scaling number as well (every rank the full shape)
    weak_ms = None
    if world > 1 and args.scaling == "strong" and not sp and not args.no_secondary:
        del inputs, step
        winputs = local_inputs("weak")
        wstep = make_step(winputs, chunk, op)
        for _ in range(3):
            wstep()
        weak_ms = timer.run(wstep, 5) / 5
        del winputs, wstep

    times = torch.tensor([total_ms, e2e_ms or 0.0, weak_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms_max, weak_ms_max = (float(v) for v in times.tolist())

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = total_ms / args.steps
        flops = step_flops(full_shape)
        scale = world if (args.scaling == "weak" and not sp) else 1  # weak: N problems; strong / sp: one problem
        value = scale * flops / (ms_per_step * 1e-3) / 1e12
        local_shape = (inputs if "inputs" in locals() else None)
        # the slowest kernel of this rank's step, on its own algorithmic bytes
        per_rank = list(full_shape)
        if sp:
            per_rank[1] //= world
        elif args.scaling == "strong":
            per_rank[2] //= world
            per_rank[6] //= world
        top = max(stage_avg, key=stage_avg.get)
        top_bytes = stage_bytes(per_rank)[top]
        achieved = top_bytes / (stage_avg[top] * 1e-3) / 1e9
        traffic = traffic_of(top) if (world == 1 and not reduced) else None
        line = {
            "metric": METRIC if not sp else METRIC + "_sequence_parallel", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if sp else args.scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "dtype_note": "fp32 tensors in HBM; tensor-core operands split into bf16 hi+lo (3 MMAs), fp32 accumulate",
            "config": bench_config(world, args.scaling, args.mode),
            "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                         "peak_source": peaks["source"], "algorithmic_bytes": top_bytes,
                         "kernel_ms": stage_avg[top]},
            "path": {"algorithmic_bytes": path_bytes(full_shape), "algorithmic_flops": flops,
                     "hbm_frac": scale * path_bytes(full_shape) / world / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "tensor_frac": value / world / peaks["bf16_tflops"]},
            "stages_ms": {k: round(v, 4) for k, v in stage_avg.items()},
            "gpu_launches": launches, "clocks": clocks,
        }
        if reduced:
            line["config"]["workload"] = ("reduced case for profiler captures: [B,L,H,P,N,chunk,G]=" +
                                          str(list(full_shape)) + " (the H256 geometry with fewer heads or tokens)")
        if sp:
            line["config"]["sp_exchange"] = args.sp_exchange
        if e2e_steps:
            e2e_value = scale * flops / (e2e_ms_max / e2e_steps * 1e-3) / 1e12
            line["e2e"] = {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": e2e_ms_max / e2e_steps, "steps": e2e_steps}
        if weak_ms is not None:
            line.setdefault("secondary", {})["weak_scaling"] = {
                "ms_per_step": weak_ms_max, "value": world * flops / (weak_ms_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                "note": "every rank runs the full 256-head shape"}
        if world == 1 and not sp and not reduced:
            if not args.no_secondary:
                del step
                inputs = None
                torch.cuda.empty_cache()
                line.setdefault("secondary", {}).update(secondary_measurements(dev, timer, peaks))
            if not args.no_cpu_baseline:
                torch.set_num_threads(os.cpu_count() or 1)
                t, kind = time_cpu_reference(repeats=3, warmup=1)
                cpu_tflops = step_flops(CPU_SAMPLE_SHAPE) / min(t) / 1e12
                line["cpu_baseline"] = {"value": cpu_tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                        "kind": kind, "sample": CPU_SAMPLE_TEXT + ", best of 3",
                                        "host_cpus": os.cpu_count()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_vmamba2(args) -> None:
    """--workload vmamba2: benchmark configuration 4, the Vision-Mamba2 tiny full-network forward (random
    init, fp32 images 3x1024x1024, 4 images per GPU = batch 32 over 8 GPUs).  Secondary to the headline."""
    import torch.distributed as dist

    from ascend_kernel import check_status, mamba2 as M
    from ascend_kernel.vmamba2 import VisionMamba2, VisionMamba2Config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234 + rank)
    net = VisionMamba2(VisionMamba2Config()).to(dev).eval()
    images = torch.randn(4, 3, 1024, 1024, device=dev)
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            net(images)
        M.stage_events = []
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            net(images)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    events, M.stage_events = M.stage_events, None
    check_status(dev)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms_step = float(ms.item()) / args.steps
        ssd_ms = sum(a.elapsed_time(b) for _n, a, b in events) / args.steps
        print(json.dumps({
            "metric": "vmamba2_tiny_forward_images_per_s", "value": world * 4 / (ms_step * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config4 Vision-Mamba2 tiny forward, 4 images of 3x1024x1024 per GPU, 12 blocks, "
                                   "SSD [4,4096,6,64,64,64,1] per block", "ssd_ms_per_step": ssd_ms},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong (default): the one H256 problem sharded over the ranks; weak: the full shape per rank")
    ap.add_argument("--mode", choices=["heads", "sp"], default="heads",
                    help="heads (default): group-aligned head blocks, no collective; sp: sequence parallel")
    ap.add_argument("--sp-exchange", choices=["chain", "allgather"], default="chain")
    ap.add_argument("--heads", type=int, default=None,
                    help="reduced head count (a multiple of 4) at the H256 geometry: the small case for profiler captures")
    ap.add_argument("--seqlen", type=int, default=None,
                    help="reduced sequence length (a multiple of 128): the small case that keeps all (batch, group) chains")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU timing on rank 0")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) measurement")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--workload", choices=["h256", "vmamba2"], default="h256",
                    help="h256 = the headline SSD forward + backward (default); vmamba2 = configuration 4")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "vmamba2" and args.impl == "ours":
        run_vmamba2(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
