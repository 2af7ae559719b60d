"""Benchmark of the Mamba-2 SSD forward + backward path at the H256 training shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward + backward of ``[B,L,H,P,N,chunk,G] = [8,4096,256,64,64,64,64]`` (fp32 public
tensors, dt_softplus, final state returned, gradients for x, dt, A, B, C) per GPU.  With N > 1 (launched by
``torch.distributed.run``) every rank processes its own block of 256 heads / 64 groups of a problem with
N x 256 heads: head blocks aligned to groups need no communication, so scaling is "weak" and no collective is
on the data path.  Rank 0 prints ONE JSON line.

``value`` is algorithmic TFLOP/s (6.7001e11 flop per step and GPU, dense tiles, forward x 3) with inputs
resident in HBM, timed with CUDA events over exactly K steps, max over ranks.  ``e2e`` repeats the step with
the inputs in pinned host memory and the gradients returned to pinned host memory inside the timed region.
The end-to-end steps run as an upload / compute / download pipeline.
``roofline`` describes the slowest kernel of the step, timed live with CUDA events on the launching stream.
``cpu_baseline`` / ``--impl reference`` time the CPU port of the reference algorithm (oracle/ssd_oracle.py,
fp32, all host threads) on a bounded sample of the same workload.  Inputs are synthetic (seeded).
"""
from __future__ import annotations

import argparse
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

SHAPE = (8, 4096, 256, 64, 64, 64, 64)  # benchmark configuration 3, per GPU
WORKLOAD = "config3 H256 fwd+bwd [B,L,H,P,N,chunk,G]=[8,4096,256,64,64,64,64] per GPU, dt_softplus, final state"
METRIC = "ssd_fwd_bwd_tflops_h256"
TILE = 128


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


def stage_bytes(shape) -> dict:
    """Algorithmic bytes of each kernel launch: its own inputs read once and outputs written once (fp32)."""
    b, l, h, p, n, _t, g = shape
    k = l // TILE
    x, dt, bc, st, fin = b * l * h * p, b * l * h, b * l * g * n, b * h * k * p * n, b * h * p * n
    words = {
        "mamba2_ssd_dt_cumsum": dt + h + 2 * dt,
        "mamba2_ssd_chunk_state": x + bc + 2 * dt + st,
        "mamba2_ssd_state_passing": 2 * st + fin + dt // TILE,
        "mamba2_ssd_chunk_scan": x + 2 * bc + st + 2 * dt + x,
        "mamba2_ssd_chunk_state_bwd": x + bc + 2 * dt + st,
        "mamba2_ssd_state_passing_bwd": 3 * st + fin + b * h * k,
        "mamba2_ssd_chunk_dx_bwd": 3 * x + 2 * bc + st + 3 * dt + x + dt,
        "mamba2_ssd_chunk_dbc_bwd": 2 * x + 2 * bc + 2 * st + 2 * dt + 2 * bc,
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
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

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


# --------------------------------------------------------------------------- CPU port of the reference
CPU_SAMPLE_SHAPE = (1, 4096, 32, 64, 64, 64, 8)  # 1/64 of the workload: one batch row, 8 of the 64 groups
CPU_SAMPLE_TEXT = "one forward+backward of a [1,4096,32,64,64,64,8] slice (1/64 of the workload: 1 batch row, 8 groups)"


def cpu_port_step(inputs, chunk) -> None:
    """One forward + backward of the reference algorithm's fp32 CPU path (oracle port)."""
    from oracle import ssd_oracle as O

    leaves = [t.detach().requires_grad_(True) for t in inputs]
    out, final = O.ssd_chunked(*leaves, chunk, dt_softplus=True, return_final_state=True)
    O.loss_fn(out, final).backward()


def time_cpu_port(repeats: int, warmup: int):
    from oracle import ssd_oracle as O

    inputs = O.make_inputs(CPU_SAMPLE_SHAPE, O.BASE_SEED + 3)
    for _ in range(warmup):
        cpu_port_step(inputs, CPU_SAMPLE_SHAPE[5])
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_port_step(inputs, CPU_SAMPLE_SHAPE[5])
        times.append(time.perf_counter() - t0)
    return times


def run_reference_arm(args) -> None:
    """--impl reference: the reference's CPU implementation of the path, on the host cores.

    The reference's own module cannot travel to the GPU box, so this is the pinned CPU port
    (oracle/ssd_oracle.py, ``compute_dtype=float32`` = the reference's public fp32 path)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)  # torch.distributed.run pins OMP_NUM_THREADS to 1
    times = time_cpu_port(args.steps, args.warmup)
    total = sum(times)
    tflops = step_flops(CPU_SAMPLE_SHAPE) * len(times) / total / 1e12
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": CPU_SAMPLE_TEXT},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": CPU_SAMPLE_TEXT, "host_cpus": os.cpu_count()},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def make_device_inputs(dev, rank: int):
    """Seeded synthetic inputs with the configuration's distributions, drawn on the device."""
    from oracle.ssd_oracle import BASE_SEED

    b, l, h, p, n, _t, g = SHAPE
    gen = torch.Generator(device=dev).manual_seed(BASE_SEED + 3 + 1000 * rank)
    x = torch.randn(b, l, h, p, device=dev, generator=gen)
    dt = torch.rand(b, l, h, device=dev, generator=gen)
    a = -torch.rand(h, device=dev, generator=gen)
    bm = torch.randn(b, l, g, n, device=dev, generator=gen)
    cm = torch.randn(b, l, g, n, device=dev, generator=gen)
    return [x, dt, a, bm, cm]


def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    from ascend_kernel import check_status, mamba2 as M, mamba2_ssd_fwd

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

    chunk = SHAPE[5]
    inputs = make_device_inputs(dev, rank)
    b, l, h, p, n, _t, g = SHAPE
    # fixed upstream gradients of the loss mean(out^2) + mean(final^2), taken from a first forward pass
    with torch.no_grad():
        out0, fin0 = mamba2_ssd_fwd(*inputs, chunk, dt_softplus=True, return_final_state=True)
        dout = (2.0 / out0.numel()) * out0
        dfin = (2.0 / fin0.numel()) * fin0
        del out0, fin0

    def step():
        leaves = [t.detach().requires_grad_(True) for t in inputs]
        out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
        torch.autograd.backward([out, final], [dout, dfin])
        return leaves

    for _ in range(args.warmup):
        step()
    check_status(dev)

    # ---- timed region: exactly K steps, CUDA events, per-stage events inside
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    M.stage_events = []
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
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
        out, final = mamba2_ssd_fwd(*leaves, chunk, dt_softplus=True, return_final_state=True)
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

    e2e_steps = max(2, min(args.steps, 6))
    run_pipeline(2)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    run_pipeline(e2e_steps)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    check_status(dev)

    times = torch.tensor([total_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = (float(v) for v in times.tolist())

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = total_ms / args.steps
        flops = step_flops(SHAPE)
        value = world * flops / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
        top = max(stage_avg, key=stage_avg.get)
        top_bytes = stage_bytes(SHAPE)[top]
        achieved = top_bytes / (stage_avg[top] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "dtype_note": "fp32 tensors in HBM; tensor-core operands split into bf16 hi+lo (3 MMAs), fp32 accumulate",
            "config": {"workload": WORKLOAD, "l2": "inputs (3.2 GB per GPU) are larger than the 126 MB L2",
                       "parallelism": f"{world} x head-block shard, no collective", "tile_tokens": TILE},
            "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": TRAFFIC.get(top),
                         "peak_source": peaks["source"], "algorithmic_bytes": top_bytes,
                         "kernel_ms": stage_avg[top]},
            "path": {"algorithmic_bytes": path_bytes(SHAPE), "algorithmic_flops": flops,
                     "hbm_frac": path_bytes(SHAPE) / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "tensor_frac": value / world / peaks["bf16_tflops"]},
            "stages_ms": {k: round(v, 4) for k, v in stage_avg.items()},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            t = time_cpu_port(repeats=3, warmup=1)
            cpu_tflops = step_flops(CPU_SAMPLE_SHAPE) / min(t) / 1e12
            line["cpu_baseline"] = {"value": cpu_tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": CPU_SAMPLE_TEXT + ", best of 3",
                                    "host_cpus": os.cpu_count()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes per launch from ncu (dram__bytes_read.sum + dram__bytes_write.sum), captured on the
# [8,4096,32,...] case of mamba-ascendc_b200/profile_case.py and scaled by 8 to the H256 launch (traffic is
# proportional to the head count); see profiles/ssd_tile_kernels_h32_sections.md.
TRAFFIC = {
    "mamba2_ssd_chunk_scan": 8 * (545.3e6 + 231.0e6),
    "mamba2_ssd_chunk_state_bwd": 8 * (344.0e6 + 107.0e6),
    "mamba2_ssd_chunk_state": 8 * (344.0e6 + 108.5e6),
    "mamba2_ssd_state_passing": 8 * (135.3e6 + 80.1e6),
    "mamba2_ssd_state_passing_bwd": 8 * (274.4e6 + 90.0e6),
    "mamba2_ssd_chunk_dx_bwd": 8 * (1089.0e6 + 263.5e6),
    "mamba2_ssd_chunk_dbc_bwd": 8 * (948.0e6 + 120.1e6),
}


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
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU port timing on rank 0")
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
