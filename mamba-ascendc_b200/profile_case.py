"""Small forward + backward case for profiler captures.

    python mamba-ascendc_b200/profile_case.py [--heads H] [--batch B] [--seqlen L] [--steps S]

Runs S steps of the SSD path on cuda:0 at the H256 per-head geometry (P = N = 64, 4 heads per group) with a
reduced head count, so that a profiler replaying a kernel many times finishes in minutes: the default
(B=8, L=4096, H=32) holds about 1.5 GB on the device, which is larger than L2.  Per-kernel traffic scales
linearly with the head count (every CTA handles one (batch, group, tile) and reads only its own data).
"""
import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from ascend_kernel import check_status, mamba2_ssd_fwd  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    b, l, h, p, n = args.batch, args.seqlen, args.heads, 64, 64
    g = h // 4
    gen = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(b, l, h, p, device=dev, generator=gen)
    dt = torch.rand(b, l, h, device=dev, generator=gen)
    a = -torch.rand(h, device=dev, generator=gen)
    bm = torch.randn(b, l, g, n, device=dev, generator=gen)
    cm = torch.randn(b, l, g, n, device=dev, generator=gen)
    dout = torch.randn_like(x) * 1e-6
    dfin = torch.randn(b, h, p, n, device=dev) * 1e-6
    for _ in range(args.steps):
        leaves = [t.detach().requires_grad_(True) for t in (x, dt, a, bm, cm)]
        out, final = mamba2_ssd_fwd(*leaves, 64, dt_softplus=True, return_final_state=True)
        torch.autograd.backward([out, final], [dout, dfin])
    check_status(dev)
    print("ok", b, l, h)


if __name__ == "__main__":
    main()
