"""Generate the golden fixtures in this directory from the reference implementation.

Run where the So-cean/mamba-ascendc checkout is importable:

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

For every case it draws seeded inputs (recipe of oracle/ssd_oracle.make_inputs),
runs the reference's ``mamba_torch/ssd_reference.py`` functions and stores inputs'
seed/shape together with the reference's outputs:

* ``seq64``  : ``ssd_sequential_ref`` in fp64 — out, final state and fp64 autograd
               gradients of mean(out^2) + mean(final^2);
* ``chunk32``: ``ssd_chunk_scan_ref`` (fp32 inside) — out and final state;
* ``segsum`` : ``segsum`` on a fixed vector (the known-answer test of
               tests/mamba2/test_reference.py:13-23).

The files are small (.npz, fp64/fp32 arrays of the two CPU-sized benchmark
configurations and three ragged/grouped shapes).
"""
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from mamba_torch.ssd_reference import segsum, ssd_chunk_scan_ref, ssd_sequential_ref  # noqa: E402

from oracle.ssd_oracle import BASE_SEED, CONFIG_SHAPES, make_inputs  # noqa: E402

# name -> ([B,L,H,P,N,chunk,G], seed, optional-feature switches)
CASES = {
    "config0": (CONFIG_SHAPES[0], BASE_SEED + 0, {}),
    "config1": (CONFIG_SHAPES[1], BASE_SEED + 1, {}),
    "two_tiles_grouped": ((1, 256, 4, 64, 64, 64, 2), 11, {}),
    "ragged_len": ((1, 100, 2, 16, 8, 32, 1), 12, {}),  # L not a multiple of the chunk
    "optional_inputs": ((2, 64, 4, 8, 16, 16, 2), 13, {"optional": True}),
}


def optional_tensors(shape, seed):
    b, l, h, p, n, _c, _g = shape
    gen = torch.Generator().manual_seed(seed + 1000)
    return dict(
        D=torch.randn(h, generator=gen),
        z=torch.randn(b, l, h, p, generator=gen),
        dt_bias=0.1 * torch.randn(h, generator=gen),
        initial_states=torch.randn(b, h, p, n, generator=gen),
    )


def main():
    for name, (shape, seed, opts) in CASES.items():
        x, dt, a, bm, cm = make_inputs(shape, seed)
        chunk = shape[5]
        extra = optional_tensors(shape, seed) if opts.get("optional") else {}
        limit = (1e-3, 1.0) if opts.get("optional") else (0.0, float("inf"))

        leaves = [t.double().requires_grad_(True) for t in (x, dt, a, bm, cm)]
        extra64 = {k: v.double() for k, v in extra.items()}
        out, final = ssd_sequential_ref(*leaves, dt_softplus=True, dt_limit=limit, return_final_state=True,
                                        **extra64)
        loss = out.pow(2).mean() + final.pow(2).mean()
        grads = torch.autograd.grad(loss, leaves)
        out32, final32 = ssd_chunk_scan_ref(x, dt, a, bm, cm, chunk, dt_softplus=True, dt_limit=limit,
                                            return_final_state=True, **extra)
        np.savez_compressed(
            HERE / f"{name}.npz",
            shape=np.array(shape), seed=np.array(seed), optional=np.array(bool(opts.get("optional"))),
            seq64_out=out.detach().numpy(), seq64_final=final.detach().numpy(),
            seq64_dx=grads[0].numpy(), seq64_ddt=grads[1].numpy(), seq64_dA=grads[2].numpy(),
            seq64_dB=grads[3].numpy(), seq64_dC=grads[4].numpy(),
            chunk32_out=out32.numpy(), chunk32_final=final32.numpy(),
        )
        print(name, shape, "loss", loss.item())
    v = torch.tensor([1.0, 2.0, 3.0, -0.5])
    np.savez_compressed(HERE / "segsum.npz", x=v.numpy(), segsum=segsum(v).numpy())


if __name__ == "__main__":
    main()
