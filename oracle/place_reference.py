"""Place the reference's own CPU implementation of the path beside the oracle.  TEST / BENCH INFRASTRUCTURE ONLY.

The reference computes this path on CPU with one pure-PyTorch file, ``mamba_torch/ssd_reference.py`` of
So-cean/mamba-ascendc.  Where the checkout is present (``SSD_REFERENCE_ROOT``, default ``/root/reference``)
this copies that file, byte for byte, to ``oracle/_ref/ssd_reference.py`` and records its sha256 next to it.
``oracle/_ref/`` is listed in .gitignore, so the file never enters the history; it travels with the working
tree to the machine the benchmark runs on, where ``bench.py --impl reference`` and the ``cpu_baseline`` leg
time its ``ssd_chunk_scan_ref`` (``kind: "reference"``).  Without the checkout and without a placed file the
benchmark falls back to the pinned port (``kind: "port"``).  Nothing else may import from ``oracle/_ref``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref" / "ssd_reference.py"


def place() -> bool:
    """Copy the file if the checkout is there; returns whether ``oracle/_ref/ssd_reference.py`` exists afterwards."""
    root = Path(os.environ.get("SSD_REFERENCE_ROOT", "/root/reference"))
    src = root / "mamba_torch" / "ssd_reference.py"
    if src.exists():
        TARGET.parent.mkdir(exist_ok=True)
        shutil.copyfile(src, TARGET)
        (TARGET.parent / "ssd_reference.sha256").write_text(hashlib.sha256(TARGET.read_bytes()).hexdigest() + "\n")
    return TARGET.exists()


if __name__ == "__main__":
    print("placed" if place() else "reference checkout not found; nothing placed")
