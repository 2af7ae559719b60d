"""B200 drop-in for the ``ascend_kernel`` package of So-cean/mamba-ascendc (Mamba-2 SSD path only).

Importing the package loads libssd_b200.so through ctypes (``_capi``); it raises if the library
has not been built.  Public names follow ascend_kernel/__init__.py:19-28 of the reference.
"""
from . import _capi  # noqa: F401  (loads the shared library, fails loudly if absent)
from .mamba2 import (SavedTensorStats, check_status, mamba2_ssd_fwd, mamba_chunk_scan_combined,
                     set_save_policy, set_state_scan)

__all__ = ["mamba2_ssd_fwd", "mamba_chunk_scan_combined", "check_status", "set_save_policy", "set_state_scan",
           "SavedTensorStats"]
