"""ctypes binding of libssd_b200.so, the C-ABI CUDA library.

The library is the only compute path: if the shared object is missing or
fails to load, importing this module raises.  There is no CPU fallback.
Signatures follow ``include/ssd_b200.h``.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIB_NAME = "libssd_b200.so"

SSD_OK = 0
SSD_FLAG_DT_SOFTPLUS = 1


class SsdShape(ctypes.Structure):
    """Mirror of ``struct SsdShape``."""

    _fields_ = [
        ("batch", ctypes.c_int32),
        ("seqlen", ctypes.c_int32),
        ("nheads", ctypes.c_int32),
        ("headdim", ctypes.c_int32),
        ("dstate", ctypes.c_int32),
        ("tile", ctypes.c_int32),
        ("ngroups", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("dt_min", ctypes.c_float),
        ("dt_max", ctypes.c_float),
        ("valid_len", ctypes.c_int32),
    ]


def library_path() -> Path:
    override = os.environ.get("SSD_B200_LIBRARY")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / LIB_NAME


def _load() -> ctypes.CDLL:
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} not found: build it with `python mamba-ascendc_b200/build.py` "
            "(ascend_kernel has no fallback path)"
        )
    return ctypes.CDLL(str(path))


lib = _load()

_p = ctypes.c_void_p
_shape_p = ctypes.POINTER(SsdShape)

# name -> (restype, argtypes); every symbol declared in include/ssd_b200.h
SIGNATURES = {
    "ssd_error_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ssd_check_shape": (ctypes.c_int, [_shape_p]),
    "ssd_buffer_bytes": (ctypes.c_size_t, [_shape_p, ctypes.c_int]),
    "ssd_selftest_wait_expiry": (ctypes.c_int, [_p, ctypes.c_int, _p]),
    "ssd_selftest_tile_walk": (ctypes.c_int, [_shape_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, _p]),
    "ssd_selftest_umma": (ctypes.c_int, [_p, _p, _p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _p, _p]),
    "ssd_dt_cumsum": (ctypes.c_int, [_shape_p, _p, _p, _p, _p, _p, _p]),
    "ssd_chunk_state": (ctypes.c_int, [_shape_p, _p, _p, _p, _p, _p, ctypes.c_int, _p, _p]),
    "ssd_state_passing_fwd": (ctypes.c_int, [_shape_p, _p, _p, _p, _p, _p]),
    "ssd_chunk_scan_fwd": (ctypes.c_int, [_shape_p] + [_p] * 9),
    "ssd_state_passing_bwd": (ctypes.c_int, [_shape_p] + [_p] * 7),
    "ssd_chunk_state_scan_supported": (ctypes.c_int, [_shape_p]),
    "ssd_chunk_state_scan": (ctypes.c_int, [_shape_p] + [_p] * 7 + [ctypes.c_int, _p, _p]),
    "ssd_state_fold": (ctypes.c_int, [_shape_p, _p, _p, _p, _p, ctypes.c_int, _p]),
    "ssd_chunk_dx_bwd": (ctypes.c_int, [_shape_p] + [_p] * 15 + [_p, ctypes.c_int, _p, _p]),
    "ssd_chunk_dbc_bwd": (ctypes.c_int, [_shape_p] + [_p] * 13),
    "ssd_dt_finalize_bwd": (ctypes.c_int, [_shape_p] + [_p] * 5),
    "ssd_gate_partial_floats": (ctypes.c_size_t, [_shape_p]),
    "ssd_gate_skip_fwd": (ctypes.c_int, [_shape_p, _p, _p, _p, ctypes.c_int, _p, _p, _p]),
    "ssd_gate_skip_bwd": (ctypes.c_int, [_shape_p, _p, _p, _p, _p, ctypes.c_int, _p, _p, _p, _p, _p, _p]),
    "ssd_block_rmsnorm_fwd": (ctypes.c_int, [_p, ctypes.c_longlong, _p, ctypes.c_longlong, _p, _p, ctypes.c_longlong,
                                            ctypes.c_int, ctypes.c_float, _p]),
    "ssd_block_conv_silu_fwd": (ctypes.c_int, [_p, ctypes.c_longlong, _p, _p, _p, _p, _p, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_int, _p]),
    "ssd_static_scratch_bytes": (ctypes.c_size_t, []),
    "ssd_forward_static": (ctypes.c_int, [_shape_p] + [_p] * 9),
}

# test-only entry points; a library built with ``build.py --product-only`` does not have them
TEST_HOOKS = {"ssd_selftest_umma", "ssd_selftest_wait_expiry", "ssd_selftest_tile_walk"}

for _name, (_res, _args) in SIGNATURES.items():
    if _name in TEST_HOOKS and not hasattr(lib, _name):
        continue
    _fn = getattr(lib, _name)  # AttributeError here means the header and the build disagree
    _fn.restype = _res
    _fn.argtypes = _args


def error_string(code: int) -> str:
    return lib.ssd_error_string(int(code)).decode()


def check(code: int, op: str) -> None:
    """Raise the reference's style of error (``RuntimeError("<op>: <message>")``) for a failed call."""
    if code != SSD_OK:
        raise RuntimeError(f"{op}: {error_string(code)} (code {code})")
