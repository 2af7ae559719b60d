"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, validates shapes like the reference's host checks, and the Python layer raises the
reference's error types."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _declared_functions():
    text = (ROOT / "include" / "ssd_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ssd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ascend_kernel import _capi

    names = _declared_functions()
    assert len(names) >= 11
    for name in names:
        assert hasattr(_capi.lib, name), f"{name} declared in include/ssd_b200.h but not exported"
        assert name in _capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_capi.SIGNATURES) == names


def _shape(b=1, l=128, h=2, p=64, n=64, t=128, g=1, flags=1):
    from ascend_kernel import _capi

    return _capi.SsdShape(b, l, h, p, n, t, g, flags, 0.0, float("inf"), 0)


@pytest.mark.parametrize("kwargs,code", [
    ({}, 0),
    ({"n": 128}, 0),
    ({"b": 0}, -2), ({"l": -1}, -2), ({"h": 3, "g": 2}, -2), ({"t": 0}, -2),   # SSD_ERR_SHAPE
    ({"p": 32}, -3), ({"n": 32}, -3), ({"l": 192}, -3), ({"t": 64}, -3),       # SSD_ERR_UNSUPPORTED
])
def test_check_shape_codes(kwargs, code):
    from ascend_kernel import _capi

    s = _shape(**kwargs)
    assert _capi.lib.ssd_check_shape(ctypes.byref(s)) == code
    assert _capi.error_string(code).startswith("ssd:")


def test_range_limits_have_their_own_code():
    """Sizes one launch cannot index: grid dimensions and the int32 coordinates of the tile loads."""
    from ascend_kernel import _capi

    for kwargs in ({"b": 65536}, {"g": 65536 * 2, "h": 65536 * 2}, {"b": 16384, "l": 131072}):
        assert _capi.lib.ssd_check_shape(ctypes.byref(_shape(**kwargs))) == -4, kwargs
    assert "out of range" in _capi.error_string(-4)
    assert _capi.lib.ssd_check_shape(ctypes.byref(_shape(b=65535))) == 0


def test_buffer_sizes_match_the_layouts_the_python_layer_allocates():
    from ascend_kernel import _capi

    s = _shape(b=2, l=384, h=6, g=3)
    b, l, h, p, n, k = 2, 384, 6, 64, 64, 3
    want = {0: 4 * b * h * l, 1: 4 * b * h * l, 2: 4 * b * h * k * p * n, 3: 4 * b * h * p * n, 4: 4 * b * h * k,
            5: 4 * b * h * l, 6: 8 * b * h * k, 7: 4 * _capi.lib.ssd_gate_partial_floats(ctypes.byref(s)), 8: 4}
    for which, nbytes in want.items():
        assert _capi.lib.ssd_buffer_bytes(ctypes.byref(s), which) == nbytes, which
    assert _capi.lib.ssd_buffer_bytes(ctypes.byref(s), 99) == 0
    assert _capi.lib.ssd_buffer_bytes(ctypes.byref(_shape(p=32)), 0) == 0
    assert _capi.lib.ssd_buffer_bytes(None, 0) == 0


def test_null_pointers_are_rejected_before_any_launch():
    from ascend_kernel import _capi

    s = _shape()
    assert _capi.lib.ssd_dt_cumsum(ctypes.byref(s), None, None, None, None, None, None) == -1
    assert _capi.lib.ssd_check_shape(None) == -1
    with pytest.raises(RuntimeError, match="ssd_dt_cumsum: ssd:"):
        _capi.check(-1, "ssd_dt_cumsum")


def test_python_layer_error_behaviour_matches_reference_style():
    """mamba2_ssd_fwd.cpp:15-112 raises RuntimeError("mamba2_ssd_fwd: ...") before launching."""
    from ascend_kernel import mamba2_ssd_fwd

    x = torch.zeros(1, 128, 2, 64)
    dt = torch.zeros(1, 128, 2)
    a = torch.zeros(2)
    b = torch.zeros(1, 128, 1, 64)
    with pytest.raises(RuntimeError, match="mamba2_ssd_fwd: x must be a CUDA tensor"):
        mamba2_ssd_fwd(x, dt, a, b, b, 64)


def test_validation_order_and_messages():
    from ascend_kernel import mamba2 as M

    class Fake(torch.Tensor):
        """CPU tensor that claims to be on CUDA so the shape checks can run without a device."""
        @property
        def is_cuda(self):
            return True

    def fake(*shape):
        return torch.zeros(*shape).as_subclass(Fake)

    x, dt, a, b = fake(1, 128, 2, 64), fake(1, 128, 2), fake(2), fake(1, 128, 1, 64)
    inf = float("inf")
    M._validate(x, dt, a, b, b, 64, None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="dt shape must equal"):
        M._validate(x, fake(1, 128, 3), a, b, b, 64, None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="B and C shapes must match"):
        M._validate(x, dt, a, b, fake(1, 128, 1, 32), 64, None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="divisible by ngroups"):
        M._validate(fake(1, 128, 3, 64), fake(1, 128, 3), fake(3), fake(1, 128, 2, 64), fake(1, 128, 2, 64), 64,
                    None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="chunk_size must be positive"):
        M._validate(x, dt, a, b, b, 0, None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        M._validate(fake(1, 128, 64, 2).transpose(2, 3), dt, a, b, b, 64, None, None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="must be float32"):
        M._validate(x.double().as_subclass(Fake), dt, a, b, b, 64, None, None, None, (0.0, inf), None)
    # optional inputs (mamba2_ssd_fwd.cpp:88-112): accepted with the right shapes, rejected otherwise
    M._validate(x, dt, a, b, b, 64, fake(2), fake(1, 128, 2, 64), fake(2), (1e-3, 1.0), fake(1, 2, 64, 64))
    M._validate(x, dt, a, b, b, 64, fake(2, 64), None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="D shape must equal"):
        M._validate(x, dt, a, b, b, 64, fake(3), None, None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="z shape must match x"):
        M._validate(x, dt, a, b, b, 64, None, fake(1, 128, 2, 32), None, (0.0, inf), None)
    with pytest.raises(RuntimeError, match="dt_bias shape must equal"):
        M._validate(x, dt, a, b, b, 64, None, None, fake(3), (0.0, inf), None)
    with pytest.raises(RuntimeError, match="initial_states shape must equal"):
        M._validate(x, dt, a, b, b, 64, None, None, None, (0.0, inf), fake(1, 2, 64, 32))
    with pytest.raises(RuntimeError, match="dt_limit min must not exceed max"):
        M._validate(x, dt, a, b, b, 64, None, None, None, (1.0, 0.5), None)


def test_persistent_tile_walk_matches_the_closed_form():
    """The persistent kernels find their (batch, group, tile, head) positions with an incremental, division-free
    walk (carries from token tile to group to batch).  The library's host-side hook runs that walk; here it is
    compared with the closed form for grids and shapes that exercise every carry."""
    import numpy as np

    from ascend_kernel import _capi

    rng = np.random.default_rng(5)
    cases = [(8, 4096, 256, 64, 148), (2, 1408, 14, 14, 148), (2, 4096, 48, 12, 148), (3, 384, 10, 5, 45),
             (1, 128, 7, 7, 7), (5, 640, 12, 3, 148), (2, 256, 6, 1, 4)]
    for _ in range(20):
        g = int(rng.integers(1, 9))
        r = int(rng.integers(1, 5))
        cases.append((int(rng.integers(1, 6)), 128 * int(rng.integers(1, 13)), g * r, g, int(rng.integers(1, 200))))
    for b, l, h, g, grid in cases:
        nchunks, hpg = l // 128, h // g
        tiles = b * g * nchunks
        grid = min(grid, tiles)
        shape = _capi.SsdShape(b, l, h, 64, 64, 128, g, 1, 0.0, float("inf"), 0)
        for cta in {0, grid // 2, grid - 1}:
            my_tiles = (tiles - cta + grid - 1) // grid
            count = my_tiles * hpg
            out = (ctypes.c_int * (4 * count))()
            rc = _capi.lib.ssd_selftest_tile_walk(ctypes.byref(shape), grid, cta, count, out)
            assert rc == 0
            got = np.array(out[:]).reshape(count, 4)
            for it in range(count):
                tile = cta + (it // hpg) * grid
                k, gi, bi = tile % nchunks, (tile // nchunks) % g, tile // (nchunks * g)
                head = gi * hpg + it % hpg
                want = (gi, head, bi * l + k * 128, (bi * h + head) * nchunks + k)
                assert tuple(got[it]) == want, (b, l, h, g, grid, cta, it, tuple(got[it]), want)
