"""The allocation-free forward entry point, ``ssd_forward_static``.

It exists for callers that cannot allocate device memory when they call the operator (a process whose
memory plan is fixed at start-up, a plug-in without a caching allocator): its temporaries live in a fixed
array inside the library.  The test calls it through the C ABI twice in a row on different inputs -- the
second call finds the first call's contents in the shared array -- and compares each result with the
staged entry points, which use caller-allocated temporaries.  Both paths launch the same kernels, so the
results are expected to be identical; the assertion uses the suite's tolerance.  This file sorts last so
that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

REL_L2_TOL = 2e-3
MAX_ABS_TOL = 1e-2


def test_static_scratch_forward_matches_staged_forward_twice():
    from ascend_kernel import _capi, check_status, mamba2 as M

    dev = torch.device("cuda:0")
    lib = _capi.lib
    limit = lib.ssd_static_scratch_bytes()
    assert limit == 64 << 20
    for call, (shape, seed) in enumerate((((2, 384, 4, 64, 64, 64, 2), 51), ((1, 256, 6, 64, 128, 128, 2), 52))):
        x, dt, a, bm, cm = (t.to(dev) for t in O.make_inputs(shape, seed))
        want_out, want_final, *_ = M.forward_stages(x, dt, a, bm, cm, True, want_final=True)
        b, l, h, p, n, _c, g = shape
        out = torch.full_like(x, float("nan"))
        final = torch.full((b, h, p, n), float("nan"), device=dev)
        status = M._status(dev)
        shp = M.make_shape(x, bm, True)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = lib.ssd_forward_static(ctypes.byref(shp), x.data_ptr(), dt.data_ptr(), a.data_ptr(), bm.data_ptr(),
                                    cm.data_ptr(), out.data_ptr(), final.data_ptr(), status.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
        _capi.check(rc, "ssd_forward_static")
        check_status(dev)
        if call > 0:
            # the point of the entry point: device memory in use does not move across a call (the first call
            # on a device may still see the driver finish loading the library's device image)
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        for got, want, name in ((out, want_out, "out"), (final, want_final, "final_state")):
            r, m = O.rel_l2(got.cpu(), want.cpu()), O.max_abs(got.cpu(), want.cpu())
            assert r <= REL_L2_TOL and m <= MAX_ABS_TOL, f"{name}: rel-L2 {r:.3e}, max-abs {m:.3e}"
        # and against the fp64 oracle, like every other parity test
        o64, f64 = O.ssd_chunked(*(t.double().cpu() for t in (x, dt, a, bm, cm)), shape[5], dt_softplus=True,
                                 return_final_state=True, compute_dtype=None)
        assert O.rel_l2(out.cpu(), o64) <= REL_L2_TOL and O.max_abs(out.cpu(), o64) <= MAX_ABS_TOL
        assert O.rel_l2(final.cpu(), f64) <= REL_L2_TOL and O.max_abs(final.cpu(), f64) <= MAX_ABS_TOL


def test_static_scratch_forward_rejects_oversized_problem():
    from ascend_kernel import _capi

    # 4*B*H*L*(2 + P*N/128) bytes: [8,4096,256,64,64] needs 4.4 GiB, far beyond the built-in 64 MiB
    shp = _capi.SsdShape(8, 4096, 256, 64, 64, 128, 64, 1, 0.0, float("inf"), 0)
    one = torch.zeros(4, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    rc = _capi.lib.ssd_forward_static(ctypes.byref(shp), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                      one.data_ptr(), one.data_ptr(), one.data_ptr(), None, status.data_ptr(), None)
    assert rc == -8
    assert "64 MiB" in _capi.error_string(rc)
    with pytest.raises(RuntimeError, match="ssd_forward_static"):
        _capi.check(rc, "ssd_forward_static")


def test_static_scratch_forward_checks_alignment_before_launching_anything():
    from ascend_kernel import _capi, mamba2 as M

    dev = torch.device("cuda:0")
    shape = (1, 128, 2, 64, 64, 64, 1)
    x, dt, a, bm, cm = (t.to(dev) for t in O.make_inputs(shape, 53))
    raw = torch.full((x.numel() + 4,), 3.25, device=dev)
    out_unaligned = raw[1:1 + x.numel()]  # 4 bytes past a 16-byte boundary
    status = M._status(dev)
    shp = M.make_shape(x, bm, True)
    rc = _capi.lib.ssd_forward_static(ctypes.byref(shp), x.data_ptr(), dt.data_ptr(), a.data_ptr(), bm.data_ptr(),
                                      cm.data_ptr(), out_unaligned.data_ptr(), None, status.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    torch.cuda.synchronize()
    assert bool((raw == 3.25).all())
