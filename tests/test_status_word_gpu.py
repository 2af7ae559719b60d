"""The give-up path of the kernels' bounded waits, driven without disturbing the GPU.

Every wait in the tile kernels (on a TMA load, on a tensor-core product, on the hand-off to the issuing warp)
polls a bounded number of times; when it runs out the kernel records a code in the per-device status word,
writes no results and returns normally, and kernels launched while the word is set return at once.  Here the
wait is made to run out on purpose in the mildest way there is: one warp polls a barrier that nothing will
ever complete, with no copy and no tensor-core instruction in flight (``ssd_selftest_wait_expiry``), for
about a millisecond.  Then: the code is there, a real kernel launched afterwards leaves its output alone,
``check_status`` raises once and clears the word, and the next forward pass is correct again.
"""
import ctypes

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def test_wait_expiry_sets_status_and_later_launches_do_nothing():
    from ascend_kernel import _capi, check_status, mamba2 as M, mamba2_ssd_fwd

    dev = torch.device("cuda:0")
    check_status(dev)  # clean before the test
    status = M._status(dev)
    stream = torch.cuda.current_stream().cuda_stream
    _capi.check(_capi.lib.ssd_selftest_wait_expiry(status.data_ptr(), 1024, stream), "ssd_selftest_wait_expiry")
    torch.cuda.synchronize()
    assert int(status.item()) & 15 == 1  # the kind of a load that did not arrive

    # a tile kernel launched while the word is set returns without touching its output
    shape = (1, 256, 4, 64, 64, 64, 2)
    x, dt, a, bm, cm = (t.to(dev) for t in O.make_inputs(shape, 5))
    q = torch.rand(1, 4, 256, device=dev)
    cs = -torch.rand(1, 4, 256, device=dev)
    states = torch.full((1, 4, 2, 64, 64), 7.5, device=dev)
    shp = M.make_shape(x, bm, True)
    _capi.check(_capi.lib.ssd_chunk_state(ctypes.byref(shp), x.data_ptr(), bm.data_ptr(), q.data_ptr(), cs.data_ptr(),
                                          states.data_ptr(), 0, status.data_ptr(), stream), "ssd_chunk_state")
    torch.cuda.synchronize()
    assert bool((states == 7.5).all())
    assert int(status.item()) & 15 == 1  # the first code is kept

    with pytest.raises(RuntimeError, match="device-side wait gave up"):
        check_status(dev)
    check_status(dev)  # raising cleared the word
    out, final = mamba2_ssd_fwd(x, dt, a, bm, cm, 64, dt_softplus=True, return_final_state=True)
    check_status(dev)
    o64, f64 = O.ssd_chunked(*(t.double().cpu() for t in (x, dt, a, bm, cm)), 64, dt_softplus=True,
                             return_final_state=True, compute_dtype=None)
    assert O.rel_l2(out.cpu(), o64) <= 2e-3 and O.max_abs(out.cpu(), o64) <= 1e-2
    assert O.rel_l2(final.cpu(), f64) <= 2e-3 and O.max_abs(final.cpu(), f64) <= 1e-2


def test_wait_expiry_rejects_long_waits():
    from ascend_kernel import _capi

    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    assert _capi.lib.ssd_selftest_wait_expiry(status.data_ptr(), 0, None) == -3
    assert _capi.lib.ssd_selftest_wait_expiry(status.data_ptr(), 1 << 20, None) == -3
    assert _capi.lib.ssd_selftest_wait_expiry(None, 16, None) == -1
