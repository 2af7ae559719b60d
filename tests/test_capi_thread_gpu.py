"""The C ABI called from a thread that has made no CUDA call of its own.

The entry points that take TMA loads encode their tensor maps with a DRIVER function, and the driver wants a
context current on the calling thread.  The framework's backward pass runs on a thread of its own; on device 0
nothing switches the device there, and when every allocation of the step comes out of the caching allocator that
thread reaches the library without ever having touched the runtime -- the encode then failed with "invalid
context" (seen on rank 0 of a four-rank run; ranks on other devices switch devices first and were fine).  The
library now binds the primary context itself before it encodes a map it has not cached yet."""
import ctypes
import threading

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def test_tensor_maps_are_encoded_on_a_thread_without_a_current_context():
    from ascend_kernel import _capi, mamba2 as M

    dev = torch.device("cuda:0")
    shape = (2, 256, 4, 64, 64, 64, 2)
    b, l, h, p, n, _chunk, g = shape
    k = l // 128
    x, dt, a, bm, _cm = [t.to(dev) for t in O.make_inputs(shape, 77)]
    lib = _capi.lib
    shp = M.make_shape(x, bm, True)
    sp = ctypes.byref(shp)
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q = torch.empty(b, h, l, device=dev)
    cs = torch.empty(b, h, l, device=dev)
    _capi.check(lib.ssd_dt_cumsum(sp, dt.data_ptr(), None, a.data_ptr(), q.data_ptr(), cs.data_ptr(), st), "dt_cumsum")
    # reference result from this thread; then fresh buffers (addresses the map table has not seen), so that the
    # other thread has to encode
    want = torch.empty(b, h, k, p, n, device=dev)
    _capi.check(lib.ssd_chunk_state(sp, x.data_ptr(), bm.data_ptr(), q.data_ptr(), cs.data_ptr(), want.data_ptr(), 0,
                                    status.data_ptr(), st), "chunk_state")
    x2, bm2 = x.clone(), bm.clone()
    got = torch.empty(b, h, k, p, n, device=dev)
    torch.cuda.synchronize()
    args = (sp, x2.data_ptr(), bm2.data_ptr(), q.data_ptr(), cs.data_ptr(), got.data_ptr(), 0, status.data_ptr(), st)
    result = {}

    def worker():  # no torch call in here: the thread reaches the library with no context bound
        result["rc"] = lib.ssd_chunk_state(*args)

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert result["rc"] == 0, _capi.error_string(result["rc"])
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got, want)
