"""Out-of-bounds guard for every output and scratch buffer of the C ABI: each buffer sits between sentinel
pads; after the full forward + backward stage sequence the pads must be untouched (the CUDA kernels write
through TMA stores and plain stores; compute-sanitizer is not available on the GPU pool).  The reference
runs its kernels under mssanitizer memcheck for the same purpose (mamba2_ssd_mssanitizer_test.py:70-78)."""
import ctypes

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

PAD = 4096  # floats on each side (keeps 16-byte alignment of the payload)
SENTINEL = 12345.678


class Padded:
    def __init__(self, shape, dev, dtype=torch.float32):
        n = 1
        for d in shape:
            n *= d
        self.raw = torch.full((n + 2 * PAD,), SENTINEL, device=dev, dtype=dtype)
        self.view = self.raw[PAD:PAD + n].view(shape)

    def intact(self):
        return bool((self.raw[:PAD] == SENTINEL).all()) and bool((self.raw[-PAD:] == SENTINEL).all())


@pytest.mark.parametrize("shape", [(2, 384, 6, 64, 64, 64, 2), (1, 640, 4, 64, 64, 64, 4)])
def test_no_stage_writes_outside_its_buffers(shape):
    from ascend_kernel import _capi, mamba2 as M

    dev = torch.device("cuda:0")
    b, l, h, p, n, _chunk, g = shape
    k = l // 128
    x, dt, a, bm, cm = [t.to(dev) for t in O.make_inputs(shape, 91)]
    dout = torch.randn(b, l, h, p, device=dev)
    dfinal = torch.randn(b, h, p, n, device=dev)
    bufs = {name: Padded(shp, dev, dty) for name, shp, dty in [
        ("q", (b, h, l), torch.float32), ("cs", (b, h, l), torch.float32),
        ("states", (b, h, k, p, n), torch.float32), ("final", (b, h, p, n), torch.float32),
        ("out", (b, l, h, p), torch.float32), ("dstates", (b, h, k, p, n), torch.float32),
        ("g_last", (b, h, k), torch.float32), ("d_initial", (b, h, p, n), torch.float32),
        ("fold", (b, h, p, n), torch.float32),
        ("dx", (b, l, h, p), torch.float32), ("ddt_t", (b, h, l), torch.float32),
        ("dA_part", (b, h, k), torch.float64), ("dB", (b, l, g, n), torch.float32),
        ("dC", (b, l, g, n), torch.float32), ("ddt", (b, l, h), torch.float32), ("dA", (h,), torch.float32)]}
    v = {name: pb.view for name, pb in bufs.items()}
    lib = _capi.lib
    shp = M.make_shape(x, bm, True)
    sp = ctypes.byref(shp)
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    calls = [
        ("dt_cumsum", lambda: lib.ssd_dt_cumsum(sp, P(dt), None, P(a), P(v["q"]), P(v["cs"]), st)),
        ("chunk_state", lambda: lib.ssd_chunk_state(sp, P(x), P(bm), P(v["q"]), P(v["cs"]), P(v["states"]), 0, P(status), st)),
        ("state_passing_fwd", lambda: lib.ssd_state_passing_fwd(sp, P(v["states"]), P(v["cs"]), None, P(v["final"]), st)),
        ("chunk_scan_fwd", lambda: lib.ssd_chunk_scan_fwd(sp, P(x), P(bm), P(cm), P(v["states"]), P(v["q"]), P(v["cs"]),
                                                         P(v["out"]), P(status), st)),
        ("chunk_state_bwd", lambda: lib.ssd_chunk_state(sp, P(dout), P(cm), P(v["q"]), P(v["cs"]), P(v["dstates"]), 1, P(status), st)),
        ("state_passing_bwd", lambda: lib.ssd_state_passing_bwd(sp, P(v["dstates"]), P(v["states"]), P(v["cs"]), P(dfinal),
                                                               P(v["g_last"]), P(v["d_initial"]), st)),
        ("chunk_dx_bwd", lambda: lib.ssd_chunk_dx_bwd(sp, P(x), P(bm), P(cm), P(dout), P(v["out"]), P(v["dstates"]), P(v["q"]),
                                                     P(v["cs"]), P(dt), None, P(a), P(v["g_last"]), P(v["dx"]), P(v["ddt_t"]),
                                                     P(v["dA_part"]), None, 0, P(status), st)),
        ("chunk_dbc_bwd", lambda: lib.ssd_chunk_dbc_bwd(sp, P(x), P(bm), P(cm), P(dout), P(v["states"]), P(v["dstates"]),
                                                       P(v["q"]), P(v["cs"]), P(v["dB"]), P(v["dC"]), P(v["g_last"]),
                                                       P(status), st)),
        ("dt_finalize_bwd", lambda: lib.ssd_dt_finalize_bwd(sp, P(v["ddt_t"]), P(v["dA_part"]), P(v["ddt"]), P(v["dA"]), st)),
        # the fused state stages and the read-only fold write the same buffers again
        ("chunk_state_scan", lambda: lib.ssd_chunk_state_scan(sp, P(x), P(bm), P(v["q"]), P(v["cs"]), None, P(v["states"]),
                                                             P(v["final"]), 0, P(status), st)),
        ("chunk_state_scan_bwd", lambda: lib.ssd_chunk_state_scan(sp, P(dout), P(cm), P(v["q"]), P(v["cs"]), P(dfinal),
                                                                 P(v["dstates"]), P(v["d_initial"]), 1, P(status), st)),
        ("state_fold", lambda: lib.ssd_state_fold(sp, P(v["dstates"]), P(v["cs"]), None, P(v["fold"]), 0, st)),
    ]
    for name, call in calls:
        _capi.check(call(), name)
        torch.cuda.synchronize()
        assert status.item() == 0, name
        broken = [bn for bn, pb in bufs.items() if not pb.intact()]
        assert not broken, f"{name} wrote outside {broken}"
    # every payload was written in full (no sentinel left) and is finite
    for name, pb in bufs.items():
        assert torch.isfinite(pb.view).all(), name
        assert not bool((pb.view == SENTINEL).any()), name
    # and the results are the real ones
    want = O.fp64_forward_backward(x.cpu(), dt.cpu(), a.cpu(), bm.cpu(), cm.cpu(), 64, dt_softplus=True,
                                   dout=dout.cpu(), dfinal=dfinal.cpu())
    got = [v["out"], v["final"], v["dx"], v["ddt"], v["dA"], v["dB"], v["dC"]]
    for gt, w, name in zip(got, want, ["out", "final", "dx", "ddt", "dA", "dB", "dC"]):
        assert O.rel_l2(gt.cpu(), w) <= 2e-3, name
