"""Tile-level parity of the tcgen05 path: one 128 x n x 128 product per operand-major combination.

Stands where the reference keeps its per-kernel component tests
(mamba_ascendc_ops/mamba2_ssd_chunk_mix/test); the checker is an fp64 matmul.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [64, 128])
@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("inplace", [0, 1, 2])  # 2: the A operand is kept in tensor memory (K-major only)
def test_umma_tile_matches_fp64(n, a_mn, b_mn, inplace):
    from ascend_kernel import _capi

    if inplace == 2 and a_mn:
        pytest.skip("an A operand in tensor memory is K-major")

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(1234 + n + 2 * a_mn + b_mn)
    a = torch.randn(128, 128, generator=g)  # [m, k]
    b = torch.randn(n, 128, generator=g)  # [n, k]
    ref = a.double() @ b.double().T
    a_dev = (a.T if a_mn else a).contiguous().to(dev)
    b_dev = (b.T if b_mn else b).contiguous().to(dev)
    d = torch.full((128, n), float("nan"), device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = _capi.lib.ssd_selftest_umma(a_dev.data_ptr(), b_dev.data_ptr(), d.data_ptr(), n, a_mn, b_mn, inplace,
                                     status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _capi.check(rc, "ssd_selftest_umma")
    torch.cuda.synchronize()
    assert status.item() == 0, f"bounded wait gave up, status {status.item()}"
    err = (d.double().cpu() - ref).abs().max().item()
    # split-bf16 keeps 16 mantissa bits per operand: |err| ~ 1e-5 * |a||b| * sqrt(k)
    assert err < 2e-3, f"max abs error {err}"
