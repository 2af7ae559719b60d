"""Vision-Mamba2 forward network around the SSD operator (benchmark configuration 4's architecture)."""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

from oracle import ssd_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def _load_module():
    # the module file alone: importing the package would load the CUDA library, which CPU tests do not need
    spec = importlib.util.spec_from_file_location("ssd_vmamba2", ROOT / "mamba-ascendc_b200/ascend_kernel/vmamba2.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ssd_vmamba2"] = mod
    spec.loader.exec_module(mod)
    return mod


def _oracle_ssd(x, dt, A, B, C, chunk_size, **kw):
    return O.ssd_chunked(x, dt, A, B, C, chunk_size, **kw)


def test_network_shapes_and_config_on_cpu():
    vm = _load_module()
    cfg = vm.VisionMamba2Config()
    assert (cfg.tokens, cfg.d_inner, cfg.nheads, cfg.d_state, cfg.ngroups, cfg.chunk_size) == (4096, 384, 6, 64, 1, 64)
    small = vm.VisionMamba2Config(image_size=64, depth=2, num_classes=10)
    torch.manual_seed(0)
    net = vm.VisionMamba2(small, ssd_fn=_oracle_ssd)
    logits = net(torch.randn(2, 3, 64, 64))
    assert logits.shape == (2, 10) and torch.isfinite(logits).all()


@pytest.mark.gpu
def test_network_with_cuda_ssd_matches_network_with_oracle_ssd():
    vm = _load_module()
    from ascend_kernel import check_status, mamba2_ssd_fwd

    cfg = vm.VisionMamba2Config(image_size=320, depth=3, num_classes=16)  # 400 tokens: ragged vs the 128 tile
    torch.manual_seed(1)
    dev = torch.device("cuda:0")
    net = vm.VisionMamba2(cfg, ssd_fn=mamba2_ssd_fwd).to(dev)
    ref = vm.VisionMamba2(cfg, ssd_fn=_oracle_ssd).to(dev)
    ref.load_state_dict(net.state_dict())
    img = torch.randn(2, 3, 320, 320, device=dev)
    with torch.no_grad():
        got, want = net(img), ref(img)
    check_status()
    rel = ((got - want).norm() / want.norm()).item()
    assert rel < 1e-4, rel


@pytest.mark.gpu
def test_fused_block_kernels_match_the_framework_operations():
    """The inference path of the packaged network (fused RMSNorm / conv1d + SiLU / gated RMSNorm kernels) against
    the same network run with gradients enabled (framework operations), and the two kernels on their own against
    torch, including a ragged token count and inputs that are column slices of a wider matrix."""
    import torch.nn.functional as F

    from ascend_kernel import _capi, check_status
    from ascend_kernel.vmamba2 import VisionMamba2, VisionMamba2Config

    dev = torch.device("cuda:0")
    cfg = VisionMamba2Config(image_size=320, depth=3, num_classes=16)  # 400 tokens: ragged vs the 128 tile
    torch.manual_seed(2)
    net = VisionMamba2(cfg).to(dev)
    img = torch.randn(2, 3, 320, 320, device=dev)
    with torch.no_grad():
        fused = net(img)
    with torch.enable_grad():
        plain = net(img).detach()
    check_status()
    assert ((fused - plain).norm() / plain.norm()).item() < 1e-5

    st = torch.cuda.current_stream().cuda_stream
    rows, width, d_in, gn = 2 * 77, 902, 384, 64
    wide = torch.randn(rows, width, device=dev)
    w = torch.randn(d_in, device=dev)
    y = torch.randn(rows, d_in, device=dev)
    out = torch.empty(rows, d_in, device=dev)
    _capi.check(_capi.lib.ssd_block_rmsnorm_fwd(y.data_ptr(), d_in, wide.data_ptr(), width, w.data_ptr(), out.data_ptr(),
                                                rows, d_in, 1e-5, st), "rmsnorm")
    t = y * F.silu(wide[:, :d_in])
    want = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(out, want, rtol=1e-5, atol=1e-5)
    conv = torch.nn.Conv1d(d_in + 2 * gn, d_in + 2 * gn, 4, groups=d_in + 2 * gn, padding=3).to(dev)
    xo, bo, co = (torch.empty(2, 77, n_, device=dev) for n_ in (d_in, gn, gn))
    _capi.check(_capi.lib.ssd_block_conv_silu_fwd(wide.data_ptr() + 4 * d_in, width, conv.weight.data_ptr(),
                                                  conv.bias.data_ptr(), xo.data_ptr(), bo.data_ptr(), co.data_ptr(),
                                                  2, 77, d_in, gn, st), "conv")
    src = wide[:, d_in:d_in + d_in + 2 * gn].reshape(2, 77, -1)
    with torch.no_grad():
        ref = F.silu(conv(src.transpose(1, 2))[..., :77].transpose(1, 2))
    got = torch.cat([xo, bo, co], dim=-1)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-5)
    # shape errors come back as codes, nothing is launched
    assert _capi.lib.ssd_block_rmsnorm_fwd(y.data_ptr(), 8, None, 0, w.data_ptr(), out.data_ptr(), rows, d_in, 1e-5, st) == -2
    assert _capi.lib.ssd_block_rmsnorm_fwd(y.data_ptr(), 1024, None, 0, w.data_ptr(), out.data_ptr(), rows, 1024, 1e-5, st) == -3
