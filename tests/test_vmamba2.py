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
