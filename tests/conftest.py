import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def to_bf16_tensor(a, device):
    """numpy floats -> torch bf16 on device, rounded as an upload rounds them (nearest even)."""
    import torch
    from oracle import bfp
    bits = bfp.bf16_bits(np.asarray(a, np.float32))
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def bits_to_tensor(bits, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16).to(device)


def to_numpy(t):
    """torch tensor (bf16 included) -> numpy float64 / its own integer type."""
    import torch
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.float().numpy().astype(np.float64)
    if t.is_floating_point():
        return t.numpy().astype(np.float64)
    return t.numpy()
