import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    def _load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))

    return _load


@pytest.fixture(scope="session")
def oracle():
    from oracle import mx_oracle

    mx_oracle.build()
    return mx_oracle


@pytest.fixture(scope="session")
def capi():
    """The C ABI through ctypes; builds the library when the sources are newer."""
    from catccos_b200 import build, capi as _capi

    build.build()
    _capi.load()
    return _capi


@pytest.fixture(scope="session")
def cuda(capi):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch


def to_dev_bf16(torch, bits: np.ndarray):
    """uint16 bf16 bit patterns -> CUDA bfloat16 tensor."""
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def to_np_f32(torch_tensor):
    return torch_tensor.float().cpu().numpy()
