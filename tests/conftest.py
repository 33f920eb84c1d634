"""Shared pytest configuration: the ``gpu`` marker and helpers that turn torch
tensors into the uint16 bit patterns the CPU oracle works on."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no device exists."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tensor_bits(t):
    """16-bit torch tensor (any device) -> numpy uint16 bit patterns."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def dtype_tag(t):
    import torch
    return "bf16" if t.dtype == torch.bfloat16 else "fp16"


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "ref_attn_cases.npz")
    return np.load(path)
