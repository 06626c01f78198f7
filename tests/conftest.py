"""Shared fixtures.  Tests marked `gpu` need a B200 and call the CUDA path through the
C ABI; everything else runs on CPU (oracle vs golden vectors, host logic, ABI exports)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
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


@pytest.fixture(scope="session")
def port():
    from oracle import binding
    return binding.Port()


@pytest.fixture(scope="session")
def ref():
    from oracle import binding
    if not binding.Ref.available():
        pytest.skip("oracle/_ref/libsfref.so not built (needs the reference sources)")
    return binding.Ref()


@pytest.fixture(scope="session")
def sfb():
    from schedforge_b200 import lib
    lib.load()
    return lib


@pytest.fixture(scope="session")
def dev():
    """Helpers that move numpy arrays to the device as torch tensors (device memory only)."""
    import torch

    class Dev:
        @staticmethod
        def f32(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()

        @staticmethod
        def bf16(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(torch.bfloat16)

        @staticmethod
        def i32(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()

        @staticmethod
        def empty(shape, dtype):
            return torch.empty(shape, dtype=dtype, device="cuda")

        @staticmethod
        def zeros(shape, dtype):
            return torch.zeros(shape, dtype=dtype, device="cuda")

        @staticmethod
        def np(t):
            torch.cuda.synchronize()
            return t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()

        @staticmethod
        def stream():
            return torch.cuda.current_stream().cuda_stream

    Dev.torch = torch
    return Dev


def rel_err(got, want):
    """max|got - want| / max|want|  (the 'max-abs relative' error of the parity bar)."""
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))
