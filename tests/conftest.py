import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # the library and the oracle are built artefacts (kept out of git): build them when a fresh
    # checkout runs the tests before anything else did (nvcc cross-compiles without a GPU)
    lib = os.path.join(ROOT, "deep_diamond_b200", "libdd_b200.so")
    if not os.path.exists(lib):
        import importlib.util
        spec = importlib.util.spec_from_file_location("dd_b200_build", os.path.join(ROOT, "deep_diamond_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build(verbose=False)


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle
    _oracle.build()
    return _oracle


@pytest.fixture(scope="session")
def fact():
    """One B200 factory (handle + stream) for the whole GPU session."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from deep_diamond_b200 import b200_factory
    f = b200_factory()
    yield f
    f.release()


class Dev:
    """Moves numpy storage to the device and back as raw bytes (plumbing for the parity tests)."""

    def __init__(self, fact):
        import torch
        self.torch = torch
        self.fact = fact

    def put(self, arr):
        t = self.torch.from_numpy(np.ascontiguousarray(arr).reshape(-1).view(np.uint8).copy())
        return t.to(self.fact.device)

    def empty(self, nbytes, fill=0xCD):
        return self.torch.full((max(int(nbytes), 1),), fill, dtype=self.torch.uint8, device=self.fact.device)

    def get(self, t, np_dtype):
        self.fact.synchronize()
        self.torch.cuda.synchronize()
        return t.cpu().numpy().view(np_dtype).copy()


@pytest.fixture(scope="session")
def dev(fact):
    return Dev(fact)


def ulp_diff_f32(a, b):
    """Distance in units of float32 last place (the oracle package's helper, re-exported for the tests)."""
    import oracle as _oracle
    return _oracle.ulp_diff_f32(a, b)
