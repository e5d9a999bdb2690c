"""Shared fixtures.  GPU tests are marked ``gpu`` and call the CUDA path through the C ABI;
everything else runs on a CPU-only machine (oracle vs golden vectors, host logic, ABI symbols)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    # Build what is missing or older than its sources (nvcc and gcc work without a GPU): build() returns at once
    # when the library is newer than every file it is made from, so an edited kernel is never tested through a
    # stale binary.
    entry._load_build_module().build()
    entry.load_oracle().build()
    entry.build_cpp_tests()


@pytest.fixture(scope="session")
def ts():
    return entry.load_package()


@pytest.fixture(scope="session")
def ora():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def gpu(ts):
    """The package with device 0 initialised; fails loudly when there is no usable GPU."""
    assert ts.cuda_is_available(), "no CUDA device visible: GPU tests cannot fall back to anything"
    ts.set_default_device(0)
    yield ts
    ts.set_matmul_precision(ts.FP32)


@pytest.fixture(autouse=True)
def _fresh_tape(request):
    yield
    if "gpu" in request.keywords:
        mod = sys.modules.get("train_station_b200")
        if mod is not None:
            mod.clear_gradients()
            mod.set_matmul_precision(mod.FP32)
            mod.set_fusion(True)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = bits(got) != bits(want)
    # NaNs with different payloads still count as equal results of the same IEEE operation
    bad &= ~(np.isnan(got) & np.isnan(want))
    if bad.any():
        i = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} elements differ bitwise; first at {tuple(i)}: "
                             f"{got[tuple(i)]!r} vs {want[tuple(i)]!r}")
