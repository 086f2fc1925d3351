import ctypes
import importlib
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))

TOL_RTOL = 1e-2   # fp16 outputs vs the fp32 oracle: |got - ref| <= atol + rtol * |ref|
TOL_ATOL = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("triton-rs_b200")


@pytest.fixture(scope="session")
def P(pkg):
    return pkg.prelude


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    return o


@pytest.fixture(scope="session")
def oracle_c():
    """The C/OpenMP oracle (built by `make -C oracle`), as a ctypes handle."""
    so = ROOT / "oracle" / "liboracle_c.so"
    if not so.exists():
        import subprocess
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True)
    return ctypes.CDLL(str(so))


def assert_close(got, ref, rtol=TOL_RTOL, atol=TOL_ATOL, what=""):
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside tolerance; worst |err| {err.max():.4g} "
                           f"at ref {ref.flat[err.argmax()]:.4g}")


def golden(name):
    return np.load(ROOT / "tests" / "golden" / f"{name}.npz")
