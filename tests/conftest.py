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


def assert_close_sum(got, ref, parts, rtol=TOL_RTOL, atol=TOL_ATOL, what=""):
    """For an output that is the SUM of fp16 tensors `parts` (e.g. the closing residual add of a layer:
    h1 + down): each summand is good to atol + rtol * |summand|, so the sum is good to the sum of those
    bounds.  The plain bound atol + rtol * |ref| is not attainable where large summands cancel: one fp16
    ulp of a summand of magnitude 40 is 0.03, whatever the sum comes to."""
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape and np.isfinite(got).all(), f"{what}: shape or non-finite output"
    bound = sum(atol + rtol * np.abs(np.asarray(p, dtype=np.float32)) for p in parts)
    err = np.abs(got - ref)
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside the propagated tolerance; worst |err| {err.max():.4g}"


def assert_close_terms(got, ref, mag, terms, rtol=TOL_RTOL, atol=TOL_ATOL, what=""):
    """For an output that is a weighted sum of `terms` fp16 tensors whose absolute values add up to `mag` (the
    fused-MoE combine): bound = terms * atol + rtol * mag, i.e. the per-term tolerance summed."""
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape and np.isfinite(got).all(), f"{what}: shape or non-finite output"
    err = np.abs(got - ref)
    bad = err > terms * atol + rtol * np.asarray(mag, dtype=np.float32)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside the propagated tolerance; worst |err| {err.max():.4g}"


def golden(name):
    return np.load(ROOT / "tests" / "golden" / f"{name}.npz")
