"""Shared test plumbing.

Markers: ``gpu`` = needs a CUDA device (the parity tests proper; they call the kernels through
the C ABI).  Everything else runs on a CPU-only machine.

Tolerance used everywhere (the meaning of "within 1e-5 relative" here):
    |got - want| <= tol + tol * |want|      tol = 1e-5 for fp32, 2e-3 for fp16
Pure relative error is meaningless next to the zeros of a normalised tensor, so the bound is
the usual allclose form with atol = rtol = tol.  Gathers and adds are compared bit for bit.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOL = {"float32": 1e-5, "float16": 2e-3}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _ensure_library_built() -> None:
    """Tests may run on a fresh checkout: compile libsdfl.so (nvcc cross-compiles without a GPU) when
    it is missing.  The package itself never builds or falls back."""
    import importlib.util
    if os.path.exists(os.path.join(ROOT, "mobile-stable-diffusion_b200", "lib", "libsdfl.so")):
        return
    spec = importlib.util.spec_from_file_location(
        "_sdfl_build", os.path.join(ROOT, "mobile-stable-diffusion_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


def load_package():
    """The product package (its directory name has a hyphen, hence importlib)."""
    _ensure_library_built()
    return importlib.import_module("mobile-stable-diffusion_b200")


@pytest.fixture(scope="session")
def sdfl():
    return load_package()


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.port_lib()
    return oracle


def assert_close(got, want, tol: float, what: str = "") -> None:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite values in result"
    err = np.abs(got - want)
    bound = tol + tol * np.abs(want)
    worst = float((err / bound).max()) if err.size else 0.0
    assert worst <= 1.0, (f"{what}: max |err|/bound = {worst:.3f} "
                          f"(max abs err {float(err.max()):.3e}, tol {tol})")


def assert_bit_equal(got, want, what: str = "") -> None:
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    assert got.dtype == want.dtype and got.shape == want.shape, what
    assert got.tobytes() == want.tobytes(), f"{what}: bit patterns differ"


def rng_for(config: int, case: int) -> np.random.Generator:
    """Seed convention of the workload: seed = 1000 * config + case."""
    return np.random.Generator(np.random.PCG64(1000 * config + case))
