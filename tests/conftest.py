"""Shared fixtures: package loader, seeded weights, golden files, metrics."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parents[1]
PKG_DIR = REPO / "qwen3.5-0.8b_b200"
GOLDEN = REPO / "tests" / "golden"
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def load_package():
    """Import the host-side package (its directory name is not a Python identifier)."""
    name = "q35_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(
        name, PKG_DIR / "__init__.py", submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def rel_l2(a, b) -> float:
    a = torch.as_tensor(np.asarray(a)).double().reshape(-1) if not torch.is_tensor(a) else a.double().reshape(-1)
    b = torch.as_tensor(np.asarray(b)).double().reshape(-1) if not torch.is_tensor(b) else b.double().reshape(-1)
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def weights(pkg):
    """Full seeded model (seed 0) as CPU bf16 tensors, checked against the stored stream pins."""
    torch.set_grad_enabled(False)
    P = pkg.weights.make_weights(seed=0)
    pins = np.load(GOLDEN / "weight_pins.npz")
    for name in pins.files:
        got = P[name].reshape(-1)[:64].float().numpy()
        assert np.array_equal(got, pins[name]), f"seeded weight stream changed: {name}"
    return P


@pytest.fixture(scope="session")
def golden():
    return {p.stem: np.load(p) for p in GOLDEN.glob("*.npz")}
