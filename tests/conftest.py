"""Shared test plumbing: the `gpu` marker, import paths, seeded inputs."""

from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_package():
    """The package directory carries a hyphen, so it is imported by name."""
    return importlib.import_module("dilution-attention_b200")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def kernels(pkg):
    return pkg.kernels


def seeded(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def make_inputs(b, h, t, d, seed, scales=(1.0, 1.0, 1.0, 1.0)):
    """q, k, v, dout from consecutive CPU seeds (same recipe as make_golden.py)."""
    return tuple(seeded((b, h, t, d), seed + i, scales[i]) for i in range(4))


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max-abs error over max-abs reference: the reference's own gradient metric
    (tests/test_kernels.py:125-126 of the reference)."""
    return (got.double() - ref.double()).abs().max().item() / (ref.double().abs().max().item() + 1e-12)


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel may have given up a bounded wait."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        lib = load_package()._lib.load()
        rc = lib.dilution_device_status()
        assert rc == 0, lib.dilution_last_error().decode()


# The bid / share ablations stored in tests/golden/variants_b1h2t80d32.npz (key prefix, bid, share_cumsum).
VARIANTS = [("softmax_exclusive", "softmax", "exclusive"), ("softmax_none", "softmax", False),
            ("sigmoid_inclusive", "sigmoid", True), ("sigmoid_exclusive", "sigmoid", "exclusive"),
            ("sigmoid_none", "sigmoid", False), ("expshift_inclusive", "expshift", True),
            ("sigshift_inclusive", "sigshift", True), ("sigshift_none", "sigshift", False),
            ("relu_inclusive", "relu", True), ("relu2_inclusive", "relu2", True),
            ("softplus_inclusive", "softplus", True), ("minshift_inclusive", "minshift", True),
            ("relu_none", "relu", False), ("softplus_exclusive", "softplus", "exclusive")]
SHIFT = 80.0      # the divisor of the shifted bids in that fixture; the other bids ignore it


def variant_case(key):
    """q, k, v, dout and the reference's out, dq, dk, dv, demand of one stored variant."""
    g = golden("variants_b1h2t80d32.npz")
    case = {n: torch.from_numpy(g[n]) for n in ("q", "k", "v", "dout")}
    case.update({n: torch.from_numpy(g[f"{key}_{n}"]) for n in ("out", "dq", "dk", "dv", "demand")})
    return case
