"""Shared test plumbing: the ``gpu`` marker, fixture loading, repo-root imports."""

from __future__ import annotations

import json
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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str):
    """Return ``(meta, tensors)``; uint16 arrays are bf16 bit patterns."""
    data = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(data["meta"]))
    tensors = {}
    for key in data.files:
        if key == "meta":
            continue
        arr = data[key]
        if arr.dtype == np.uint16:
            tensors[key] = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
        else:
            tensors[key] = torch.from_numpy(arr.copy())
    return meta, tensors


def regenerate_op_inputs(meta):
    """Re-create the seeded inputs of a sampled (large) golden op case.

    Must stay in lock-step with ``op_case`` in ``tests/golden/make_golden.py``.
    """
    dtype = getattr(torch, meta["dtype"])
    b, g, slots, c, events = (meta[k] for k in ("b", "g", "slots", "c", "events"))
    mean_a, scale_a, mean_b, scale_b = 0.25, 0.02, 1.0, 0.02
    torch.manual_seed(meta["seed"])
    k = int(round(slots ** 0.5))
    x = torch.randn(b, g * k, g * k, c).to(dtype)
    alpha = (mean_a + scale_a * torch.randn(events, c, slots)).to(dtype)
    beta = (mean_b + scale_b * torch.randn(events, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * k, g * k, c).to(dtype)
    return dict(x=x, alpha=alpha, beta=beta, dz=torch.stack(dz), gz=torch.stack(gz), gy=gy)


@pytest.fixture(scope="session", autouse=True)
def full_precision_reference_math():
    """fp32 comparisons must not silently use TF32 (mirrors the reference's conftest)."""
    old = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = old
