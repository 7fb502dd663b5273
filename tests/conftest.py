"""Shared pytest configuration: markers, import paths, fixtures."""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
for extra in (ROOT, ROOT / "oracle"):
    if str(extra) not in sys.path:
        sys.path.insert(0, str(extra))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")
    config.addinivalue_line("markers", "slow: full-size configuration, takes longer")


def b200_available() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def pytest_collection_modifyitems(config, items):
    if b200_available():
        return
    skip = pytest.mark.skip(reason="requires a B200 (compute capability 10.x) GPU")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


_TORCH_DTYPES = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16,
                 "torch.float32": torch.float32}


def load_golden(name: str) -> dict:
    """Decode one fixture written by tests/golden/make_golden.py into torch tensors."""

    raw = np.load(GOLDEN / f"{name}.npz")
    dtype = _TORCH_DTYPES[str(raw["dtype"])]
    g_dtype = _TORCH_DTYPES[str(raw["g_dtype"])]
    scale = float(raw["scale"])
    out = {"dtype": dtype, "g_dtype": g_dtype, "scale": None if scale < 0 else scale}
    low = {"q", "k", "v", "beta", "w", "out", "out_chunk16", "dq", "dk", "dv", "dbeta", "dw", "d_out"}
    for key in raw.files:
        if key in ("dtype", "g_dtype", "scale"):
            continue
        arr = raw[key]
        if key in low or (key in ("g", "dg") and g_dtype != torch.float32):
            want = dtype if key in low else g_dtype
            out[key] = torch.from_numpy(arr.copy()).view(want)
        else:
            out[key] = torch.from_numpy(np.asarray(arr).copy())
    return out


@pytest.fixture
def golden():
    return load_golden
