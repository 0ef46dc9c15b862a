"""Shared pytest setup: the ``gpu`` marker, repo root on sys.path, golden-case loader."""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"
JD_PATH = ROOT / "zippel_b200" / "data" / "jd.npz"

torch.set_num_threads(8)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_names() -> list[str]:
    return sorted(p.stem for p in GOLDEN.glob("*.npz"))


def load_golden(name: str) -> dict:
    """One golden case as torch FP64/int64 tensors plus ``cfg`` and ``params`` dicts."""
    z = np.load(GOLDEN / f"{name}.npz")
    cfg = {}
    for k, v in zip(z["cfg_keys"], z["cfg_vals"]):
        cfg[str(k)] = float(v) if str(k) == "cutoff" else int(v)
    case = {"cfg": cfg, "params": {}, "vjp_params": {}}
    for key in z.files:
        if key.startswith("cfg_"):
            continue
        t = torch.from_numpy(z[key])
        if key.startswith("param:"):
            case["params"][key[6:]] = t
        elif key.startswith("vjp_param:"):
            case["vjp_params"][key[10:]] = t
        else:
            case[key] = t
    return case


@pytest.fixture(scope="session")
def jd64():
    from oracle.eso2_oracle import load_jd
    return load_jd(JD_PATH, 8)
