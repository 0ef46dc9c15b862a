"""The C-ABI library on a machine without a GPU: it builds, loads, exports every function that
include/zippel_b200.h declares, the ctypes binding lists exactly those, and the entry points
that need no device (status strings, size queries, argument checks) behave."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "zippel_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(zp_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from zippel_b200 import _lib, build
    build.build_library()
    return _lib.load()


def test_header_declares_the_path():
    names = declared_functions()
    for must in ("zp_plan_create", "zp_csr_build", "zp_eso2_forward", "zp_eso2_backward",
                 "zp_wigner_forward", "zp_wigner_backward", "zp_linear_forward",
                 "zp_layernorm_silu_forward", "zp_plan_device_status"):
        assert must in names


def test_every_declared_symbol_is_exported_and_bound(lib):
    from zippel_b200 import _lib
    raw = ctypes.CDLL(str(_lib.lib_path()))
    names = declared_functions()
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert sorted(_lib.SIGNATURES) == names


def test_host_only_entry_points(lib):
    assert lib.zp_status_string(0).decode().lower().startswith("ok")
    texts = {lib.zp_status_string(i).decode() for i in range(8)}
    assert len(texts) == 8                                     # one text per status code
    assert lib.zp_kernel_class_name(0).decode() and lib.zp_kernel_class_name(13).decode()
    assert lib.zp_csr_work_bytes(1000, 100) > 0
    assert lib.zp_layernorm_work_bytes(128) >= 2 * 128 * 4
    # argument checks come before any CUDA call
    assert lib.zp_layernorm_silu_forward(4, 6, None, None, None, 1e-5, None, None, None, None) == 2
    assert lib.zp_plan_destroy(None) in (0, 1)
    assert lib.zp_workspace_bytes(None, 10, 10, 1) == 0
