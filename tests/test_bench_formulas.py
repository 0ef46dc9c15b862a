"""The work and traffic counts bench.py reports its roofline fractions against, checked against
the shapes of the block (reference blocks/eso2_ref.py:252-293 for the six SO(2) products)."""

import importlib.util
import pathlib

import pytest

from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block

ROOT = pathlib.Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_contraction_macs_per_edge(bench):
    # conv1: 1280x1152 + 2*1024*1024 + 2*768*768 ; conv2: 640x640 + 2*512*1024 + 2*384*768
    want = 1280 * 1152 + 2 * 1024 * 1024 + 2 * 768 * 768 + 640 * 640 + 2 * 512 * 1024 + 2 * 384 * 768
    assert bench.gemm_macs_per_edge(bench.CFG) == want == 6_799_360


def test_hbm_bytes_per_step(bench, monkeypatch):
    block = ESO2Block(BlockConfig(**bench.CFG))             # fp32 precision: two fp16 planes
    n, e = 2000, 60000
    got = bench.hbm_bytes_per_step(block, n, e)
    km, k, c, h, r = 19, 25, 128, 128, 3072
    w1 = 4 * h + km * h
    assert got["rotate_in"] == e * (r * 4 + km * 2 * c * 2 * 2)
    assert got["gate_fwd"] == e * (w1 * 4 + km * h * 2 * 2)
    assert got["rotate_grad_out"] == e * (km * c * 4 + km * c * 2 * 2)
    assert got["gate_bwd"] == e * (w1 * 4 + km * h * 4 + w1 * 2 * 2)
    assert got["rotate_in_bwd"] == e * (km * 2 * c * 4 + 2 * r * 4 + 2 * k * c * 4)
    assert got["src_reduce"] == e * 2 * k * c * 4 + n * k * c * 4
    assert got["rotate_back_scatter"] == e * km * c * 4 + n * k * c * 4
    # opt-in fused epilogues: the gate runs inside conv1, and what is left of the scatter is the
    # sum of the per-row partial sums (115 x C per node and per 32 edges)
    monkeypatch.setenv("ZP_FUSED_EPILOGUE", "1")
    fused = bench.hbm_bytes_per_step(block, n, e)
    assert "gate_fwd" not in fused
    assert fused["rotate_back_scatter"] == e * 115 * c * 4 // 32 + n * (k + 115) * c * 4
    monkeypatch.delenv("ZP_FUSED_EPILOGUE")
    one_plane = ESO2Block(BlockConfig(**bench.CFG), precision="bf16")
    assert bench.hbm_bytes_per_step(one_plane, n, e)["rotate_in"] == e * (r * 4 + km * 2 * c * 2)


def test_chunk_budget_quantisation():
    """The per-call edge budget keeps four significant bits: stable under small drifts of the
    free memory, never above the raw budget, never less than 7/8 of it."""
    from zippel_b200.blocks.eso2 import _quantise_budget

    for raw in (1024, 1025, 60000, 383_999, 384_000, 1_000_003, 6_000_000):
        q = _quantise_budget(raw)
        assert q <= raw and q * 8 >= raw * 7
        assert _quantise_budget(q) == q
    assert _quantise_budget(700_000) == _quantise_budget(710_000)     # same bucket
    assert _quantise_budget(15) == 15 and _quantise_budget(1) == 1
