"""The reference's benchmark fixtures rebuilt from their recipe: the content hashes recorded in
the reference's manifest (tests/golden/reference_fixtures.json) must be reproduced bit for bit.
That pins the structure generator, the neighbour-list rule (uncapped), the edge order and the
file schema to the reference's own records.  CPU: the brute-force oracle and the host k-d tree;
GPU: the device neighbour list, all six fixtures up to 48 668 atoms / 3.8 M edges."""

from __future__ import annotations

import json
import pathlib

import numpy as np
import pytest
import torch

from zippel_b200 import fixtures as fx

GOLD = {r["name"]: r for r in json.loads(
    (pathlib.Path(__file__).parent / "golden" / "reference_fixtures.json").read_text())["fixtures"]}


def check_meta(meta, gold):
    for key in ("n_atoms", "n_edges", "avg_degree", "reps", "lattice_a", "seed"):
        assert meta[key] == gold[key], key
    assert meta["min_edge_len"] == gold["min_edge_len"]
    assert meta["max_edge_len"] == gold["max_edge_len"]
    assert meta["sha256_content"] == gold["sha256_content"]


@pytest.mark.parametrize("name", ["si_small", "cu_small"])
def test_oracle_neighbour_rule_reproduces_the_reference_hash(name):
    from oracle import neighbors_oracle as no
    element, z, structure, a, reps = fx.SPECS[name]
    pos, cell = fx.bulk_supercell(structure, a, reps, 0)
    ei, sh, _ = no.neighbor_list(pos, a * reps, fx.CUTOFF, None)
    ei, sh = fx.canonical_order(ei, sh)
    arrays = dict(pos=pos, cell=cell, atomic_numbers=np.full(len(pos), z, np.int64),
                  edge_index=ei, shifts=sh)
    assert fx.content_hash(arrays) == GOLD[name]["sha256_content"]


@pytest.mark.parametrize("name", ["si_small", "cu_small", "si_medium", "cu_medium"])
def test_host_generator_reproduces_the_reference_hash(name):
    arrays, meta = fx.build_fixture(name, device="cpu")
    check_meta(meta, GOLD[name])


def test_round_trip_and_schema_checks(tmp_path):
    arrays, meta = fx.build_fixture("si_small", device="cpu")
    path = tmp_path / "si_small.npz"
    fx.write_fixture(path, arrays, meta)
    back, meta2 = fx.read_fixture(path)
    assert meta2 == meta and fx.content_hash(back) == meta["sha256_content"]
    for k in fx.CONTENT_KEYS:
        assert back[k].dtype == arrays[k].dtype and np.array_equal(back[k], arrays[k])
    # another schema version is rejected; so is a file whose arrays do not match its record
    np.savez_compressed(tmp_path / "v2.npz", schema_version=np.array(2), meta=json.dumps(meta),
                        **arrays)
    with pytest.raises(ValueError):
        fx.read_fixture(tmp_path / "v2.npz")
    bad = dict(arrays); bad["pos"] = arrays["pos"] + 1e-9
    fx.write_fixture(tmp_path / "bad.npz", bad, meta)
    with pytest.raises(ValueError):
        fx.read_fixture(tmp_path / "bad.npz")
    with pytest.raises(FileNotFoundError):
        fx.read_fixture(tmp_path / "nope.npz")


def test_load_batch_schema(tmp_path):
    from zippel_b200.blocks.eso2 import BlockConfig
    arrays, meta = fx.build_fixture("si_small", device="cpu")
    cfg = BlockConfig(lmax=2, mmax=2, sphere_channels=8, hidden_channels=8)
    b = fx.load_batch((arrays, meta), "cpu", torch.float64, cfg)
    assert set(b) == {"pos", "cell", "atomic_numbers", "x_node", "edge_index", "shifts",
                      "cos_gamma_k", "sin_gamma_k", "e_ref", "f_ref", "meta"}
    assert b["x_node"].shape == (216, 9, 8) and b["cos_gamma_k"].shape == (9576, 3)
    assert b["pos"].requires_grad and b["edge_index"].dtype == torch.int64
    b2 = fx.load_batch((arrays, meta), "cpu", torch.float64, cfg)
    assert torch.equal(b["x_node"], b2["x_node"]) and torch.equal(b["cos_gamma_k"], b2["cos_gamma_k"])
    assert torch.allclose(b["cos_gamma_k"] ** 2 + b["sin_gamma_k"] ** 2,
                          torch.ones_like(b["cos_gamma_k"]))


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(fx.SPECS))
def test_device_neighbour_list_reproduces_the_reference_hash(name):
    arrays, meta = fx.build_fixture(name, device="cuda")
    check_meta(meta, GOLD[name])


@pytest.mark.gpu
def test_block_parity_on_a_reference_fixture(jd64):
    """si_small (216 atoms, 9 576 edges, no cap) through the module against the oracle: node
    output and every gradient within the fp32 tolerance of 1e-5."""
    from oracle import eso2_oracle as orc
    from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                               oracle_node_out_and_vjp)
    from zippel_b200.blocks.eso2 import BlockConfig
    cfg = dict(lmax=2, mmax=2, sphere_channels=16, hidden_channels=16, edge_channels=16,
               num_distance_basis=16, cutoff=6.0)
    arrays, meta = fx.build_fixture("si_small", device="cuda")
    batch = fx.load_batch((arrays, meta), "cpu", torch.float64, BlockConfig(**cfg),
                          requires_grad=False)
    params = orc.init_params(cfg, seed=3)
    g = torch.Generator("cpu").manual_seed(5)
    up = torch.randn(batch["x_node"].shape, generator=g, dtype=torch.float64)
    want = oracle_node_out_and_vjp(cfg, params, batch, up, jd64)
    got = gpu_node_out_and_vjp(make_block(cfg, params), batch, up)
    check_against(*got, *want, tol=1e-5)
