"""The oracle against the golden vectors produced by the unmodified reference
(tests/golden/make_golden.py), plus the reference's own pinned layout tables."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.conftest import golden_names, load_golden


def rel(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()


@pytest.mark.parametrize("name", golden_names())
def test_wigner_matches_reference(name, jd64):
    c = load_golden(name)
    edge_vec, _ = orc.edge_geometry(c["pos"], c["edge_index"], c["shifts"])
    w = orc.wigner_full(edge_vec, c["cos_gamma_k"], c["sin_gamma_k"], c["cfg"]["lmax"], jd64)
    assert (w - c["wigner"]).abs().max().item() < 1e-14


@pytest.mark.parametrize("name", golden_names())
def test_forward_matches_reference(name, jd64):
    c = load_golden(name)
    args = (c["params"], c["cfg"], c["pos"], c["atomic_numbers"], c["x_node"], c["edge_index"],
            c["shifts"], c["cos_gamma_k"], c["sin_gamma_k"], jd64)
    node_out = orc.block_node_out(*args)
    assert rel(node_out, c["node_out"]) < 1e-13
    energy = orc.block_energy(*args)
    assert abs(energy.item() - c["energy"].item()) < 1e-12 * max(1.0, abs(c["energy"].item()))


@pytest.mark.parametrize("name", golden_names())
def test_vjp_matches_reference(name, jd64):
    c = load_golden(name)
    pos = c["pos"].clone().requires_grad_(True)
    x_node = c["x_node"].clone().requires_grad_(True)
    params = {k: v.clone().requires_grad_(True) for k, v in c["params"].items()}
    node_out = orc.block_node_out(params, c["cfg"], pos, c["atomic_numbers"], x_node,
                                  c["edge_index"], c["shifts"], c["cos_gamma_k"],
                                  c["sin_gamma_k"], jd64)
    names = list(params)
    grads = torch.autograd.grad((node_out * c["upstream"]).sum(),
                                [x_node, pos, *params.values()], allow_unused=True)
    assert rel(grads[0], c["vjp_x_node"]) < 1e-12
    assert rel(grads[1], c["vjp_pos"]) < 1e-11
    for n, g in zip(names, grads[2:]):
        want = c["vjp_params"][n]
        if g is None:
            assert want.abs().max().item() == 0.0, n
        else:
            assert rel(g, want) < 1e-11 or (g - want).abs().max().item() < 1e-13, n


@pytest.mark.parametrize("name", golden_names())
def test_force_matches_reference(name, jd64):
    c = load_golden(name)
    pos = c["pos"].clone().requires_grad_(True)
    e = orc.block_energy(c["params"], c["cfg"], pos, c["atomic_numbers"], c["x_node"],
                         c["edge_index"], c["shifts"], c["cos_gamma_k"], c["sin_gamma_k"], jd64)
    (f,) = torch.autograd.grad(e, pos)
    assert rel(f, c["de_dpos"]) < 1e-11


def test_layout_tables_pinned_by_reference_tests():
    # tests/test_anchor_lmax4.py:38-44 and tests/test_ref_vs_fairchem.py:145-155
    assert orc.m_sizes(4, 4) == (5, 4, 3, 2, 1)
    assert orc.m_splits(4, 4) == (5, 8, 6, 4, 2)
    assert orc.gate_expand_index(4, 4).numel() == 24
    assert orc.m_splits(2, 2) == (3, 4, 2)
    cfg = dict(lmax=2, mmax=2, sphere_channels=128, hidden_channels=128, edge_channels=128,
               num_distance_basis=64)
    shapes = orc.param_shapes(cfg)
    assert shapes["rad_func.6.weight"][0] == 1536
    assert shapes["c1_m0.weight"] == (128 * 3 + 256, 768)
    assert len(shapes) == 23
    # mmax < lmax extension
    assert orc.m_splits(4, 2) == (5, 8, 6) and orc.m_splits(6, 2) == (7, 12, 10)
    assert orc.gate_expand_index(4, 2).tolist() == [0, 1, 2, 3, 0, 1, 2, 3, 0, 1, 2, 3,
                                                    1, 2, 3, 1, 2, 3]
    cfg4 = dict(cfg, lmax=4)
    assert orc.param_shapes(cfg4)["rad_func.6.weight"][0] == 3072
    assert sum(torch.Size(s).numel() for s in orc.param_shapes(cfg4).values()) == 4892929


def test_to_m_is_permutation_when_square():
    for l in (1, 2, 3, 4):
        m = orc.to_m_matrix(l, l)
        assert m.shape == ((l + 1) ** 2, (l + 1) ** 2)
        assert torch.equal(m @ m.T, torch.eye((l + 1) ** 2, dtype=m.dtype))
