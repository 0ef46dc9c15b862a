"""Size-independent properties of the block at the benchmark shape (2000 atoms / 60 000 edges,
lmax 4, mmax 2, C 128), where the CPU oracle is too slow to evaluate the whole graph:

* the edge frame's third Euler angle is a gauge: node_out does not depend on gamma
  (reference blocks/wigner.py:145-146; tests/test_ref_block.py holds the same property for E);
* E is invariant and the forces are equivariant under a global rotation when the input
  embeddings are scalars (l = 0 rows only);
* the order of the edge list does not matter (the CSR sort canonicalises it);
* the VJP is linear in the upstream gradient.

The tolerances are those of the fp32 path against the FP64 oracle (1e-5): every comparison is
between two runs of the CUDA path that differ by rounding only."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.helpers import gpu_node_out_and_vjp, make_block, rel_l2
from zippel_b200.blocks.wigner import gamma_harmonics
from zippel_b200.graph import synthetic_batch

pytestmark = pytest.mark.gpu

CFG = dict(lmax=4, mmax=2, sphere_channels=128, hidden_channels=128, edge_channels=128,
           num_distance_basis=64, cutoff=6.0)


@pytest.fixture(scope="module")
def setup():
    batch = synthetic_batch(2000, 4, 128, 6.0, seed=3)
    assert batch["meta"]["n_edges"] == 60000
    block = make_block(CFG, orc.init_params(CFG, seed=0))
    g = torch.Generator().manual_seed(5)
    up = torch.randn(batch["x_node"].shape, generator=g)
    return batch, block, up


def test_gamma_is_a_gauge(setup):
    batch, block, up = setup
    e = batch["meta"]["n_edges"]
    g = torch.Generator().manual_seed(7)
    cg, sg = gamma_harmonics(torch.rand(e, generator=g, dtype=torch.float64) * 2 * math.pi, 4)
    other = dict(batch, cos_gamma_k=cg.float(), sin_gamma_k=sg.float())
    a = gpu_node_out_and_vjp(block, batch, up)
    b = gpu_node_out_and_vjp(block, other, up)
    assert rel_l2(a[0], b[0]) < 1e-5
    assert rel_l2(a[1], b[1]) < 1e-5 and rel_l2(a[2], b[2]) < 1e-5
    for name in ("c1_m0.weight", "c2_m.1.weight", "rad_func.6.weight"):
        assert rel_l2(a[3][name], b[3][name]) < 1e-5, name


def _rotation(seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(3, 3, generator=g, dtype=torch.float64))
    q = q * torch.sign(torch.diagonal(r))
    if torch.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


def _energy_and_forces(block, batch):
    pos = batch["pos"].cuda().requires_grad_(True)
    e = block(pos, batch["atomic_numbers"].cuda(), batch["x_node"].cuda(), batch["edge_index"].cuda(),
              batch["shifts"].cuda(), batch["cos_gamma_k"].cuda(), batch["sin_gamma_k"].cuda())
    (de,) = torch.autograd.grad(e, pos)
    return e.detach().double().cpu(), -de.double().cpu()


def test_energy_invariant_and_forces_equivariant_under_rotation(setup):
    batch, block, _ = setup
    x0 = torch.zeros_like(batch["x_node"])
    x0[:, 0] = batch["x_node"][:, 0]                      # scalar embeddings only
    rot = _rotation(11)
    base = dict(batch, x_node=x0)
    turned = dict(base, pos=(batch["pos"].double() @ rot.T).float(),
                  shifts=(batch["shifts"].double() @ rot.T).float())
    e0, f0 = _energy_and_forces(block, base)
    e1, f1 = _energy_and_forces(block, turned)
    assert abs(e1 - e0).item() < 1e-5 * max(abs(e0).item(), 1.0)
    assert rel_l2(f1, f0 @ rot.T) < 2e-5


def test_edge_order_does_not_matter(setup):
    batch, block, up = setup
    e = batch["meta"]["n_edges"]
    perm = torch.randperm(e, generator=torch.Generator().manual_seed(13))
    shuffled = dict(batch, edge_index=batch["edge_index"][:, perm], shifts=batch["shifts"][perm],
                    cos_gamma_k=batch["cos_gamma_k"][perm], sin_gamma_k=batch["sin_gamma_k"][perm])
    a = gpu_node_out_and_vjp(block, batch, up)
    b = gpu_node_out_and_vjp(block, shuffled, up)
    assert rel_l2(a[0], b[0]) < 2e-6 and rel_l2(a[1], b[1]) < 2e-6 and rel_l2(a[2], b[2]) < 2e-6


def test_vjp_is_linear_in_the_upstream_gradient(setup):
    batch, block, up = setup
    up2 = torch.randn(up.shape, generator=torch.Generator().manual_seed(17))
    a = gpu_node_out_and_vjp(block, batch, up)
    b = gpu_node_out_and_vjp(block, batch, up2)
    c = gpu_node_out_and_vjp(block, batch, up + 2.0 * up2)
    assert rel_l2(c[1], a[1] + 2.0 * b[1]) < 1e-5
    assert rel_l2(c[2], a[2] + 2.0 * b[2]) < 1e-5
    for name in ("c1_m0.weight", "c1_m.0.weight", "c2_m0.bias", "elem_emb.weight"):
        assert rel_l2(c[3][name], a[3][name] + 2.0 * b[3][name]) < 1e-5, name
