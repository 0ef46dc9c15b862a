"""Parity at the benchmark configurations' own shapes.

cfg0 (64 atoms, lmax 2, C 32) is compared with the oracle in full.  For the large shapes the GPU
runs the full graph while the oracle evaluates only the edges into a sample of destination nodes:
the upstream gradient is non-zero on those nodes only, so node_out rows, and ALL gradients
(x_node, positions, every parameter) are exactly those of the sub-edge-list -- a size-independent
check of the full-size run.  Run-to-run determinism of the scatter is checked bit for bit."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.helpers import check_against, gpu_node_out_and_vjp, make_block, oracle_node_out_and_vjp
from zippel_b200.graph import synthetic_batch

pytestmark = pytest.mark.gpu


def _cfg(lmax, mmax, c, nb, cutoff):
    return dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=c, edge_channels=c,
                num_distance_basis=nb, cutoff=cutoff)


def test_cfg0_full_oracle_parity(jd64):
    cfg = _cfg(2, 2, 32, 32, 5.0)
    batch = synthetic_batch(64, 2, 32, 5.0, box=10.0, max_neighbors=None, seed=0, dtype=torch.float64)
    assert batch["meta"]["n_edges"] == 2220
    params = orc.init_params(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    up = torch.randn(batch["x_node"].shape, generator=g, dtype=torch.float64)
    want = oracle_node_out_and_vjp(cfg, params, batch, up, jd64)
    got = gpu_node_out_and_vjp(make_block(cfg, params), batch, up)
    check_against(*got, *want, tol=1e-5)


def _sampled_check(cfg, batch, params, jd, precision, tol, n_sample, seed):
    n = batch["pos"].shape[0]
    g = torch.Generator().manual_seed(seed)
    nodes = torch.randperm(n, generator=g)[:n_sample]
    up = torch.zeros(batch["x_node"].shape, dtype=torch.float64)
    up[nodes] = torch.randn(n_sample, *up.shape[1:], generator=g, dtype=torch.float64)
    mask = torch.zeros(n, dtype=torch.bool)
    mask[nodes] = True
    keep = mask[batch["edge_index"][1]]
    sub = dict(batch, edge_index=batch["edge_index"][:, keep], shifts=batch["shifts"][keep],
               cos_gamma_k=batch["cos_gamma_k"][keep], sin_gamma_k=batch["sin_gamma_k"][keep])
    sub = {k: (v.double() if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in sub.items()}
    want = oracle_node_out_and_vjp(cfg, params, sub, up, jd)
    block = make_block(cfg, params, precision=precision)
    got = gpu_node_out_and_vjp(block, batch, up)
    again = gpu_node_out_and_vjp(block, batch, up)
    assert block.plan("cuda").device_status() == 0
    check_against(*got, *want, tol=tol, rows=nodes)             # gradients over ALL rows
    assert torch.equal(got[0], again[0]) and torch.equal(got[1], again[1])     # deterministic
    assert torch.equal(got[3]["c1_m.0.weight"], again[3]["c1_m.0.weight"])
    return got


def test_cfg1_cfg2_full_size_sampled(jd64):
    cfg = _cfg(4, 2, 128, 64, 6.0)
    batch = synthetic_batch(2000, 4, 128, 6.0, seed=0)
    assert batch["meta"]["n_edges"] == 60000
    _sampled_check(cfg, batch, orc.init_params(cfg, seed=0), jd64, "fp32", 1e-5, 40, seed=3)


def test_cfg3_batched_structures_bf16_sampled(jd64):
    cfg = _cfg(4, 2, 128, 64, 6.0)
    batch = synthetic_batch(200, 4, 128, 6.0, n_structures=16, seed=1)
    ei = batch["edge_index"]
    assert (ei[0] // 200 == ei[1] // 200).all()                   # block diagonal
    _sampled_check(cfg, batch, orc.init_params(cfg, seed=1), jd64, "bf16", 2e-2, 40, seed=4)


def test_cfg4_shape_lmax6_sampled(jd64):
    cfg = _cfg(6, 2, 128, 64, 6.0)
    batch = synthetic_batch(400, 6, 128, 6.0, seed=2)
    _sampled_check(cfg, batch, orc.init_params(cfg, seed=2), jd64, "fp32", 1e-5, 20, seed=5)
