"""Property tests of the oracle, after the reference's tests/test_ref_block.py:95-225 and
tests/test_ir_wigner.py:93-100; they are what validates the ``mmax < lmax`` extension, for
which the reference has no output to compare against."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc

DT = torch.float64


def small_cfg(lmax, mmax, c=6):
    return dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=c, edge_channels=4,
                num_distance_basis=5, cutoff=9.0)


def make_batch(cfg, n=10, e=36, seed=0):
    g = torch.Generator("cpu").manual_seed(seed)
    gamma = torch.rand(e, generator=g, dtype=DT) * 2 * torch.pi
    src = torch.randint(0, n, (e,), generator=g)
    dst = (src + 1 + torch.randint(0, n - 1, (e,), generator=g)) % n
    return dict(
        pos=torch.rand(n, 3, generator=g, dtype=DT) * 4.0,
        z=torch.randint(1, 30, (n,), generator=g),
        x_node=torch.randn(n, (cfg["lmax"] + 1) ** 2, cfg["sphere_channels"], generator=g, dtype=DT),
        edge_index=torch.stack([src, dst]), shifts=torch.zeros(e, 3, dtype=DT), gamma=gamma)


def energy(params, cfg, b, jd, pos=None, x_node=None, gamma=None):
    cg, sg = orc.gamma_harmonics(b["gamma"] if gamma is None else gamma, cfg["lmax"])
    return orc.block_energy(params, cfg, b["pos"] if pos is None else pos, b["z"],
                            b["x_node"] if x_node is None else x_node, b["edge_index"],
                            b["shifts"], cg, sg, jd)


SHAPES = [(2, 2), (4, 2), (6, 2), (3, 1)]


@pytest.mark.parametrize("lmax,mmax", SHAPES)
def test_wigner_blocks_orthogonal(lmax, mmax, jd64):
    b = make_batch(small_cfg(lmax, mmax))
    ev, _ = orc.edge_geometry(b["pos"], b["edge_index"], b["shifts"])
    cg, sg = orc.gamma_harmonics(b["gamma"], lmax)
    w = orc.wigner_full(ev, cg, sg, lmax, jd64)
    eye = torch.eye(w.shape[1], dtype=DT)
    assert (w @ w.transpose(1, 2) - eye).abs().max().item() < 1e-12
    # the edge frame maps the edge direction onto +y (l = 1 block is the cartesian rotation)
    unit = ev / ev.norm(dim=-1, keepdim=True)
    y = torch.einsum("eij,ej->ei", w[:, 1:4, 1:4], unit)
    assert (y - torch.tensor([0.0, 1.0, 0.0], dtype=DT)).abs().max().item() < 1e-12


@pytest.mark.parametrize("lmax,mmax", SHAPES)
def test_energy_independent_of_gamma(lmax, mmax, jd64):
    cfg = small_cfg(lmax, mmax)
    params, b = orc.init_params(cfg, 1), make_batch(cfg)
    g = torch.Generator("cpu").manual_seed(99)
    vals = [energy(params, cfg, b, jd64,
                   gamma=torch.rand(b["gamma"].shape, generator=g, dtype=DT) * 6.28).item()
            for _ in range(3)]
    assert max(vals) - min(vals) < 1e-11 * max(1.0, abs(vals[0]))


@pytest.mark.parametrize("lmax,mmax", SHAPES)
def test_rotation_invariance_and_force_equivariance(lmax, mmax, jd64):
    cfg = small_cfg(lmax, mmax)
    params, b = orc.init_params(cfg, 2), make_batch(cfg, seed=3)
    ang = lambda v: torch.tensor([v], dtype=DT)  # noqa: E731
    d = orc.wigner_from_angles(ang(0.7), ang(1.9), ang(4.1), lmax, jd64)[0]
    r = d[1:4, 1:4]
    p0 = b["pos"].clone().requires_grad_(True)
    e0 = energy(params, cfg, b, jd64, pos=p0)
    (f0,) = torch.autograd.grad(e0, p0)
    p1 = (b["pos"] @ r.T).clone().requires_grad_(True)
    e1 = energy(params, cfg, b, jd64, pos=p1,
                x_node=torch.einsum("ij,njc->nic", d, b["x_node"]))
    (f1,) = torch.autograd.grad(e1, p1)
    assert abs(e0.item() - e1.item()) < 1e-10 * max(1.0, abs(e0.item()))
    assert (f1 - f0 @ r.T).abs().max().item() < 1e-9 * max(1.0, f0.abs().max().item())


def test_force_matches_central_differences(jd64):
    cfg = small_cfg(4, 2, c=4)
    params, b = orc.init_params(cfg, 4), make_batch(cfg, n=6, e=14, seed=5)
    p0 = b["pos"].clone().requires_grad_(True)
    (f,) = torch.autograd.grad(energy(params, cfg, b, jd64, pos=p0), p0)
    h = 1e-5
    for (i, a) in [(0, 0), (2, 1), (5, 2)]:
        dp = torch.zeros_like(b["pos"]); dp[i, a] = h
        fd = (energy(params, cfg, b, jd64, pos=b["pos"] + dp)
              - energy(params, cfg, b, jd64, pos=b["pos"] - dp)) / (2 * h)
        assert abs(fd.item() - f[i, a].item()) < 1e-6 * max(1.0, abs(fd.item()))


def test_translation_and_permutation_invariance(jd64):
    cfg = small_cfg(4, 2)
    params, b = orc.init_params(cfg, 6), make_batch(cfg, seed=7)
    e0 = energy(params, cfg, b, jd64).item()
    e1 = energy(params, cfg, b, jd64, pos=b["pos"] + torch.tensor([0.3, -1.2, 2.0], dtype=DT)).item()
    assert abs(e0 - e1) < 1e-10 * max(1.0, abs(e0))
    perm = torch.randperm(b["pos"].shape[0], generator=torch.Generator().manual_seed(1))
    inv = torch.empty_like(perm); inv[perm] = torch.arange(len(perm))
    b2 = dict(b, pos=b["pos"][perm], z=b["z"][perm], x_node=b["x_node"][perm],
              edge_index=inv[b["edge_index"]])
    assert abs(e0 - energy(params, cfg, b2, jd64).item()) < 1e-10 * max(1.0, abs(e0))
