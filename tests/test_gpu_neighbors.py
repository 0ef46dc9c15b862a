"""Device neighbour list (zp_neighbors_count / zp_neighbors_fill through graph.neighbor_list)
against the CPU oracle: index arrays and shifts bit-exact; larger cases against the k-d tree
generator and through properties."""

from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [  # atoms, box, cutoff, cap
    (64, 10.0, 5.0, None),
    (64, 10.0, 5.0, 30),
    (200, 12.599, 6.0, 30),
    (40, 4.0, 6.0, 30),           # box smaller than the cutoff
    (40, 4.0, 6.0, None),
    (300, 18.0, 6.0, 12),
    (500, 12.0, 6.0, 30),         # box an exact multiple of the cutoff
    (1, 5.0, 6.0, None),
    (0, 5.0, 6.0, 30),
]


def run(pos, box, cutoff, cap):
    from zippel_b200.graph import neighbor_list
    ei, sh, rp = neighbor_list(torch.from_numpy(pos).cuda(), box, cutoff, cap)
    return ei.cpu().numpy(), sh.cpu().numpy(), rp.cpu().numpy()


@pytest.mark.parametrize("n,box,cutoff,cap", CASES)
def test_matches_oracle_bit_for_bit(n, box, cutoff, cap):
    from oracle import neighbors_oracle as no
    rng = np.random.default_rng(n + int(box * 10))
    pos = rng.random((n, 3)) * box
    want = no.neighbor_list(pos, box, cutoff, cap) if n else (
        np.zeros((2, 0), np.int64), np.zeros((0, 3)), np.zeros(1, np.int32))
    got = run(pos, box, cutoff, cap)
    for g, w in zip(got, want):
        assert g.shape == w.shape and np.array_equal(g, w)


@pytest.mark.parametrize("cap", [None, 20])
def test_positions_outside_the_box(cap):
    """Unwrapped positions (up to three boxes away): shifts refer to the positions as given."""
    from oracle import neighbors_oracle as no
    rng = np.random.default_rng(11)
    box = 9.0
    pos = rng.random((150, 3)) * box + rng.integers(-2, 3, (150, 3)) * box
    pos[:10] += rng.normal(0, 0.05, (10, 3))
    want = no.neighbor_list(pos, box, 5.0, cap)
    got = run(pos, box, 5.0, cap)
    for g, w in zip(got, want):
        assert g.shape == w.shape and np.array_equal(g, w)
    # the same atoms wrapped into the box give the same graph with shifted images
    wrapped = pos - np.floor(pos / box) * box
    ei_w, sh_w, rp_w = run(wrapped, box, 5.0, None)
    ei_u, sh_u, rp_u = run(pos, box, 5.0, None)
    assert np.array_equal(rp_w, rp_u) and np.array_equal(ei_w, ei_u)


def test_bench_graph_matches_generator_and_feeds_the_csr_build():
    """2000 atoms / 60 000 edges: same edges as the host generator; the list is already in the
    sorted order zp_csr_build defines (identity permutation, same row_ptr)."""
    from oracle import neighbors_oracle as no
    from zippel_b200.graph import EdgeGraph, periodic_neighbors
    box = float((2000 / 0.1) ** (1.0 / 3.0))
    pos = np.random.default_rng(0).random((2000, 3)) * box
    ei, sh, rp = run(pos, box, 6.0, 30)
    ei_k, sh_k = no.canonical(*periodic_neighbors(pos, box, 6.0, 30))
    assert ei.shape[1] == 60000
    assert np.array_equal(ei, ei_k) and np.array_equal(sh, sh_k)
    g = EdgeGraph.build(torch.from_numpy(ei).cuda(), 2000)
    assert torch.equal(g.perm.cpu(), torch.arange(60000, dtype=torch.int32))
    assert np.array_equal(g.row_ptr.cpu().numpy(), rp)


def test_large_box_properties_and_reproducibility():
    n, box = 100000, float((100000 / 0.1) ** (1.0 / 3.0))
    pos = np.random.default_rng(3).random((n, 3)) * box
    ei, sh, rp = run(pos, box, 6.0, 30)
    ei2, sh2, rp2 = run(pos, box, 6.0, 30)
    assert np.array_equal(ei, ei2) and np.array_equal(sh, sh2) and np.array_equal(rp, rp2)
    counts = np.diff(rp)
    assert counts.max() == 30 and counts.sum() == ei.shape[1]
    key = ei[1] * n + ei[0]
    assert np.all(np.diff(key) >= 0)
    vec = pos[ei[1]] - pos[ei[0]] + sh
    d2 = (vec * vec).sum(1)
    assert np.all(d2 < 36.0) and d2.min() > 0
    # the cap keeps the nearest: for sampled atoms compare with a direct search
    for j in np.random.default_rng(1).integers(0, n, 20):
        d = pos[j] - pos
        d -= box * np.round(d / box)
        dist2 = np.sort((d * d).sum(1))[1:31]
        mine = np.sort(d2[rp[j]:rp[j + 1]])
        assert np.allclose(mine, dist2, rtol=1e-12, atol=0)


def test_rejections():
    from zippel_b200 import _lib
    from zippel_b200.graph import neighbor_list
    with pytest.raises(ValueError):
        neighbor_list(torch.tensor([[0.5, 0.5, float("nan")]], dtype=torch.float64).cuda(), 10.0,
                      5.0, 30)
    with pytest.raises(_lib.ZpError):
        neighbor_list(torch.rand(10, 3, dtype=torch.float64).cuda(), 10.0, 5.0, 1000)
    with pytest.raises(_lib.ZpError):
        neighbor_list(torch.rand(10, 3, dtype=torch.float64).cuda(), 0.1, 5.0, 30)   # reach > 8
