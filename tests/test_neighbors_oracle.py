"""The neighbour-list oracle (brute force, squared distances) against the package's k-d tree
generator (sqrt distances) on the same seeded inputs: identical edge sets, shifts and caps."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import neighbors_oracle as no
from zippel_b200.graph import periodic_neighbors

CASES = [  # atoms, box, cutoff, cap
    (64, 10.0, 5.0, None),
    (64, 10.0, 5.0, 30),
    (200, 12.599, 6.0, 30),       # one structure of the batched configuration
    (40, 4.0, 6.0, 30),           # box smaller than the cutoff: several images, self images
    (40, 4.0, 6.0, None),
    (300, 18.0, 6.0, 12),
    (1, 5.0, 6.0, None),          # a single atom sees only its own images
]


@pytest.mark.parametrize("n,box,cutoff,cap", CASES)
def test_oracle_matches_kd_tree_generator(n, box, cutoff, cap):
    rng = np.random.default_rng(n + int(box * 10))
    pos = rng.random((n, 3)) * box
    ei, sh, row_ptr = no.neighbor_list(pos, box, cutoff, cap)
    ei_k, sh_k = periodic_neighbors(pos, box, cutoff, cap)
    ei_k, sh_k = no.canonical(ei_k, sh_k)
    assert np.array_equal(ei, ei_k) and np.array_equal(sh, sh_k)
    counts = np.diff(row_ptr)
    assert counts.sum() == ei.shape[1]
    if cap:
        assert counts.max() <= cap
    assert np.all(np.diff(ei[1]) >= 0)                      # destination-sorted
    vec = pos[ei[1]] - pos[ei[0]] + sh
    assert np.all((vec * vec).sum(1) < cutoff * cutoff)
    assert not np.any((ei[0] == ei[1]) & (np.abs(sh).sum(1) == 0))


def test_cap_keeps_the_nearest():
    rng = np.random.default_rng(7)
    pos = rng.random((120, 3)) * 9.0
    full = no.neighbor_list(pos, 9.0, 6.0, None)
    capped = no.neighbor_list(pos, 9.0, 6.0, 10)
    d_full = np.linalg.norm(pos[full[0][1]] - pos[full[0][0]] + full[1], axis=1)
    d_cap = np.linalg.norm(pos[capped[0][1]] - pos[capped[0][0]] + capped[1], axis=1)
    for j in range(120):
        a = np.sort(d_full[full[0][1] == j])[:10]
        b = np.sort(d_cap[capped[0][1] == j])
        assert np.array_equal(a, b)
