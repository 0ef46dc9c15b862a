"""CPU statement of the neighbour-list rule the device kernel implements (test infrastructure:
only tests may import this).

The reference project builds edge lists on the host with an external package and no neighbour
cap (fixtures/make_fixtures.py:13-15, 78-100: all pairs within the cutoff, both directions,
periodic shifts).  The rule restated here adds what the library defines on top of that:

* a pair is an edge iff  d2 = (dx*dx + dy*dy) + dz*dz < cutoff*cutoff  with
  d = (pos[dst] - pos[src]) + shift, shift = image * box, all in float64 in exactly this order;
* the zero-shift self pair is excluded;
* per destination only the ``max_neighbors`` smallest by (d2, src, shift_x, shift_y, shift_z)
  are kept;
* edges are listed in (dst, src, shift_x, shift_y, shift_z) order.

Brute force over all pairs and images: small inputs only.  Parity unpinned against the external
neighbour-list package (absent here); pinned against ``zippel_b200.graph.periodic_neighbors``
(k-d tree, sqrt distances) in tests/test_neighbors_oracle.py.
"""

from __future__ import annotations

import itertools

import numpy as np


def neighbor_list(pos: np.ndarray, box: float, cutoff: float,
                  max_neighbors: int | None) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Returns (edge_index [2, E] int64, shifts [E, 3] float64, row_ptr [N + 1] int32)."""
    pos = np.ascontiguousarray(pos, np.float64)
    n = pos.shape[0]
    reach = max(1, int(np.ceil(cutoff / box)))
    if n and (pos.min() < 0.0 or pos.max() >= box):
        # atoms given outside the box: their separations exceed one box length
        reach += int(np.ceil((pos.max() - pos.min()) / box))
    c2 = cutoff * cutoff
    srcs, dsts, shs, d2s = [], [], [], []
    for img in itertools.product(range(-reach, reach + 1), repeat=3):
        shift = np.asarray(img, np.float64) * box
        d = (pos[None, :, :] - pos[:, None, :]) + shift          # [src, dst, xyz]
        d2 = (d[..., 0] * d[..., 0] + d[..., 1] * d[..., 1]) + d[..., 2] * d[..., 2]
        hit = d2 < c2
        if img == (0, 0, 0):
            np.fill_diagonal(hit, False)
        i, j = np.nonzero(hit)
        srcs.append(i.astype(np.int64)); dsts.append(j.astype(np.int64))
        shs.append(np.broadcast_to(shift, (i.size, 3))); d2s.append(d2[i, j])
    src, dst = np.concatenate(srcs), np.concatenate(dsts)
    sh, d2 = np.concatenate(shs), np.concatenate(d2s)
    if max_neighbors is not None and max_neighbors > 0:
        order = np.lexsort((sh[:, 2], sh[:, 1], sh[:, 0], src, d2, dst))
        dst_o = dst[order]
        start = np.searchsorted(dst_o, np.arange(n))
        rank = np.arange(dst_o.size) - start[dst_o]
        keep = order[rank < max_neighbors]
        src, dst, sh = src[keep], dst[keep], sh[keep]
    order = np.lexsort((sh[:, 2], sh[:, 1], sh[:, 0], src, dst))
    src, dst, sh = src[order], dst[order], np.ascontiguousarray(sh[order])
    row_ptr = np.zeros(n + 1, np.int32)
    np.cumsum(np.bincount(dst, minlength=n), out=row_ptr[1:])
    return np.stack([src, dst]), sh, row_ptr


def canonical(edge_index: np.ndarray, shifts: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Any edge list in the (dst, src, shift) order of ``neighbor_list``."""
    src, dst = edge_index[0], edge_index[1]
    order = np.lexsort((shifts[:, 2], shifts[:, 1], shifts[:, 0], src, dst))
    return edge_index[:, order], np.ascontiguousarray(shifts[order])
