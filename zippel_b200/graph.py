"""Edge lists for the SO(2) block: synthetic periodic graphs, the neighbour cap, and the
destination-sorted CSR form the kernels consume.

The reference has no sorted form (it scatters with ``index_add_``, blocks/eso2_ref.py:346-349)
and applies no neighbour cap (fixtures/make_fixtures.py:13-15); both are defined here:

* cap: per destination node keep the ``max_neighbors`` incoming edges of smallest distance,
  ties broken by ``(dist, src, shift_x, shift_y, shift_z)``;
* order: edges sorted by ``(dst, src, original position)``; ``row_ptr[n]:row_ptr[n+1]`` are the
  edges into node ``n``.  ``csr_reference`` (numpy ``lexsort``) is the bit-exact statement of the
  order; ``EdgeGraph.build`` produces the same arrays on the device through ``zp_csr_build``.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import _lib


def csr_reference(edge_index: np.ndarray, n_nodes: int) -> dict[str, np.ndarray]:
    """Host statement of the sorted order (numpy).  Returns int32 arrays."""
    src, dst = np.asarray(edge_index[0], np.int64), np.asarray(edge_index[1], np.int64)
    e = src.shape[0]
    perm = np.lexsort((np.arange(e), src, dst)).astype(np.int32)
    src_s, dst_s = src[perm].astype(np.int32), dst[perm].astype(np.int32)
    row_ptr = np.zeros(n_nodes + 1, np.int32)
    np.cumsum(np.bincount(dst, minlength=n_nodes), out=row_ptr[1:])
    perm_src = np.lexsort((np.arange(e), src_s)).astype(np.int32)
    row_ptr_src = np.zeros(n_nodes + 1, np.int32)
    np.cumsum(np.bincount(src, minlength=n_nodes), out=row_ptr_src[1:])
    return dict(perm=perm, src=src_s, dst=dst_s, row_ptr=row_ptr, perm_src=perm_src,
                row_ptr_src=row_ptr_src)


@dataclasses.dataclass
class EdgeGraph:
    """Destination-sorted edges on the device (all int32 except ``perm64``)."""

    n_nodes: int
    n_edges: int
    perm: torch.Tensor          # [E] original position of sorted edge i
    src: torch.Tensor           # [E] sorted
    dst: torch.Tensor           # [E] sorted
    row_ptr: torch.Tensor       # [N+1]
    perm_src: torch.Tensor      # [E] sorted-edge ids in (src, id) order
    row_ptr_src: torch.Tensor   # [N+1]

    @property
    def perm64(self) -> torch.Tensor:
        return self.perm.long()

    def chunks(self, max_edges: int) -> list["EdgeChunk"]:
        """Splits the sorted edge list at destination-node boundaries into pieces of at most
        ``max_edges`` edges (a single node with more incoming edges than that gets a piece of
        its own).  Each piece carries its own sub-graph: the same node numbering, only its edges.
        Cached per ``max_edges``."""
        cache = self.__dict__.setdefault("_chunk_cache", {})
        if max_edges in cache:
            return cache[max_edges]
        cache.clear()                     # one entry: the chunking for the latest budget
        if self.n_edges <= max_edges:
            out = [EdgeChunk(0, self.n_edges, 0, self.n_nodes, self)]
        else:
            rp = self.row_ptr.cpu().numpy().astype(np.int64)
            out, n0, start = [], 0, 0
            while n0 < self.n_nodes:
                # furthest node boundary n1 > n0 with rp[n1] - rp[n0] <= max_edges
                n1 = int(np.searchsorted(rp, rp[n0] + max_edges, side="right")) - 1
                n1 = min(max(n1, n0 + 1), self.n_nodes)
                if n1 == self.n_nodes or rp[n1] > rp[n0]:
                    out.append((start, n1))          # `start` < n0: edge-less nodes carried along
                    start = n1
                elif out:
                    out[-1] = (out[-1][0], n1)
                    start = n1
                n0 = n1
            assert out[0][0] == 0 and out[-1][1] == self.n_nodes
            assert all(a[1] == b[0] for a, b in zip(out, out[1:]))
            pieces = []
            for n0, n1 in out:
                e0, e1 = int(rp[n0]), int(rp[n1])
                ei = torch.stack([self.src[e0:e1].long(), self.dst[e0:e1].long()])
                sub = EdgeGraph.build(ei, self.n_nodes, validate=False)
                sub.node_range = (n0, n1)            # all of its edges end in these rows
                pieces.append(EdgeChunk(e0, e1, n0, n1, sub))
            out = pieces
        cache[max_edges] = out
        return out

    @staticmethod
    def build(edge_index: torch.Tensor, n_nodes: int, validate: bool = True) -> "EdgeGraph":
        """Runs ``zp_csr_build`` on ``edge_index`` ([2, E] int64, CUDA).

        ``validate``: read back the kernel's range flag (one device synchronisation) and raise
        ``IndexError`` if a node index lies outside ``[0, n_nodes)``, as indexing with it raises in
        the reference.  Skipped while the stream is being captured into a CUDA graph (no
        synchronisation is possible there; the kernels leave such edges out either way)."""
        if not edge_index.is_cuda:
            raise RuntimeError("EdgeGraph.build needs a CUDA edge_index; there is no CPU path")
        lib = _lib.load()
        ei = edge_index.to(torch.int64).contiguous()
        e, dev = ei.shape[1], ei.device
        i32 = dict(dtype=torch.int32, device=dev)
        perm, src, dst, perm_src = (torch.empty(max(e, 1), **i32) for _ in range(4))
        row_ptr, row_ptr_src = (torch.empty(n_nodes + 1, **i32) for _ in range(2))
        nbytes = lib.zp_csr_work_bytes(e, n_nodes)
        work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_csr_build(ei.data_ptr(), e, n_nodes, perm.data_ptr(), src.data_ptr(),
                                        dst.data_ptr(), row_ptr.data_ptr(), perm_src.data_ptr(),
                                        row_ptr_src.data_ptr(), work.data_ptr(), nbytes, st),
                       "zp_csr_build")
            if validate and e and not torch.cuda.is_current_stream_capturing():
                import ctypes
                flag = ctypes.c_int(0)
                _lib.check(lib.zp_csr_status(work.data_ptr(), st, ctypes.byref(flag)), "zp_csr_status")
                if flag.value:
                    raise IndexError(f"edge_index names a node outside [0, {n_nodes})")
        return EdgeGraph(n_nodes, e, perm[:e], src[:e], dst[:e], row_ptr, perm_src[:e], row_ptr_src)


@dataclasses.dataclass
class EdgeChunk:
    """Edges ``e0:e1`` (all edges into nodes ``n0:n1``) with their own sorted sub-graph."""

    e0: int
    e1: int
    n0: int
    n1: int
    sub: EdgeGraph

    @property
    def n_edges(self) -> int:
        return self.e1 - self.e0


# --------------------------------------------------------------------------------------------
# synthetic periodic structures
# --------------------------------------------------------------------------------------------


def periodic_neighbors(pos: np.ndarray, box: float, cutoff: float,
                       max_neighbors: int | None) -> tuple[np.ndarray, np.ndarray]:
    """All directed edges (src -> dst) with |pos[dst] - pos[src] + shift| < cutoff in a cubic
    periodic box, no self-interaction at zero shift, optionally capped per destination.
    Returns (edge_index [2, E] int64, shifts [E, 3] float64), unsorted."""
    from scipy.spatial import cKDTree

    n = pos.shape[0]
    reach = int(np.ceil(cutoff / box))
    images = [(i, j, k) for i in range(-reach, reach + 1) for j in range(-reach, reach + 1)
              for k in range(-reach, reach + 1)]
    tree = cKDTree(pos)
    srcs, dsts, shs, dists = [], [], [], []
    for img in images:
        shift = np.asarray(img, np.float64) * box
        # j within the cutoff of the shifted copy pos[i] - shift  <=>  edge i -> j with vector
        # pos[j] - pos[i] + shift
        hits = cKDTree(pos - shift).sparse_distance_matrix(tree, cutoff, output_type="ndarray")
        i, j = hits["i"].astype(np.int64), hits["j"].astype(np.int64)
        d = np.linalg.norm(pos[j] - pos[i] + shift, axis=1)
        keep = d < cutoff
        if img == (0, 0, 0):
            keep &= i != j
        i, j, d = i[keep], j[keep], d[keep]
        srcs.append(i); dsts.append(j)
        shs.append(np.broadcast_to(shift, (j.size, 3))); dists.append(d)
    src = np.concatenate(srcs); dst = np.concatenate(dsts)
    sh = np.concatenate(shs); dist = np.concatenate(dists)
    if max_neighbors is not None:
        order = np.lexsort((sh[:, 2], sh[:, 1], sh[:, 0], src, dist, dst))
        dst_o = dst[order]
        start = np.searchsorted(dst_o, np.arange(n))
        rank = np.arange(dst_o.size) - start[dst_o]
        order = order[rank < max_neighbors]
        order.sort()
        src, dst, sh = src[order], dst[order], sh[order]
    return np.stack([src, dst]), sh


def neighbor_list(pos: torch.Tensor, box: float, cutoff: float,
                  max_neighbors: int | None = 30) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The neighbour list on the device (``zp_neighbors_count`` / ``zp_neighbors_fill``): all edges
    src -> dst with ``|pos[dst] - pos[src] + shift|^2 < cutoff^2`` in a cubic periodic box of edge
    ``box`` (positions need not be wrapped into it), per destination the ``max_neighbors``
    smallest by (d2, src, shift) kept.
    ``pos``: CUDA tensor [N, 3] (computed in float64).  Returns (edge_index [2, E] int64,
    shifts [E, 3] float64, row_ptr [N + 1] int32) in (dst, src, shift) order, which is already the
    destination-sorted form the kernels consume.  One host read (the edge count) in between the
    two passes."""
    if not pos.is_cuda:
        raise RuntimeError("neighbor_list needs a CUDA tensor: there is no CPU path")
    lib = _lib.load()
    p = pos.detach().to(torch.float64).contiguous()
    n = p.shape[0]
    cap = int(max_neighbors) if max_neighbors else 0
    nbytes = lib.zp_neighbors_work_bytes(n, float(box), float(cutoff))
    if nbytes == 0:
        raise _lib.ZpError(1, "zp_neighbors_work_bytes")
    dev = p.device
    work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    row_ptr = torch.empty(n + 1, dtype=torch.int32, device=dev)
    flags = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.zp_neighbors_count(p.data_ptr(), n, float(box), float(cutoff), cap,
                                          row_ptr.data_ptr(), flags.data_ptr(), work.data_ptr(),
                                          nbytes, st), "zp_neighbors_count")
        e, fl = int(row_ptr[n].item()), int(flags.item())
        if fl & 1:
            raise ValueError("neighbor_list: positions must be finite")
        if fl & 2:
            raise _lib.ZpError(7, "zp_neighbors_count (more neighbours per atom than an uncapped "
                                  "list can hold)")
        edge_index = torch.empty(2, e, dtype=torch.int64, device=dev)
        shifts = torch.empty(e, 3, dtype=torch.float64, device=dev)
        _lib.check(lib.zp_neighbors_fill(p.data_ptr(), n, float(box), float(cutoff), cap,
                                         row_ptr.data_ptr(), e, edge_index.data_ptr(),
                                         shifts.data_ptr(), flags.data_ptr(), work.data_ptr(),
                                         nbytes, st), "zp_neighbors_fill")
        if int(flags.item()):
            raise RuntimeError(f"zp_neighbors_fill: device flags {int(flags.item())}")
    return edge_index, shifts, row_ptr


def synthetic_batch(n_atoms: int, lmax: int, channels: int, cutoff: float, *,
                    density: float | None = 0.1, box: float | None = None,
                    max_neighbors: int | None = 30, n_structures: int = 1, seed: int = 0,
                    dtype=torch.float32) -> dict:
    """Seeded batch in the reference's batch-dict schema (fixtures/load.py:73-87): uniform atoms
    in a periodic cube, block-diagonal over ``n_structures`` independent structures.  All random
    draws come from one CPU generator in FP64 and are cast afterwards."""
    from .blocks.wigner import gamma_harmonics

    if box is None:
        box = float((n_atoms / density) ** (1.0 / 3.0))
    while True:
        g = torch.Generator("cpu").manual_seed(seed)
        pos_l, ei_l, sh_l = [], [], []
        for s in range(n_structures):
            p = torch.rand(n_atoms, 3, generator=g, dtype=torch.float64) * box
            ei, sh = periodic_neighbors(p.numpy(), box, cutoff, max_neighbors)
            pos_l.append(p); ei_l.append(torch.from_numpy(ei) + s * n_atoms)
            sh_l.append(torch.from_numpy(sh))
        pos, edge_index, shifts = torch.cat(pos_l), torch.cat(ei_l, dim=1), torch.cat(sh_l)
        vec = pos[edge_index[1]] - pos[edge_index[0]] + shifts
        if vec.norm(dim=1).min().item() > 1e-3:
            break
        seed += 1000                      # a zero-length edge leaves the frame undefined
    n, e = pos.shape[0], edge_index.shape[1]
    k = (lmax + 1) ** 2
    x_node = torch.randn(n, k, channels, generator=g, dtype=torch.float64)
    gamma = torch.rand(e, generator=g, dtype=torch.float64) * 2 * torch.pi
    z = torch.randint(1, 30, (n,), generator=g)
    cos_g, sin_g = gamma_harmonics(gamma, lmax)
    return {
        "pos": pos.to(dtype), "cell": torch.eye(3, dtype=dtype) * box, "atomic_numbers": z,
        "x_node": x_node.to(dtype), "edge_index": edge_index, "shifts": shifts.to(dtype),
        "cos_gamma_k": cos_g.to(dtype), "sin_gamma_k": sin_g.to(dtype),
        "e_ref": torch.zeros((), dtype=dtype), "f_ref": torch.zeros(n, 3, dtype=dtype),
        "meta": {"seed": seed, "box": box, "cutoff": cutoff, "n_atoms": n, "n_edges": e,
                 "n_structures": n_structures, "max_neighbors": max_neighbors},
    }
