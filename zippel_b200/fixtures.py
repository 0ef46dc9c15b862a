"""Reader, writer and generator for the reference project's benchmark fixtures (schema v1).

The reference stores six perturbed bulk crystals (Si diamond, Cu fcc; small / medium / large) as
``.npz`` files written by ``fixtures/make_fixtures.py:142-163`` and read by
``fixtures/load.py:25-38, 52-87``; their content hashes are pinned in ``fixtures/manifest.json``.
The files themselves are not shipped and the packages that wrote them (an atomistic-structure
library and a neighbour-list library) are optional, so this module rebuilds them from the
recorded recipe with the library's own neighbour list:

* structure: conventional cubic cell (8 diamond / 4 fcc sites), replicated ``reps`` times per
  axis with the cell index varying slowest along x, Gaussian displacement of std 0.05 A from
  ``numpy.random.default_rng(seed)`` (make_fixtures.py:60-66);
* edges: every directed pair within 6 A including periodic images, no cap (:69-92), listed in
  (src, dst, shift) order (:95-100); shifts are cartesian;
* file: arrays ``pos, cell, atomic_numbers, edge_index, shifts`` plus ``schema_version`` and a
  JSON ``meta`` string; ``sha256_content`` hashes key, dtype, shape and bytes of the five arrays
  in that order (:103-112).

``build_fixture`` reproduces the manifest's ``sha256_content`` bit for bit (checked by the
tests for all six), which pins the neighbour-list rule, the order and the schema to the
reference's own records.
"""

from __future__ import annotations

import hashlib
import json
import pathlib

import numpy as np
import torch

SCHEMA_VERSION = 1
CUTOFF = 6.0
RATTLE = 0.05
CONTENT_KEYS = ("pos", "cell", "atomic_numbers", "edge_index", "shifts")

#: name -> (element, atomic number, structure, lattice constant, repeats); make_fixtures.py:44-51
SPECS = {
    "si_small": ("Si", 14, "diamond", 5.431, 3),
    "si_medium": ("Si", 14, "diamond", 5.431, 9),
    "si_large": ("Si", 14, "diamond", 5.431, 18),
    "cu_small": ("Cu", 29, "fcc", 3.615, 4),
    "cu_medium": ("Cu", 29, "fcc", 3.615, 11),
    "cu_large": ("Cu", 29, "fcc", 3.615, 23),
}

_FCC = [(0, 0, 0), (0, 0.5, 0.5), (0.5, 0, 0.5), (0.5, 0.5, 0)]
_SITES = {
    "fcc": _FCC,
    # each fcc site followed by its partner displaced by (1/4, 1/4, 1/4)
    "diamond": [q for p in _FCC for q in (p, tuple(c + 0.25 for c in p))],
}


def bulk_supercell(structure: str, a: float, reps: int, seed: int,
                   rattle: float = RATTLE) -> tuple[np.ndarray, np.ndarray]:
    """Positions [N, 3] and cell [3, 3] (float64) of the rattled cubic supercell."""
    cell1 = np.diag([a, a, a]).astype(np.float64)
    base = np.dot(np.asarray(_SITES[structure], np.float64), cell1)
    blocks = [base + np.dot((m0, m1, m2), cell1)
              for m0 in range(reps) for m1 in range(reps) for m2 in range(reps)]
    pos = np.concatenate(blocks)
    pos = pos + np.random.default_rng(seed).normal(0.0, rattle, pos.shape)
    return pos, cell1 * reps


def canonical_order(edge_index: np.ndarray, shifts: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Edges in the fixtures' (src, dst, shift_x, shift_y, shift_z) order."""
    order = np.lexsort((shifts[:, 2], shifts[:, 1], shifts[:, 0], edge_index[1], edge_index[0]))
    return np.ascontiguousarray(edge_index[:, order]), np.ascontiguousarray(shifts[order])


def content_hash(arrays: dict) -> str:
    h = hashlib.sha256()
    for key in CONTENT_KEYS:
        a = np.ascontiguousarray(arrays[key])
        h.update(key.encode())
        h.update(str(a.dtype).encode())
        h.update(str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


def build_fixture(name: str, device: str | torch.device = "cuda", seed: int = 0) -> tuple[dict, dict]:
    """Arrays and meta of one of the six reference fixtures.  ``device`` selects who builds the
    neighbour list: a CUDA device runs ``graph.neighbor_list`` (the library's kernel), "cpu" the
    host k-d tree generator ``graph.periodic_neighbors``."""
    from . import graph

    element, z, structure, a, reps = SPECS[name]
    pos, cell = bulk_supercell(structure, a, reps, seed)
    box = a * reps
    if torch.device(device).type == "cuda":
        ei, sh, _ = graph.neighbor_list(torch.from_numpy(pos).to(device), box, CUTOFF, None)
        ei, sh = ei.cpu().numpy(), sh.cpu().numpy()
        backend = "zippel_b200.neighbor_list"
    else:
        ei, sh = graph.periodic_neighbors(pos, box, CUTOFF, None)
        backend = "zippel_b200.periodic_neighbors"
    ei, sh = canonical_order(ei.astype(np.int64), sh.astype(np.float64))
    n, e = pos.shape[0], ei.shape[1]
    dist = np.linalg.norm(pos[ei[1]] - pos[ei[0]] + sh, axis=1)
    if not dist.min() > 1e-6:
        raise ValueError("zero-length edge in neighbour list")
    arrays = {
        "pos": np.ascontiguousarray(pos, np.float64),
        "cell": cell,
        "atomic_numbers": np.full(n, z, np.int64),
        "edge_index": ei,
        "shifts": sh,
    }
    meta = {
        "schema_version": SCHEMA_VERSION, "name": name, "element": element,
        "structure": structure, "n_atoms": int(n), "n_edges": int(e),
        "avg_degree": round(e / n, 4), "cutoff": CUTOFF, "rattle_std": RATTLE, "reps": reps,
        "lattice_a": a, "seed": seed, "backend": backend,
        "min_edge_len": float(dist.min()), "max_edge_len": float(dist.max()),
    }
    meta["sha256_content"] = content_hash(arrays)
    return arrays, meta


def write_fixture(path, arrays: dict, meta: dict) -> None:
    """Writes schema v1 (make_fixtures.py:158-161)."""
    np.savez_compressed(pathlib.Path(path), schema_version=np.array(SCHEMA_VERSION),
                        meta=json.dumps(meta), **{k: arrays[k] for k in CONTENT_KEYS})


def read_fixture(path) -> tuple[dict, dict]:
    """Reads schema v1; another version is rejected (load.py:31-37).  The stored content hash,
    when present, must match the arrays."""
    path = pathlib.Path(path)
    if not path.exists():
        raise FileNotFoundError(f"{path} missing")
    raw = np.load(path, allow_pickle=False)
    version = int(raw["schema_version"])
    if version != SCHEMA_VERSION:
        raise ValueError(f"{path} is schema v{version}, this reader expects v{SCHEMA_VERSION}")
    meta = json.loads(str(raw["meta"]))
    arrays = {k: raw[k] for k in CONTENT_KEYS}
    want = meta.get("sha256_content")
    if want is not None and content_hash(arrays) != want:
        raise ValueError(f"{path}: content hash does not match its meta record")
    return arrays, meta


def load_batch(source, device, dtype=torch.float32, cfg=None, requires_grad: bool = True) -> dict:
    """The batch dict of ``fixtures/load.py:52-87`` from a fixture file (path) or from
    ``(arrays, meta)``: geometry from the fixture; ``x_node`` and the roll angles regenerated on
    the CPU from ``seed + 1`` in float64, so every implementation sees the same inputs."""
    from .blocks.eso2 import BlockConfig
    from .blocks.wigner import gamma_harmonics

    cfg = cfg or BlockConfig()
    arrays, meta = read_fixture(source) if isinstance(source, (str, pathlib.Path)) else source
    pos = torch.as_tensor(arrays["pos"], device=device, dtype=dtype)
    edge_index = torch.as_tensor(arrays["edge_index"], device=device)
    n, e = pos.shape[0], edge_index.shape[1]
    g = torch.Generator(device="cpu").manual_seed(int(meta["seed"]) + 1)
    k = (cfg.lmax + 1) ** 2
    x_node = torch.randn(n, k, cfg.sphere_channels, generator=g, dtype=torch.float64)
    gamma = torch.rand(e, generator=g, dtype=torch.float64) * 2 * np.pi
    cos_g, sin_g = gamma_harmonics(gamma.to(device=device, dtype=dtype), cfg.lmax)
    return {
        "pos": pos.clone().requires_grad_(requires_grad),
        "cell": torch.as_tensor(arrays["cell"], device=device, dtype=dtype),
        "atomic_numbers": torch.as_tensor(arrays["atomic_numbers"], device=device),
        "x_node": x_node.to(device=device, dtype=dtype),
        "edge_index": edge_index,
        "shifts": torch.as_tensor(arrays["shifts"], device=device, dtype=dtype),
        "cos_gamma_k": cos_g, "sin_gamma_k": sin_g,
        "e_ref": torch.zeros((), device=device, dtype=dtype),
        "f_ref": torch.zeros(n, 3, device=device, dtype=dtype),
        "meta": meta,
    }
