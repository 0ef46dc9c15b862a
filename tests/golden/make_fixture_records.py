"""Copies the records that pin the reference's benchmark fixtures out of its manifest.

    python tests/golden/make_fixture_records.py /path/to/reference

Reads ``fixtures/manifest.json`` of the reference checkout (written by its
``fixtures/make_fixtures.py``) and stores, per fixture, the fields a rebuilt fixture must
reproduce -- atom and edge counts, average degree, shortest and longest edge, and the SHA-256
over the array contents -- in ``tests/golden/reference_fixtures.json``.
"""

from __future__ import annotations

import json
import pathlib
import sys

HERE = pathlib.Path(__file__).resolve().parent
FIELDS = ("name", "element", "structure", "n_atoms", "n_edges", "avg_degree", "cutoff",
          "rattle_std", "reps", "lattice_a", "seed", "min_edge_len", "max_edge_len",
          "sha256_content")


def main(ref_root: str) -> None:
    manifest = json.loads((pathlib.Path(ref_root) / "fixtures" / "manifest.json").read_text())
    records = [{k: entry[k] for k in FIELDS} for entry in manifest["fixtures"]]
    out = {"schema_version": manifest["schema_version"], "cutoff": manifest["cutoff"],
           "fixtures": records}
    (HERE / "reference_fixtures.json").write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {len(records)} records")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
