"""Exact program clean-up: common-subexpression elimination and dead-code elimination.

Public surface of the reference's ``zippel/simplify.py`` that stays meaningful here (``cse:28``,
``dce:51``, ``simplify:73``, ``op_stats``-style counting).  Both rewrites are exact: they only
merge ops with identical structure and identical inputs, or drop ops nothing depends on, so an
evaluator returns bit-identical outputs.  The reference's ``fusion_groups`` partitioner is not
provided: the kernels here are hand-fused, there is nothing to partition.
"""

from __future__ import annotations

from .ir import Op, Program


def _renamed(op: Op, alias: dict, name: str) -> Op:
    r = lambda b: alias.get(b, b) if b is not None else None      # noqa: E731
    return Op(op.kind, tuple(r(b) for b in op.inputs), op.out_type,
              tuple(r(m) for m in op.index_maps), r(op.out_index_map), op.paths, op.fn, op.order,
              name)


def cse(prog: Program) -> Program:
    """Merges ops whose kind, attributes and (already merged) inputs coincide."""
    out = Program(inputs=dict(prog.inputs))
    alias: dict = {}
    seen: dict = {}
    for name, op in prog.ops.items():
        new = _renamed(op, alias, name)
        key = new.key()
        if key in seen:
            alias[name] = seen[key]
        else:
            seen[key] = name
            out.ops[name] = new
    out.outputs = tuple(alias.get(o, o) for o in prog.outputs)
    return out


def dce(prog: Program) -> Program:
    """Drops every op the outputs do not depend on."""
    live = set(prog.outputs)
    for name in reversed(prog.topo()):
        if name in live:
            op = prog.ops[name]
            live.update(op.inputs)
            live.update(m for m in (*op.index_maps, op.out_index_map) if m)
    out = Program(inputs=dict(prog.inputs), outputs=prog.outputs)
    out.ops = {n: op for n, op in prog.ops.items() if n in live}
    return out


def simplify(prog: Program) -> Program:
    """CSE then DCE, repeated until the op count stops changing."""
    count = None
    while count != len(prog.ops):
        count = len(prog.ops)
        prog = dce(cse(prog))
    return prog


def op_stats(prog: Program) -> dict:
    contractions = [op for op in prog.ops.values() if op.kind == "segmented_contraction"]
    return {"ops": len(prog.ops), "contractions": len(contractions),
            "scalar_maps": len(prog.ops) - len(contractions),
            "paths": sum(len(op.paths) for op in contractions),
            "signatures": len({op.signature() for op in prog.ops.values()})}


__all__ = ["cse", "dce", "simplify", "op_stats"]
