"""FP64 CPU evaluator of segmented-polynomial programs.  TEST INFRASTRUCTURE ONLY.

This is the second oracle: it defines what a program built with ``zippel_b200.zippel.ir`` means,
following the reference's ``zippel/interp.py`` (``apply_scalar:56``, ``eval_op:85``, ``run:135``).
It is imported by tests only; the shipped package never evaluates programs on the CPU.
"""

from __future__ import annotations

import torch

from zippel_b200.zippel.ir import IndexType, Op, Program

DTYPE = torch.float64

_P = 5.0
_A, _B, _C = -(_P + 1) * (_P + 2) / 2, _P * (_P + 2), -_P * (_P + 1) / 2


def _envelope(d: torch.Tensor, order: int) -> torch.Tensor:
    """1 + a d^5 + b d^6 + c d^7 and its derivatives; zero at and beyond d = 1."""
    powers = {0: [(1.0, 0), (_A, 5), (_B, 6), (_C, 7)]}
    for k in range(1, 4):
        powers[k] = [(c * e, e - 1) for c, e in powers[k - 1] if e > 0]
    if order not in powers:
        raise NotImplementedError(f"poly_envelope order {order}")
    val = sum(c * d ** e for c, e in powers[order])
    return torch.where(d < 1, val, torch.zeros_like(val))


def apply_scalar(fn: str, x: torch.Tensor, order: int = 0) -> torch.Tensor:
    table = {"exp": torch.exp, "sigmoid": torch.sigmoid, "silu": torch.nn.functional.silu,
             "rsqrt": torch.rsqrt, "reciprocal": torch.reciprocal, "sin": torch.sin,
             "cos": torch.cos}
    if fn in table:
        return table[fn](x)
    if fn == "poly_envelope":
        return _envelope(x, order)
    raise ValueError(f"unknown scalar function {fn!r}")


def segment_length(seg: str, sizes: dict) -> int:
    return 1 if seg == "none" else sizes[seg]


def eval_op(op: Op, env: dict, sizes: dict) -> torch.Tensor:
    if op.kind == "scalar_map":
        return apply_scalar(op.fn, env[op.inputs[0]], op.order)
    if op.kind != "segmented_contraction":
        raise ValueError(f"unknown op kind {op.kind!r}")
    n_out = segment_length(op.out_type.segment, sizes)
    out = torch.zeros((n_out, *op.out_type.sizes), dtype=DTYPE)
    for path in op.paths:
        args = []
        for pos, k in enumerate(path.operands):
            a = env[op.inputs[k]]
            if op.index_maps[k] is not None:
                a = a[env[op.index_maps[k]]]
            sl = path.slices_for(pos)
            if sl:
                a = a[(slice(None), *sl)]
            args.append(a)
        lengths = {a.shape[0] for a in args if a.shape[0] != 1}
        if len(lengths) > 1:
            raise ValueError(f"operands disagree on the segment length: {sorted(lengths)}")
        n_c = lengths.pop() if lengths else (n_out if op.out_index_map is None else 1)
        args = [a.expand(n_c, *a.shape[1:]) if a.shape[0] == 1 and n_c != 1 else a for a in args]
        terms, result = path.parse()
        contrib = path.coeff * torch.einsum(",".join("Z" + t for t in terms) + "->Z" + result, *args)
        target = out[(slice(None), *path.out_slice)] if path.out_slice else out
        if op.out_index_map is not None:
            target.index_add_(0, env[op.out_index_map], contrib)
        else:
            target += contrib if contrib.shape[0] == target.shape[0] else contrib.expand_as(target)
    return out


def run(prog: Program, inputs: dict, sizes: dict) -> dict:
    """Evaluates every op; returns the environment {buffer name: tensor}."""
    env = {}
    for name, t in prog.inputs.items():
        if name not in inputs:
            raise KeyError(f"missing input {name!r}")
        if isinstance(t, IndexType):
            env[name] = inputs[name].to("cpu", torch.long)
            continue
        a = inputs[name].to("cpu", DTYPE)
        want = (segment_length(t.segment, sizes), *t.sizes)
        if tuple(a.shape) != want:
            raise ValueError(f"input {name!r} has shape {tuple(a.shape)}, expected {want}")
        env[name] = a
    for name in prog.topo():
        env[name] = eval_op(prog.ops[name], env, sizes)
    return env
