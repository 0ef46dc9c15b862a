"""Reverse-mode differentiation as a program-to-program transformation.

Keeps the public names of the reference's ``zippel/vjp.py`` (``vjp``, ``assert_closed``,
``ClosureError``, ``Cotangents``); the rules are those of the IR specification (the reference's
``docs/ir.md`` section 3), written here from that specification:

* contraction, operand k:  in every path that reads operand k, the cotangent takes the operand's
  place among the einsum terms and the operand's subscripts become the result's; the slice read
  from the operand and the slice written to the result trade places; a gather of the operand
  becomes a scatter-add of its cotangent, a scatter of the result becomes a gather of the
  cotangent; the coefficient stays.  A ``none``-segment operand is broadcast along a segment in
  the forward direction, so its cotangent is summed along that segment: a scatter-add through an
  all-zero index buffer (``zero_index[segment]``).
* scalar map:  ``cot * f'(x)`` with ``f'`` assembled from buffers and ops of the same vocabulary;
  ``poly_envelope`` differentiates into the next member of its own family (``order + 1``).

Nothing is evaluated.  The transformation only appends ops of the two existing kinds, so a
derived program can be differentiated again (``build_dbwd`` relies on it).
"""

from __future__ import annotations

from typing import Callable

from .ir import SCALAR_FNS, ContractionPath, IndexType, Program, default_spec, full_slice


class ClosureError(RuntimeError):
    """The program contains an op or a scalar function outside the two-op vocabulary."""


def assert_closed(prog: Program) -> None:
    """Raises ``ClosureError`` unless every op is a contraction or a known scalar map."""
    offenders = []
    for name, op in prog.ops.items():
        if op.kind == "segmented_contraction":
            continue
        if op.kind == "scalar_map" and op.fn in SCALAR_FNS:
            continue
        what = f"scalar function {op.fn!r}" if op.kind == "scalar_map" else f"op kind {op.kind!r}"
        offenders.append(f"{name} ({what})")
    if offenders:
        raise ClosureError("outside the vocabulary: " + ", ".join(offenders))


class Cotangents:
    """Collects the cotangent contributions of each buffer; ``pop`` returns their sum (one
    contraction with a unit path per contribution) or the single contribution itself."""

    def __init__(self, prog: Program):
        self.prog = prog
        self._parts: dict[str, list[str]] = {}

    def add(self, buf: str, contribution: str) -> None:
        self._parts.setdefault(buf, []).append(contribution)

    def has(self, buf: str) -> bool:
        return len(self._parts.get(buf, ())) > 0

    def pop(self, buf: str):
        parts = self._parts.pop(buf, [])
        if not parts:
            return None
        if len(parts) == 1:
            return parts[0]
        t = self.prog.type_of(parts[0])
        ident = _elementwise(t)
        return self.prog.contract(parts, t, [ident(1.0, i) for i in range(len(parts))],
                                  hint="cotsum")


def _elementwise(t) -> Callable:
    """Path factory for full-buffer elementwise terms over buffers of type ``t``:
    ``f(c, i)`` = c * operand_i,  ``f(c, i, j)`` = c * operand_i * operand_j."""
    spec, whole = default_spec(t), full_slice(t)

    def path(coeff: float, *operands: int) -> ContractionPath:
        lhs = ",".join([spec] * len(operands))
        return ContractionPath(coeff, f"{lhs}->{spec}", tuple(operands),
                               tuple(whole for _ in operands), whole)

    return path


# --------------------------------------------------------------------------------------------
# scalar maps: y = f(x); each rule returns a buffer holding cot * f'(x)
# --------------------------------------------------------------------------------------------

def _d_exp(prog, op, cot, y):                     # f' = y
    return prog.mul(cot, y, hint="g_exp")


def _d_sigmoid(prog, op, cot, y):                 # f' = y (1 - y)
    t = prog.type_of(y)
    el = _elementwise(t)
    slope = prog.contract([y], t, [el(1.0, 0), el(-1.0, 0, 0)], hint="sig_slope")
    return prog.mul(cot, slope, hint="g_sig")


def _d_silu(prog, op, cot, y):                    # f' = s (1 + x (1 - s)),  s = sigmoid(x)
    x = op.inputs[0]
    t = prog.type_of(x)
    el = _elementwise(t)
    s = prog.scalar(x, "sigmoid", hint="silu_s")
    xs = prog.mul(x, s, hint="silu_xs")
    slope = prog.contract([s, xs], t, [el(1.0, 0), el(1.0, 1), el(-1.0, 1, 0)], hint="silu_slope")
    return prog.mul(cot, slope, hint="g_silu")


def _d_rsqrt(prog, op, cot, y):                   # f' = -y / (2 x)
    x_inv = prog.scalar(op.inputs[0], "reciprocal", hint="rsqrt_xinv")
    return prog.mul(cot, prog.mul(y, x_inv, hint="rsqrt_yx"), coeff=-0.5, hint="g_rsqrt")


def _d_reciprocal(prog, op, cot, y):              # f' = -y^2
    return prog.mul(cot, prog.mul(y, y, hint="recip_sq"), coeff=-1.0, hint="g_recip")


def _d_sin(prog, op, cot, y):
    return prog.mul(cot, prog.scalar(op.inputs[0], "cos", hint="sin_cos"), hint="g_sin")


def _d_cos(prog, op, cot, y):
    return prog.mul(cot, prog.scalar(op.inputs[0], "sin", hint="cos_sin"), coeff=-1.0, hint="g_cos")


def _d_poly_envelope(prog, op, cot, y):           # next member of the family
    nxt = prog.scalar(op.inputs[0], "poly_envelope", order=op.order + 1, hint="env_next")
    return prog.mul(cot, nxt, hint="g_env")


_SCALAR_RULES: dict[str, Callable] = {
    "exp": _d_exp, "sigmoid": _d_sigmoid, "silu": _d_silu, "rsqrt": _d_rsqrt,
    "reciprocal": _d_reciprocal, "sin": _d_sin, "cos": _d_cos, "poly_envelope": _d_poly_envelope,
}


def _vjp_scalar(prog: Program, op, cot: str, y: str, ones=None) -> str:
    rule = _SCALAR_RULES.get(op.fn)
    if rule is None:
        raise ClosureError(f"scalar function {op.fn!r} has no derivative rule")
    return rule(prog, op, cot, y)


# --------------------------------------------------------------------------------------------
# contractions
# --------------------------------------------------------------------------------------------

def _transposed_path(path: ContractionPath, slot: int, cot_operand: int) -> ContractionPath:
    """The path with the term at position ``slot`` exchanged with the result."""
    terms, result = path.parse()
    slices = [path.slices_for(i) for i in range(len(path.operands))]
    read_from_operand = slices[slot]
    terms, operands = list(terms), list(path.operands)
    want = terms[slot]
    terms[slot], operands[slot], slices[slot] = result, cot_operand, tuple(path.out_slice)
    return ContractionPath(path.coeff, ",".join(terms) + "->" + want, tuple(operands),
                           tuple(slices), tuple(read_from_operand))


def _vjp_contraction(prog: Program, op, cot: str, k: int, zero_index: dict):
    """Cotangent buffer of input ``k`` of contraction ``op`` (None when no path reads it).  One
    transposed path per OCCURRENCE of the operand: a path reading it twice yields two."""
    cot_operand = len(op.inputs)                       # the cotangent is appended as a new input
    paths = [_transposed_path(p, slot, cot_operand)
             for p in op.paths for slot, which in enumerate(p.operands) if which == k]
    if not paths:
        return None
    wanted = prog.type_of(op.inputs[k])
    scatter_to = op.index_maps[k]                      # gather in the forward -> scatter-add here
    if scatter_to is None and wanted.segment == "none":
        lives_on = (prog.type_of(op.out_index_map).segment if op.out_index_map is not None
                    else op.out_type.segment)
        if lives_on != "none":                         # broadcast in the forward -> sum here
            scatter_to = zero_index[lives_on]
    return prog.contract([*op.inputs, cot], wanted, paths,
                         index_maps=[*op.index_maps, op.out_index_map],
                         out_index_map=scatter_to, hint="g")


# --------------------------------------------------------------------------------------------
# the reverse sweep
# --------------------------------------------------------------------------------------------

def vjp(prog: Program, output: str, wrt: list, seed: str, ones=None, zero_index=None) -> dict:
    """Appends to ``prog`` the ops that compute ``seed * d(output)/d(buffer)`` for every buffer in
    ``wrt`` and returns ``{buffer: cotangent buffer}`` (buffers ``output`` does not depend on are
    left out).  ``zero_index[segment]`` names an all-zero index buffer over that segment.
    Only the ops present when the call starts are differentiated; they are visited in reverse
    topological order, each after all of its consumers."""
    zero_index = dict(zero_index or {})
    pending = Cotangents(prog)
    pending.add(output, seed)
    for name in reversed(prog.topo()):
        if not pending.has(name):
            continue
        op, cot = prog.ops[name], pending.pop(name)
        if op.kind == "scalar_map":
            pending.add(op.inputs[0], _vjp_scalar(prog, op, cot, y=name, ones=ones))
        else:
            for k, operand in enumerate(op.inputs):
                if isinstance(prog.type_of(operand), IndexType):
                    continue                           # index buffers carry no gradient
                g = _vjp_contraction(prog, op, cot, k, zero_index)
                if g is not None:
                    pending.add(operand, g)
    found = {w: pending.pop(w) for w in wrt}
    assert_closed(prog)
    return {w: g for w, g in found.items() if g is not None}


__all__ = ["vjp", "assert_closed", "ClosureError", "Cotangents"]
