"""Reverse-mode differentiation as a program transformation.

Public surface of the reference's ``zippel/vjp.py`` (``vjp:208``, ``assert_closed:29``,
``ClosureError:25``, ``Cotangents:48``).  Nothing is evaluated: every rule appends ops of the same
two kinds, which is the property ("closed under differentiation") the IR is built around.

Transpose of a contraction path with respect to one operand occurrence: the cotangent takes that
operand's place in the einsum, the operand's subscripts become the output subscripts, its input
slice becomes the output slice and vice versa, a gather on the operand becomes a scatter-add of
the result, and a scatter of the forward result becomes a gather of the cotangent.  The transpose
of broadcasting a ``none``-segment operand over a segment is a sum over that segment, written as
a scatter-add through an all-zero index map.
"""

from __future__ import annotations

from .ir import SCALAR_FNS, ContractionPath, IndexType, Program, default_spec, full_slice


class ClosureError(RuntimeError):
    """A derived program contains something outside the two-op vocabulary."""


def assert_closed(prog: Program) -> None:
    bad = []
    for name, op in prog.ops.items():
        if op.kind == "scalar_map":
            if op.fn not in SCALAR_FNS:
                bad.append(f"{name}: scalar function {op.fn!r}")
        elif op.kind != "segmented_contraction":
            bad.append(f"{name}: op kind {op.kind!r}")
    if bad:
        raise ClosureError("program left the vocabulary: " + "; ".join(bad))


class Cotangents:
    """Contributions to each buffer's cotangent, summed (as ONE contraction) when taken."""

    def __init__(self, prog: Program):
        self.prog = prog
        self._pending: dict = {}

    def add(self, buf: str, contribution: str) -> None:
        self._pending.setdefault(buf, []).append(contribution)

    def has(self, buf: str) -> bool:
        return bool(self._pending.get(buf))

    def pop(self, buf: str):
        parts = self._pending.pop(buf, [])
        if len(parts) <= 1:
            return parts[0] if parts else None
        t = self.prog.type_of(parts[0])
        spec, sl = default_spec(t), full_slice(t)
        paths = [ContractionPath(1.0, f"{spec}->{spec}", (i,), (sl,), sl) for i in range(len(parts))]
        return self.prog.contract(parts, t, paths, hint="acc")


def _vjp_contraction(prog: Program, op, cot: str, k: int, zero_index: dict):
    """Cotangent of input ``k`` of a contraction, or None if no path reads it."""
    hits = [(p, pos) for p in op.paths for pos, which in enumerate(p.operands) if which == k]
    if not hits:
        return None
    target = prog.type_of(op.inputs[k])
    cot_slot = len(op.inputs)
    new_paths = []
    for p, pos in hits:                      # one term per OCCURRENCE (x*x reads x twice)
        terms, result = p.parse()
        slices = [p.slices_for(i) for i in range(len(p.operands))]
        new_terms, new_ops, new_slices = list(terms), list(p.operands), list(slices)
        new_terms[pos], new_ops[pos], new_slices[pos] = result, cot_slot, tuple(p.out_slice)
        new_paths.append(ContractionPath(p.coeff, ",".join(new_terms) + "->" + terms[pos],
                                         tuple(new_ops), tuple(new_slices), tuple(slices[pos])))
    scatter = op.index_maps[k]
    if scatter is None and target.segment == "none":
        produced_on = (prog.type_of(op.out_index_map).segment if op.out_index_map is not None
                       else op.out_type.segment)
        if produced_on != "none":
            scatter = zero_index[produced_on]        # sum over the broadcast segment
    return prog.contract(list(op.inputs) + [cot], target, new_paths,
                         index_maps=list(op.index_maps) + [op.out_index_map],
                         out_index_map=scatter, hint="d")


def _vjp_scalar(prog: Program, op, cot: str, y: str, ones=None) -> str:
    """cot * f'(x), with f' written in products/sums of buffers that already exist."""
    x, fn = op.inputs[0], op.fn
    t = prog.type_of(x)
    spec, sl = default_spec(t), full_slice(t)
    one = lambda c, i: ContractionPath(c, f"{spec}->{spec}", (i,), (sl,), sl)            # noqa: E731
    two = lambda c, i, j: ContractionPath(c, f"{spec},{spec}->{spec}", (i, j), (sl, sl), sl)  # noqa: E731
    if fn == "exp":
        return prog.mul(cot, y, hint="dexp")
    if fn == "sigmoid":                                   # y - y^2
        d = prog.contract([y], t, [one(1.0, 0), two(-1.0, 0, 0)], hint="dsig")
        return prog.mul(cot, d, hint="dsg")
    if fn == "silu":                                      # s + x s - x s^2, s = sigmoid(x)
        s = prog.scalar(x, "sigmoid", hint="s")
        xs = prog.mul(x, s, hint="xs")
        d = prog.contract([s, xs], t, [one(1.0, 0), one(1.0, 1), two(-1.0, 1, 0)], hint="dsilu")
        return prog.mul(cot, d, hint="dsl")
    if fn == "rsqrt":                                     # -y / (2x)
        inv = prog.scalar(x, "reciprocal", hint="rx")
        return prog.mul(cot, prog.mul(y, inv, hint="yr"), coeff=-0.5, hint="drsq")
    if fn == "reciprocal":                                # -y^2
        return prog.mul(cot, prog.mul(y, y, hint="y2"), coeff=-1.0, hint="drec")
    if fn == "sin":
        return prog.mul(cot, prog.scalar(x, "cos", hint="cx"), hint="dsin")
    if fn == "cos":
        return prog.mul(cot, prog.scalar(x, "sin", hint="sx"), coeff=-1.0, hint="dcos")
    if fn == "poly_envelope":
        return prog.mul(cot, prog.scalar(x, "poly_envelope", order=op.order + 1, hint="denv"),
                        hint="dpe")
    raise ClosureError(f"no derivative rule for scalar function {fn!r}")


def vjp(prog: Program, output: str, wrt: list, seed: str, ones=None, zero_index=None) -> dict:
    """Appends to ``prog`` the VJP of ``output`` w.r.t. the buffers in ``wrt``, seeded by ``seed``.
    ``zero_index[segment]`` names an all-zero index buffer of that segment.  Returns
    ``{buffer: cotangent buffer}`` for the buffers the output depends on."""
    zero_index = zero_index or {}
    cots = Cotangents(prog)
    cots.add(output, seed)
    for name in reversed(prog.topo()):                    # the ops present before the transform
        if not cots.has(name):
            continue
        op, cot = prog.ops[name], cots.pop(name)
        if op.kind == "scalar_map":
            cots.add(op.inputs[0], _vjp_scalar(prog, op, cot, y=name, ones=ones))
            continue
        for k, src in enumerate(op.inputs):
            if isinstance(prog.type_of(src), IndexType):
                continue
            grad = _vjp_contraction(prog, op, cot, k, zero_index)
            if grad is not None:
                cots.add(src, grad)
    grads = {w: cots.pop(w) for w in wrt}
    assert_closed(prog)
    return {w: g for w, g in grads.items() if g is not None}


__all__ = ["vjp", "assert_closed", "ClosureError", "Cotangents"]
