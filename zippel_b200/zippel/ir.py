"""Segmented-polynomial IR: buffer types, the two ops, and a type-checked program builder.

Same public surface as the reference's ``zippel/ir.py`` (``BufferType:33``, ``IndexType:63``,
``ContractionPath:78``, ``Op:113``, ``Program:150`` with ``contract`` / ``scalar`` / ``add`` /
``mul`` / ``scale``), so programs written against the reference build here unchanged.

A program is an ordered list of single-output ops over named buffers.  A buffer is either a value
array whose leading axis is a *segment* axis (one row per node / edge / graph, or a single shared
row for ``"none"``) followed by fixed trailing axes, or an index array used to gather operands or
scatter results.  The vocabulary has exactly two ops:

``segmented_contraction``
    a sum of *paths*; each path is a coefficient times an einsum over the trailing axes of some
    of the op's inputs (optionally gathered through an index map and sliced), written into a
    slice of the result (optionally scatter-added through an index map);
``scalar_map``
    one of a small set of elementwise functions.

Everything is checked when an op is added: an ill-typed program cannot be constructed.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field

SEGMENTS = ("node", "edge", "graph", "none")
SCALAR_FNS = ("exp", "sigmoid", "silu", "rsqrt", "reciprocal", "sin", "cos", "poly_envelope")


@dataclass(frozen=True)
class BufferType:
    """Value buffer: segment axis + named trailing axes."""

    segment: str
    axes: tuple = ()
    dtype: str = "f64"

    def __post_init__(self):
        if self.segment not in SEGMENTS:
            raise ValueError(f"segment must be one of {SEGMENTS}, got {self.segment!r}")
        seen = set()
        for name, size in self.axes:
            if name in seen:
                raise ValueError(f"axis name {name!r} appears twice in {self.axes}")
            seen.add(name)
            if size <= 0:
                raise ValueError(f"axis {name!r} must have a positive size, got {size}")

    @property
    def sizes(self) -> tuple:
        return tuple(size for _, size in self.axes)

    @property
    def rank(self) -> int:
        return len(self.axes)

    def __str__(self) -> str:
        inner = ",".join(f"{n}:{s}" for n, s in self.axes)
        return f"{self.segment}[{inner}]:{self.dtype}"


@dataclass(frozen=True)
class IndexType:
    """Integer buffer (gather source / scatter target); carries no gradient."""

    segment: str

    def __str__(self) -> str:
        return f"{self.segment}[]:idx"


def _slice_key(s: slice) -> tuple:
    return (s.start, s.stop, s.step)


@dataclass(frozen=True)
class ContractionPath:
    """One multilinear term: ``coeff * einsum(subscripts, inputs[operands[0]][in_slices[0]], ...)``
    accumulated into ``out[out_slice]``.  Subscripts cover trailing axes only."""

    coeff: float
    subscripts: str
    operands: tuple
    in_slices: tuple = ()
    out_slice: tuple = ()

    def parse(self):
        if "->" not in self.subscripts:
            raise ValueError(f"subscripts need an explicit '->': {self.subscripts!r}")
        lhs, rhs = self.subscripts.split("->", 1)
        return [term.strip() for term in lhs.split(",")], rhs.strip()

    def slices_for(self, position: int) -> tuple:
        return self.in_slices[position] if self.in_slices else ()

    def key(self) -> tuple:
        return (self.coeff, self.subscripts, self.operands,
                tuple(tuple(_slice_key(s) for s in grp) for grp in self.in_slices),
                tuple(_slice_key(s) for s in self.out_slice))


@dataclass(frozen=True)
class Op:
    kind: str
    inputs: tuple
    out_type: BufferType
    index_maps: tuple = ()
    out_index_map: str | None = None
    paths: tuple = ()
    fn: str | None = None
    order: int = 0
    name: str = ""

    def key(self) -> tuple:
        """Structural identity including which buffers feed the op (used by CSE)."""
        return (self.kind, self.inputs, str(self.out_type), self.index_maps, self.out_index_map,
                tuple(p.key() for p in self.paths), self.fn, self.order)

    def signature(self) -> tuple:
        """Shape-and-structure identity, independent of buffer names and path coefficients."""
        if self.kind == "scalar_map":
            return ("scalar_map", self.fn, self.order, str(self.out_type))
        return ("segmented_contraction", str(self.out_type),
                tuple(m is not None for m in self.index_maps), self.out_index_map is not None,
                tuple(p.key()[1:] for p in self.paths))


def default_spec(t: BufferType) -> str:
    return "abcdefghijklmnopqrstuvwxy"[: t.rank]


def full_slice(t: BufferType) -> tuple:
    return (slice(None),) * t.rank


def sliced_sizes(t: BufferType, slices: tuple) -> tuple:
    out = []
    for axis, size in enumerate(t.sizes):
        if axis < len(slices):
            out.append(len(range(*slices[axis].indices(size))))
        else:
            out.append(size)
    return tuple(out)


@dataclass
class Program:
    inputs: dict = field(default_factory=dict)
    ops: dict = field(default_factory=dict)
    outputs: tuple = ()
    _counter: itertools.count = field(default_factory=itertools.count)

    # -- buffers ------------------------------------------------------------------------------
    def add_input(self, name: str, type_) -> str:
        if name in self.inputs or name in self.ops:
            raise ValueError(f"buffer {name!r} is already defined")
        self.inputs[name] = type_
        return name

    def type_of(self, name: str):
        if name in self.inputs:
            return self.inputs[name]
        if name in self.ops:
            return self.ops[name].out_type
        raise KeyError(f"no buffer named {name!r}")

    def _fresh(self, hint: str) -> str:
        return f"{hint}_{next(self._counter)}"

    # -- the two ops ----------------------------------------------------------------------------
    def contract(self, inputs, out_type, paths, index_maps=None, out_index_map=None,
                 hint="c") -> str:
        inputs = list(inputs)
        index_maps = [None] * len(inputs) if index_maps is None else list(index_maps)
        if len(index_maps) != len(inputs):
            raise ValueError("index_maps needs exactly one entry (or None) per input")
        paths = list(paths)
        _check_contraction(self, inputs, index_maps, out_index_map, out_type, paths)
        name = self._fresh(hint)
        self.ops[name] = Op("segmented_contraction", tuple(inputs), out_type, tuple(index_maps),
                            out_index_map, tuple(paths), None, 0, name)
        return name

    def scalar(self, x: str, fn: str, order: int = 0, hint: str | None = None) -> str:
        if fn not in SCALAR_FNS:
            raise ValueError(f"scalar function {fn!r} is not in the vocabulary {SCALAR_FNS}")
        if order != 0 and fn != "poly_envelope":
            raise ValueError("a derivative order is only defined for poly_envelope")
        t = self.type_of(x)
        if not isinstance(t, BufferType):
            raise TypeError(f"scalar_map needs a value buffer, {x!r} is an index buffer")
        name = self._fresh(hint or fn)
        self.ops[name] = Op("scalar_map", (x,), t, (), None, (), fn, order, name)
        return name

    # -- conveniences (each is one contraction) -------------------------------------------------
    def add(self, a: str, b: str, ca: float = 1.0, cb: float = 1.0, hint="add") -> str:
        t = self.type_of(a)
        spec, sl = default_spec(t), full_slice(t)
        return self.contract([a, b], t,
                             [ContractionPath(ca, f"{spec}->{spec}", (0,), (sl,), sl),
                              ContractionPath(cb, f"{spec}->{spec}", (1,), (sl,), sl)], hint=hint)

    def mul(self, a: str, b: str, coeff: float = 1.0, hint="mul") -> str:
        t = self.type_of(a)
        spec, sl = default_spec(t), full_slice(t)
        return self.contract([a, b], t,
                             [ContractionPath(coeff, f"{spec},{spec}->{spec}", (0, 1), (sl, sl), sl)],
                             hint=hint)

    def scale(self, a: str, coeff: float, hint="scale") -> str:
        t = self.type_of(a)
        spec, sl = default_spec(t), full_slice(t)
        return self.contract([a], t, [ContractionPath(coeff, f"{spec}->{spec}", (0,), (sl,), sl)],
                             hint=hint)

    # -- queries ----------------------------------------------------------------------------------
    def consumers(self) -> dict:
        users: dict = {}
        for name, op in self.ops.items():
            for src in op.inputs:
                users.setdefault(src, []).append(name)
        return users

    def topo(self) -> list:
        return list(self.ops)

    def __str__(self) -> str:
        rows = [f"  in  {n}: {t}" for n, t in self.inputs.items()]
        for name, op in self.ops.items():
            if op.kind == "scalar_map":
                tag = f"[order={op.order}]" if op.order else ""
                rows.append(f"  {name} = {op.fn}{tag}({op.inputs[0]})  : {op.out_type}")
            else:
                gathers = ",".join(m or "-" for m in op.index_maps)
                rows.append(f"  {name} = contract({','.join(op.inputs)}) gather[{gathers}] "
                            f"scatter[{op.out_index_map or '-'}] paths={len(op.paths)}  : {op.out_type}")
        rows.append("  out " + ", ".join(self.outputs))
        return "\n".join(rows)


# ---------------------------------------------------------------------------------------------
# validation of a contraction
# ---------------------------------------------------------------------------------------------

def _check_contraction(prog, inputs, index_maps, out_index_map, out_type, paths) -> None:
    if not paths:
        raise ValueError("a segmented_contraction needs at least one path")
    in_types = []
    for pos, (buf, imap) in enumerate(zip(inputs, index_maps)):
        t = prog.type_of(buf)
        if not isinstance(t, BufferType):
            raise TypeError(f"input {pos} ({buf!r}) is an index buffer; operands must be values")
        if imap is not None:
            if not isinstance(prog.type_of(imap), IndexType):
                raise TypeError(f"index_maps[{pos}] = {imap!r} is not an index buffer")
            if t.segment == "none":
                raise TypeError(f"{buf!r} has segment 'none' and cannot be gathered from")
        elif t.segment not in (out_type.segment, "none") and out_index_map is None:
            raise TypeError(f"input {pos} ({buf!r}) lives on segment {t.segment!r} but the result "
                            f"on {out_type.segment!r}, with neither a gather nor a scatter")
        in_types.append(t)
    if out_index_map is not None and not isinstance(prog.type_of(out_index_map), IndexType):
        raise TypeError(f"out_index_map {out_index_map!r} is not an index buffer")
    for path in paths:
        _check_path(path, in_types, out_type)


def _check_path(path: ContractionPath, in_types, out_type) -> None:
    terms, result = path.parse()
    if len(terms) != len(path.operands):
        raise ValueError(f"{path.subscripts!r} has {len(terms)} terms for "
                         f"{len(path.operands)} operands")
    if path.in_slices and len(path.in_slices) != len(path.operands):
        raise ValueError("in_slices needs one entry per operand of the path")
    for k in path.operands:
        if not 0 <= k < len(in_types):
            raise ValueError(f"path refers to input {k}; the op has {len(in_types)} inputs")

    # an index that is summed away must be shared by at least two operands: otherwise the
    # transpose of the path would have to broadcast, which no path can express
    occurrences: dict = {}
    for term in terms:
        for ch in set(term):
            occurrences[ch] = occurrences.get(ch, 0) + 1
    for ch, count in occurrences.items():
        if ch not in result and count < 2:
            raise ValueError(f"index {ch!r} of {path.subscripts!r} is summed but appears in only "
                             "one operand; its transpose is not expressible")
    for ch in result:
        if ch not in occurrences:
            raise ValueError(f"output index {ch!r} of {path.subscripts!r} is supplied by no operand")

    extent: dict = {}
    for position, (k, term) in enumerate(zip(path.operands, terms)):      # by position: an input
        shape = sliced_sizes(in_types[k], path.slices_for(position))      # may occur twice
        if len(term) != len(shape):
            raise ValueError(f"term {term!r} has rank {len(term)} but operand {k} sliced to "
                             f"{shape} ({in_types[k]})")
        for ch, size in zip(term, shape):
            if extent.setdefault(ch, size) != size:
                raise ValueError(f"index {ch!r} has extents {extent[ch]} and {size} in "
                                 f"{path.subscripts!r}")
    out_shape = sliced_sizes(out_type, path.out_slice)
    if len(result) != len(out_shape):
        raise ValueError(f"result term {result!r} has rank {len(result)} but the sliced output "
                         f"has rank {len(out_shape)} ({out_type})")
    for ch, size in zip(result, out_shape):
        if extent.get(ch, size) != size:
            raise ValueError(f"output index {ch!r} has extent {extent[ch]}, the result slot {size}")


__all__ = ["BufferType", "IndexType", "ContractionPath", "Op", "Program", "SCALAR_FNS", "SEGMENTS",
           "default_spec", "full_slice", "sliced_sizes"]
