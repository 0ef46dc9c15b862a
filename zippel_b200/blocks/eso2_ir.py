"""The eSEN SO(2) block written in the segmented-polynomial IR.

Public surface of the reference's ``blocks/eso2_ir.py``: ``build_wigner`` (``:90``),
``build_forward(cfg, gauss_coeff) -> (Program, meta)`` (``:290``) and ``build_force`` (``:579``),
with the input names that ``blocks/ir_bind.bind`` produces.  The program states the same
computation as ``ESO2Block`` / the reference's ``ESO2RefBlock.forward`` (``eso2_ref.py:317-362``)
-- position to energy -- in the two-op vocabulary, and ``build_force`` appends its VJP with respect
to the positions.  Unlike the reference's, the layout may have ``mmax < lmax``: ``to_m`` is the
rectangular ``[Km, K]`` selection and every m'-major buffer has ``Km`` rows.

The programs are *descriptions*: the FP64 interpreter (test oracle) evaluates them literally, and
``zippel_b200.codegen.compose`` recognises them and runs the hand-written kernels instead.
"""

from __future__ import annotations

from ..zippel.ir import BufferType, ContractionPath, IndexType, Program
from .eso2 import BlockConfig, Layout

S = slice(None)
P = ContractionPath


class _Builder:
    """Small vocabulary of scalar / vector helpers over one Program."""

    def __init__(self, prog: Program):
        self.p = prog

    def scalar_t(self, seg="edge"):
        return BufferType(seg, ())

    def component(self, vec: str, i: int, hint: str) -> str:
        """vec[:, i] as a rank-0 buffer, via a contraction against the static unit vector so the
        transpose is an ordinary scatter into slot i."""
        seg = self.p.type_of(vec).segment
        return self.p.contract([vec, "unit"], self.scalar_t(seg),
                               [P(1.0, "x,x->", (0, 1), ((slice(i, i + 1),), (S,)), ())], hint=hint)

    def prod(self, a: str, b: str, coeff: float = 1.0, hint="sm") -> str:
        return self.p.contract([a, b], self.p.type_of(a), [P(coeff, ",->", (0, 1), ((), ()), ())],
                               hint=hint)

    def lin(self, terms, hint="sa") -> str:
        """sum_i coeff_i * scalar_i."""
        bufs = [b for _, b in terms]
        return self.p.contract(bufs, self.p.type_of(bufs[0]),
                               [P(c, "->", (i,), ((),), ()) for i, (c, _) in enumerate(terms)],
                               hint=hint)


def _zrot(b: _Builder, cos_k, sin_k, l: int, sign: float, hint: str) -> str:
    """Z-rotation block [edge, n, n]: cos(f t) on the diagonal, sign*sgn(f)*sin(|f| t) on the
    anti-diagonal, f = l - row; the centre entry is cos(0 t) alone."""
    n = 2 * l + 1
    inputs, paths = ["unit_mat"], []

    def slot(buf):
        if buf not in inputs:
            inputs.append(buf)
        return inputs.index(buf)

    for i in range(n):
        f = l - i
        paths.append(P(1.0, ",ij->ij", (slot(cos_k[abs(f)]), 0), ((), (S, S)),
                       (slice(i, i + 1), slice(i, i + 1))))
        if f != 0:
            paths.append(P(sign if f > 0 else -sign, ",ij->ij", (slot(sin_k[abs(f)]), 0),
                           ((), (S, S)), (slice(i, i + 1), slice(n - 1 - i, n - i))))
    return b.p.contract(inputs, BufferType("edge", (("i", n), ("j", n))), paths, hint=hint)


def build_wigner(p: Program, edge_vec: str, cos_g: str, sin_g: str, lmax: int, jd: str, ones: str,
                 unit: str, unit_mat: str) -> str:
    """Block-diagonal Wigner-D [edge, K, K] from the edge vector, rsqrt the only non-polynomial
    primitive (the reference's rational construction, blocks/wigner.py:60-160)."""
    assert unit == "unit" and unit_mat == "unit_mat"
    b = _Builder(p)
    sc = b.scalar_t()
    r2 = p.contract([edge_vec, edge_vec], sc, [P(1.0, "x,x->", (0, 1), ((S,), (S,)), ())], hint="r2")
    inv_norm = p.scalar(r2, "rsqrt", hint="invnorm")
    xyz = p.contract([edge_vec, inv_norm], p.type_of(edge_vec),
                     [P(1.0, "x,->x", (0, 1), ((S,), ()), (S,))], hint="xyz")
    xh, yh, zh = (b.component(xyz, i, h) for i, h in enumerate(("xh", "yh", "zh")))
    s2 = b.lin([(1.0, b.prod(xh, xh, hint="xx")), (1.0, b.prod(zh, zh, hint="zz"))], hint="s2")
    inv_r = p.scalar(s2, "rsqrt", hint="invr")
    r = b.prod(s2, inv_r, hint="r")

    cos_b, u = [ones, yh], [ones, b.lin([(2.0, yh)], hint="u1")]
    for k in range(2, lmax + 1):
        cos_b.append(b.lin([(2.0, b.prod(yh, cos_b[k - 1])), (-1.0, cos_b[k - 2])], hint=f"T{k}"))
        u.append(b.lin([(2.0, b.prod(yh, u[k - 1])), (-1.0, u[k - 2])], hint=f"U{k}"))
    sin_b = [None] + [b.prod(r, u[k - 1], hint=f"sb{k}") for k in range(1, lmax + 1)]
    ca1, sa1 = b.prod(zh, inv_r, hint="ca1"), b.prod(xh, inv_r, hint="sa1")
    cos_a, sin_a = [ones, ca1], [None, sa1]
    for k in range(2, lmax + 1):
        cos_a.append(b.lin([(1.0, b.prod(ca1, cos_a[k - 1])), (-1.0, b.prod(sa1, sin_a[k - 1]))],
                           hint=f"ca{k}"))
        sin_a.append(b.lin([(1.0, b.prod(sa1, cos_a[k - 1])), (1.0, b.prod(ca1, sin_a[k - 1]))],
                           hint=f"sa{k}"))
    cos_gk = [b.component(cos_g, k, f"cg{k}") for k in range(lmax + 1)]
    sin_gk = [b.component(sin_g, k, f"sg{k}") for k in range(lmax + 1)]

    k_axis = (lmax + 1) ** 2
    blocks = []
    for l in range(lmax + 1):
        n, blk = 2 * l + 1, slice(l * l, (l + 1) ** 2)
        bt = BufferType("edge", (("i", n), ("j", n)))
        mm = lambda x, y, ys, h: p.contract([x, y], bt, [P(1.0, "ik,kj->ij", (0, 1), ((S, S), ys), (S, S))], hint=h)  # noqa: E731
        acc = _zrot(b, cos_gk, sin_gk, l, -1.0, f"Xa{l}")
        acc = mm(acc, jd, (blk, blk), f"aj{l}")
        acc = mm(acc, _zrot(b, cos_b, sin_b, l, -1.0, f"Xb{l}"), (S, S), f"ajb{l}")
        acc = mm(acc, jd, (blk, blk), f"ajbj{l}")
        acc = mm(acc, _zrot(b, cos_a, sin_a, l, -1.0, f"Xc{l}"), (S, S), f"D{l}")
        blocks.append((acc, blk))
    return p.contract([name for name, _ in blocks],
                      BufferType("edge", (("i", k_axis), ("j", k_axis))),
                      [P(1.0, "ij->ij", (i,), ((S, S),), (blk, blk)) for i, (_, blk) in enumerate(blocks)],
                      hint="wigner")


def linear(p: Program, x: str, w: str, bias, n_out: int, axis: str, hint="lin") -> str:
    seg = p.type_of(x).segment
    inputs, paths = [x, w], [P(1.0, "i,oi->o", (0, 1), ((S,), (S, S)), (S,))]
    if bias is not None:
        inputs.append(bias)
        paths.append(P(1.0, "o->o", (2,), ((S,),), (S,)))
    return p.contract(inputs, BufferType(seg, ((axis, n_out),)), paths, hint=hint)


def layernorm(p: Program, x: str, gamma: str, beta: str, ones_c: str, eps: float, hint="ln") -> str:
    t = p.type_of(x)
    n, sc = t.sizes[0], BufferType(t.segment, ())
    mean = p.contract([x, ones_c], sc, [P(1.0 / n, "c,c->", (0, 1), ((S,), (S,)), ())], hint="mean")
    cen = p.contract([x, mean, ones_c], t, [P(1.0, "c->c", (0,), ((S,),), (S,)),
                                            P(-1.0, ",c->c", (1, 2), ((), (S,)), (S,))], hint="cen")
    var = p.contract([cen, ones_c], sc,
                     [P(1.0 / n, "c,c->", (0, 0), ((S,), (S,)), ()),
                      P(eps / n, "c,c->", (1, 1), ((S,), (S,)), ())], hint="vareps")
    inv = p.scalar(var, "rsqrt", hint="invstd")
    return p.contract([cen, inv, gamma, beta], t, [P(1.0, "c,,c->c", (0, 1, 2), ((S,), (), (S,)), (S,)),
                                                   P(1.0, "c->c", (3,), ((S,),), (S,))], hint=hint)


def _so2_conv(p: Program, x: str, tag: str, c_in: int, c_out: int, layout: Layout, radial,
              extra_m0: int, hint: str):
    """One SO(2) convolution over the m'-major rows of ``x`` [edge, Km, c_in].  Returns the
    output [edge, Km, c_out] and the gate scalars (or None).  For m > 0,
    out_re = Wa x_re - Wb x_im and out_im = Wa x_im + Wb x_re (eso2_ref.py:282-291)."""
    km_rows = sum(layout.m_split)
    n0 = layout.m_size[0]
    x0 = x
    sl0 = (slice(0, n0), S)
    if radial is not None:
        x0 = p.contract([x, radial[0]], BufferType("edge", (("k", n0), ("c", c_in))),
                        [P(1.0, "kc,kc->kc", (0, 1), (sl0, (S, S)), (S, S))], hint=f"{hint}_mod0")
        sl0 = (S, S)
    n_flat = c_out * n0 + extra_m0
    flat = p.contract([x0, f"{tag}_w0", f"{tag}_b0"], BufferType("edge", (("o", n_flat),)),
                      [P(1.0, "mc,omc->o", (0, 1), (sl0, (S, S, S)), (S,)),
                       P(1.0, "o->o", (2,), ((S,),), (S,))], hint=f"{hint}_m0")
    gate = None
    if extra_m0:
        gate = p.contract([flat], BufferType("edge", (("o", extra_m0),)),
                          [P(1.0, "o->o", (0,), ((slice(0, extra_m0),),), (S,))], hint=f"{hint}_gate")
    inputs = [flat, "unit_m"]
    paths = [P(1.0, "c,m->mc", (0, 1),
               ((slice(extra_m0 + i * c_out, extra_m0 + (i + 1) * c_out),), (S,)),
               (slice(i, i + 1), S)) for i in range(n0)]
    row = n0
    for m in range(1, layout.mmax + 1):
        km = layout.m_size[m]
        re_rows, im_rows = slice(row, row + km), slice(row + km, row + 2 * km)
        src, re_in, im_in = x, re_rows, im_rows
        if radial is not None:
            src = p.contract([x, radial[m]], BufferType("edge", (("k", 2 * km), ("c", c_in))),
                             [P(1.0, "kc,kc->kc", (0, 1), ((re_rows, S), (S, S)), (slice(0, km), S)),
                              P(1.0, "kc,kc->kc", (0, 1), ((im_rows, S), (S, S)), (slice(km, 2 * km), S))],
                             hint=f"{hint}_mod{m}")
            re_in, im_in = slice(0, km), slice(km, 2 * km)
        i0 = len(inputs)
        inputs += [src, f"{tag}_w{m}a", f"{tag}_w{m}b"]
        w4 = (S, S, S, S)
        for coeff, x_rows, w_slot, out_rows in ((1.0, re_in, 1, re_rows), (-1.0, im_in, 2, re_rows),
                                                (1.0, im_in, 1, im_rows), (1.0, re_in, 2, im_rows)):
            paths.append(P(coeff, "kc,jokc->jo", (i0, i0 + w_slot), ((x_rows, S), w4), (out_rows, S)))
        row += 2 * km
    out = p.contract(inputs, BufferType("edge", (("m", km_rows), ("c", c_out))), paths, hint=hint)
    return out, gate


def _gate(p: Program, gate: str, x: str, layout: Layout, h: int) -> str:
    """SiLU on row 0; sigmoid(gate block l-1) on the row of degree l (eso2_ref.py:295-301)."""
    t = p.type_of(x)
    sig = p.scalar(gate, "sigmoid", hint="gsig")
    act = p.scalar(x, "silu", hint="gsilu")
    paths = [P(1.0, "mc->mc", (0,), ((slice(0, 1), S),), (slice(0, 1), S))]
    for row, (l, _m) in enumerate(layout.rows[1:], start=1):
        paths.append(P(1.0, "mc,c->mc", (1, 2), ((slice(row, row + 1), S), (slice((l - 1) * h, l * h),)),
                       (slice(row, row + 1), S)))
    return p.contract([act, x, sig], t, paths, hint="gate")


def build_forward(cfg: BlockConfig = BlockConfig(), gauss_coeff: float | None = None):
    """The block, position -> E.  Returns (program, meta); meta names the energy, the positions,
    the parameter inputs, the node output and the layout."""
    L, C, H, mmax = cfg.lmax, cfg.sphere_channels, cfg.hidden_channels, cfg.mmax
    K, EC, NB, C2 = cfg.num_coeffs, cfg.edge_channels, cfg.num_distance_basis, 2 * cfg.sphere_channels
    layout = Layout.make(L, mmax)
    m_size, Km = layout.m_size, sum(layout.m_split)
    p = Program()
    b = _Builder(p)
    vt = lambda seg, *axes: BufferType(seg, tuple(axes))                         # noqa: E731

    for name, t in (("pos", vt("node", ("x", 3))), ("x_node", vt("node", ("m", K), ("c", C))),
                    ("shifts", vt("edge", ("x", 3))), ("cos_g", vt("edge", ("k", L + 1))),
                    ("sin_g", vt("edge", ("k", L + 1))), ("emb_src", vt("edge", ("c", EC))),
                    ("emb_dst", vt("edge", ("c", EC))), ("src", IndexType("edge")),
                    ("dst", IndexType("edge")), ("zn", IndexType("node")), ("ze", IndexType("edge")),
                    ("jd", vt("none", ("i", K), ("j", K))), ("to_m", vt("none", ("m", Km), ("k", K))),
                    ("gauss_offset", vt("none", ("g", NB))), ("ones_g", vt("none", ("g", NB))),
                    ("ones", vt("edge")), ("unit", vt("none", ("x", 1))),
                    ("unit_mat", vt("none", ("i", 1), ("j", 1))), ("unit_m", vt("none", ("m", 1))),
                    ("ones_ec", vt("none", ("c", EC)))):
        p.add_input(name, t)
    params = []

    def par(name, t):
        params.append(p.add_input(name, t))

    w_in = NB + 2 * EC
    par("rad_w0", vt("none", ("o", EC), ("i", w_in))); par("rad_b0", vt("none", ("o", EC)))
    par("rad_g0", vt("none", ("c", EC))); par("rad_be0", vt("none", ("c", EC)))
    par("rad_w1", vt("none", ("o", EC), ("i", EC))); par("rad_b1", vt("none", ("o", EC)))
    par("rad_g1", vt("none", ("c", EC))); par("rad_be1", vt("none", ("c", EC)))
    for m in range(mmax + 1):
        par(f"rad_wm{m}", vt("none", ("k", m_size[m]), ("c", C2), ("h", EC)))
        par(f"rad_bm{m}", vt("none", ("k", m_size[m]), ("c", C2)))
    par("c1_w0", vt("none", ("o", H * (L + 1) + L * H), ("m", m_size[0]), ("c", C2)))
    par("c1_b0", vt("none", ("o", H * (L + 1) + L * H)))
    par("c2_w0", vt("none", ("o", C * (L + 1)), ("m", m_size[0]), ("c", H)))
    par("c2_b0", vt("none", ("o", C * (L + 1))))
    for m in range(1, mmax + 1):
        for tag, cin, cout in (("c1", C2, H), ("c2", H, C)):
            for half in "ab":
                par(f"{tag}_w{m}{half}", vt("none", ("j", m_size[m]), ("o", cout), ("k", m_size[m]), ("c", cin)))
    par("ro_w0", vt("none", ("o", C), ("i", C * (L + 1)))); par("ro_b0", vt("none", ("o", C)))
    par("ro_w1", vt("none", ("o", 1), ("i", C))); par("ro_b1", vt("none", ("o", 1)))

    # geometry
    edge_vec = p.contract(["pos", "pos", "shifts"], vt("edge", ("x", 3)),
                          [P(1.0, "x->x", (0,), ((S,),), (S,)), P(-1.0, "x->x", (1,), ((S,),), (S,)),
                           P(1.0, "x->x", (2,), ((S,),), (S,))], index_maps=["dst", "src", None],
                          hint="evec")
    r2 = p.contract([edge_vec, edge_vec], vt("edge"), [P(1.0, "x,x->", (0, 1), ((S,), (S,)), ())], hint="r2")
    dist = b.prod(r2, p.scalar(r2, "rsqrt", hint="invd"), hint="dist")

    # radial front end
    diff = p.contract([dist, "ones_g", "gauss_offset"], vt("edge", ("g", NB)),
                      [P(1.0, ",g->g", (0, 1), ((), (S,)), (S,)), P(-1.0, "g->g", (2,), ((S,),), (S,))],
                      hint="gdiff")
    coeff = -0.5 / (cfg.cutoff / (NB - 1)) ** 2 if gauss_coeff is None else gauss_coeff
    gauss = p.scalar(p.contract([diff], vt("edge", ("g", NB)),
                                [P(coeff, "g,g->g", (0, 0), ((S,), (S,)), (S,))], hint="gsq"),
                     "exp", hint="gauss")
    x_edge = p.contract([gauss, "emb_src", "emb_dst"], vt("edge", ("i", w_in)),
                        [P(1.0, "i->i", (0,), ((S,),), (slice(0, NB),)),
                         P(1.0, "i->i", (1,), ((S,),), (slice(NB, NB + EC),)),
                         P(1.0, "i->i", (2,), ((S,),), (slice(NB + EC, w_in),))], hint="xedge")
    h = linear(p, x_edge, "rad_w0", "rad_b0", EC, "c", hint="rl0")
    h = p.scalar(layernorm(p, h, "rad_g0", "rad_be0", "ones_ec", 1e-5, hint="rln0"), "silu", hint="rs0")
    h = linear(p, h, "rad_w1", "rad_b1", EC, "c", hint="rl1")
    h = p.scalar(layernorm(p, h, "rad_g1", "rad_be1", "ones_ec", 1e-5, hint="rln1"), "silu", hint="rs1")
    radial = {m: p.contract([h, f"rad_wm{m}", f"rad_bm{m}"], vt("edge", ("k", m_size[m]), ("c", C2)),
                            [P(1.0, "h,kch->kc", (0, 1), ((S,), (S, S, S)), (S, S)),
                             P(1.0, "kc->kc", (2,), ((S, S),), (S, S))], hint=f"radm{m}")
              for m in range(mmax + 1)}

    # rotation into the edge frame fused with the l-major -> m'-major selection
    wig = build_wigner(p, edge_vec, "cos_g", "sin_g", L, "jd", "ones", "unit", "unit_mat")
    rot = p.contract(["to_m", wig], vt("edge", ("m", Km), ("j", K)),
                     [P(1.0, "mk,kj->mj", (0, 1), ((S, S), (S, S)), (S, S))], hint="rot")
    gathered = p.contract(["x_node", "x_node"], vt("edge", ("m", K), ("c", C2)),
                          [P(1.0, "mc->mc", (0,), ((S, S),), (S, slice(0, C))),
                           P(1.0, "mc->mc", (1,), ((S, S),), (S, slice(C, C2)))],
                          index_maps=["src", "dst"], hint="cat")
    msg = p.contract([rot, gathered], vt("edge", ("m", Km), ("c", C2)),
                     [P(1.0, "mj,jc->mc", (0, 1), ((S, S), (S, S)), (S, S))], hint="rotin")

    conv1, gate = _so2_conv(p, msg, "c1", C2, H, layout, radial, L * H, "conv1")
    gated = _gate(p, gate, conv1, layout, H)
    conv2, _ = _so2_conv(p, gated, "c2", H, C, layout, None, 0, "conv2")

    env = p.scalar(p.contract([dist], vt("edge"), [P(1.0 / cfg.cutoff, "->", (0,), ((),), ())], hint="dsc"),
                   "poly_envelope", hint="env")
    damped = p.contract([conv2, env], vt("edge", ("m", Km), ("c", C)),
                        [P(1.0, "mc,->mc", (0, 1), ((S, S), ()), (S, S))], hint="damp")
    back = p.contract([rot, damped], vt("edge", ("m", K), ("c", C)),
                      [P(1.0, "jm,jc->mc", (0, 1), ((S, S), (S, S)), (S, S))], hint="rotback")
    node_out = p.contract([back], vt("node", ("m", K), ("c", C)),
                          [P(1.0, "mc->mc", (0,), ((S, S),), (S, S))], out_index_map="dst", hint="scatter")

    # rotation-invariant readout
    inv_paths = [P(1.0, "mi,m->i", (0, 1), ((slice(0, 1), S), (S,)), (slice(0, C),))]
    for l in range(1, L + 1):
        blk = slice(l * l, (l + 1) ** 2)
        inv_paths.append(P(1.0, "mi,mi->i", (0, 0), ((blk, S), (blk, S)), (slice(l * C, (l + 1) * C),)))
    invar = p.contract([node_out, "unit_m"], vt("node", ("i", C * (L + 1))), inv_paths, hint="invar")
    r = p.scalar(linear(p, invar, "ro_w0", "ro_b0", C, "c", hint="rol0"), "silu", hint="rosl")
    r = linear(p, r, "ro_w1", "ro_b1", 1, "c", hint="rol1")
    energy = p.contract([r, "unit_m"], vt("graph"), [P(1.0, "c,c->", (0, 1), ((S,), (S,)), ())],
                        out_index_map="zn", hint="E")
    p.outputs = (energy,)
    return p, {"energy": energy, "pos": "pos", "params": params, "cfg": cfg, "layout": layout,
               "node_out": node_out, "kind": "forward"}


def build_force(cfg: BlockConfig = BlockConfig(), gauss_coeff=None):
    """Forward plus the VJP slice that yields F = -dE/dpos."""
    from ..zippel.vjp import vjp

    p, meta = build_forward(cfg, gauss_coeff)
    seed = p.add_input("seed_E", BufferType("graph", ()))
    grads = vjp(p, meta["energy"], ["pos"], seed=seed, zero_index={"node": "zn", "edge": "ze"})
    force = p.scale(grads["pos"], -1.0, hint="F")
    p.outputs = (meta["energy"], force)
    meta |= {"force": force, "seed_E": seed, "dE_dpos": grads["pos"], "kind": "force"}
    return p, meta


def build_dbwd(cfg: BlockConfig = BlockConfig(), gauss_coeff=None, w_e: float = 1.0,
               w_f: float = 1.0):
    """The conservative training step as one program (reference ``blocks/eso2_ir.py:593-636`` for
    ``conservative_training_step``, ``blocks/eso2_ref.py:365-385``): energy, force F = -dE/dpos,
    loss L = w_e (E - e_ref)^2 + w_f mean((F - f_ref)^2), and dL/d(parameters, pos, x_node).

    The second ``vjp`` runs over a program that already contains the force ops, so it
    differentiates through them: a genuine double backward, not two first-order passes.
    Extra inputs: ``e_ref`` [graph], ``f_ref`` [node, 3], ``inv_nf`` = 1 / (3 N) as a rank-0
    constant (N is a run-time size and cannot sit in a path coefficient), ``seed_L`` [graph].
    """
    from ..zippel.vjp import vjp

    p, meta = build_force(cfg, gauss_coeff)
    graph_t, vec_t = BufferType("graph", ()), BufferType("node", (("x", 3),))
    p.add_input("e_ref", graph_t)
    p.add_input("f_ref", vec_t)
    p.add_input("inv_nf", BufferType("none", ()))
    b = _Builder(p)

    err_e = b.lin([(1.0, meta["energy"]), (-1.0, "e_ref")], hint="dE")
    term_e = b.prod(err_e, err_e, coeff=w_e, hint="Eterm")         # one graph: the mean is the square
    err_f = p.contract([meta["force"], "f_ref"], vec_t,
                       [P(1.0, "x->x", (0,), ((S,),), (S,)), P(-1.0, "x->x", (1,), ((S,),), (S,))],
                       hint="dF")
    term_f = p.contract([err_f, err_f, "inv_nf"], graph_t,
                        [P(w_f, "x,x,->", (0, 1, 2), ((S,), (S,), ()), ())], out_index_map="zn",
                        hint="Fterm")
    loss = b.lin([(1.0, term_e), (1.0, term_f)], hint="loss")

    seed = p.add_input("seed_L", graph_t)
    wrt = [*meta["params"], "pos", "x_node"]
    grads = vjp(p, loss, wrt, seed=seed, zero_index={"node": "zn", "edge": "ze"})
    p.outputs = (loss, *grads.values())
    meta |= {"loss": loss, "seed_L": seed, "grads": grads, "kind": "dbwd"}
    return p, meta


__all__ = ["build_wigner", "build_forward", "build_force", "build_dbwd", "linear", "layernorm"]
