"""CPU oracle for the eSEN SO(2) edge-convolution block.  TEST INFRASTRUCTURE ONLY.

This file is the checker, never the product: only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import it.  Nothing under the shipped package does.

It restates, in plain functional torch (any dtype, CPU), the algorithm of the reference's
``blocks/eso2_ref.py`` and ``blocks/wigner.py``:

* layout tables            -- ``blocks/eso2_ref.py:98-146`` (``Layout.make``, ``to_m``,
                              ``gate_expand_index``), extended to ``mmax < lmax`` with a
                              rectangular ``[Km, K]`` selection (the reference's square
                              matrix cannot be multiplied with a full Wigner there;
                              identical to the reference's matrix when ``mmax == lmax``)
* rational Wigner-D        -- ``blocks/wigner.py:60-160``
* radial front end         -- ``blocks/eso2_ref.py:164-182, 248-250, 323-327``
* SO(2) convolution        -- ``blocks/eso2_ref.py:252-293``
* gate activation          -- ``blocks/eso2_ref.py:295-301``
* envelope                 -- ``blocks/eso2_ref.py:242-246``
* block forward            -- ``blocks/eso2_ref.py:317-349`` (``node_out``) and ``:351-362`` (E)

Parity pin: ``tests/golden/*.npz`` hold inputs, parameters and outputs produced by importing
the unmodified reference (``tests/golden/make_golden.py``) at ``mmax == lmax``; the
``mmax < lmax`` extension has no reference output to pin against and is checked through the
reference's own property tests (gamma independence, rotation invariance).

Parameters are passed as a ``dict[str, Tensor]`` keyed exactly like the reference module's
``state_dict()`` (``elem_emb.weight``, ``rad_func.0.weight`` ... ``c1_m0.weight``,
``c1_m.0.weight`` ... ``readout.2.bias``), so a reference ``state_dict`` drops straight in.
"""

from __future__ import annotations

import math

import torch

# ----------------------------------------------------------------------------------------
# layout tables
# ----------------------------------------------------------------------------------------


def m_sizes(lmax: int, mmax: int) -> tuple[int, ...]:
    """Number of degrees l that carry order m, for m = 0..mmax (eso2_ref.py:106-110)."""
    return tuple(lmax + 1 - m for m in range(mmax + 1))


def m_splits(lmax: int, mmax: int) -> tuple[int, ...]:
    ms = m_sizes(lmax, mmax)
    return (ms[0],) + tuple(2 * s for s in ms[1:])


def mprime_rows(lmax: int, mmax: int) -> list[tuple[int, int]]:
    """(l, signed m) of every m'-major row: m = 0 rows, then per |m| the +m then the -m rows."""
    rows = [(l, 0) for l in range(lmax + 1)]
    for m in range(1, mmax + 1):
        rows += [(l, m) for l in range(m, lmax + 1)]
        rows += [(l, -m) for l in range(m, lmax + 1)]
    return rows


def to_m_matrix(lmax: int, mmax: int, dtype=torch.float64) -> torch.Tensor:
    """0/1 selection [Km, K] from the full l-major basis (l, m=-l..l) to m'-major rows."""
    rows = mprime_rows(lmax, mmax)
    k = (lmax + 1) ** 2
    mat = torch.zeros(len(rows), k, dtype=dtype)
    for r, (l, m) in enumerate(rows):
        mat[r, l * l + l + m] = 1.0
    return mat


def gate_expand_index(lmax: int, mmax: int) -> torch.Tensor:
    """Which of the lmax gate scalars multiplies each m' row 1.. (entry = l - 1)."""
    return torch.tensor([l - 1 for (l, _m) in mprime_rows(lmax, mmax)[1:]], dtype=torch.long)


# ----------------------------------------------------------------------------------------
# Wigner-D in rational form
# ----------------------------------------------------------------------------------------

S2_FLOOR = 1e-12  # wigner.py:57


def _zrot(cos_k, sin_k, l: int, sign: float) -> torch.Tensor:
    """Z-rotation in the real basis: frequencies l..-l down the rows, cos on the diagonal,
    signed sin on the anti-diagonal; the centre element is cos(0) = 1 (wigner.py:89-112)."""
    n = 2 * l + 1
    ref = cos_k[0]
    mat = ref.new_zeros(ref.shape + (n, n))
    for i in range(n):
        f = l - i
        if f != 0:
            mat[..., i, n - 1 - i] = (sign if f > 0 else -sign) * sin_k[abs(f)]
        mat[..., i, i] = cos_k[abs(f)]
    return mat


def edge_frame_harmonics(edge_vec: torch.Tensor, lmax: int):
    """cos/sin of k*beta and k*alpha, k = 0..lmax, from the edge vector (wigner.py:60-70,
    131-143).  rsqrt is the only non-polynomial primitive."""
    inv_norm = torch.rsqrt(edge_vec.pow(2).sum(-1, keepdim=True).clamp_min(S2_FLOOR))
    xh, yh, zh = (edge_vec * inv_norm).unbind(-1)
    s2 = (xh * xh + zh * zh).clamp_min(S2_FLOOR)
    inv_r = torch.rsqrt(s2)
    r = s2 * inv_r
    one, zero = torch.ones_like(yh), torch.zeros_like(yh)
    cos_b, u = [one, yh], [one, 2.0 * yh]
    for k in range(2, lmax + 1):
        cos_b.append(2.0 * yh * cos_b[k - 1] - cos_b[k - 2])
        u.append(2.0 * yh * u[k - 1] - u[k - 2])
    sin_b = [zero] + [r * u[k - 1] for k in range(1, lmax + 1)]
    ca1, sa1 = zh * inv_r, xh * inv_r
    cos_a, sin_a = [one, ca1], [zero, sa1]
    for k in range(2, lmax + 1):
        cos_a.append(ca1 * cos_a[k - 1] - sa1 * sin_a[k - 1])
        sin_a.append(sa1 * cos_a[k - 1] + ca1 * sin_a[k - 1])
    return (cos_b[: lmax + 1], sin_b[: lmax + 1]), (cos_a[: lmax + 1], sin_a[: lmax + 1])


def wigner_blocks(edge_vec, cos_gamma_k, sin_gamma_k, lmax: int, jd) -> list[torch.Tensor]:
    """Per-degree blocks D_l = Xa(-gamma) J Xb(-beta) J Xc(-alpha), each [E, 2l+1, 2l+1]."""
    (cb, sb), (ca, sa) = edge_frame_harmonics(edge_vec, lmax)
    cg = [cos_gamma_k[:, k] for k in range(lmax + 1)]
    sg = [sin_gamma_k[:, k] for k in range(lmax + 1)]
    out = []
    for l in range(lmax + 1):
        j = jd[l].to(dtype=edge_vec.dtype, device=edge_vec.device)
        out.append(_zrot(cg, sg, l, -1.0) @ j @ _zrot(cb, sb, l, -1.0) @ j @ _zrot(ca, sa, l, -1.0))
    return out


def wigner_full(edge_vec, cos_gamma_k, sin_gamma_k, lmax: int, jd) -> torch.Tensor:
    """Block-diagonal [E, K, K] (wigner.py:115-160)."""
    k = (lmax + 1) ** 2
    w = edge_vec.new_zeros(edge_vec.shape[0], k, k)
    for l, blk in enumerate(wigner_blocks(edge_vec, cos_gamma_k, sin_gamma_k, lmax, jd)):
        w[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = blk
    return w


def edge_rotation(edge_vec, cos_gamma_k, sin_gamma_k, lmax: int, mmax: int, jd) -> torch.Tensor:
    """rot [E, Km, K] = to_m @ wigner (eso2_ref.py:329-331)."""
    w = wigner_full(edge_vec, cos_gamma_k, sin_gamma_k, lmax, jd)
    return torch.einsum("mk,ekj->emj", to_m_matrix(lmax, mmax, w.dtype), w)


def gamma_harmonics(gamma: torch.Tensor, lmax: int):
    """cos(k gamma), sin(k gamma), k = 0..lmax, [E, lmax+1] each (wigner.py:203-213)."""
    kg = gamma[:, None] * torch.arange(lmax + 1, dtype=gamma.dtype)[None, :]
    return torch.cos(kg), torch.sin(kg)


def wigner_from_angles(alpha, beta, gamma, lmax: int, jd) -> torch.Tensor:
    """D(R) from explicit ZYZ angles -- property tests only (wigner.py:163-200)."""
    k = (lmax + 1) ** 2
    out = alpha.new_zeros(alpha.shape[0], k, k)
    trig = []
    for ang in (alpha, beta, gamma):
        c, s = gamma_harmonics(ang, lmax)
        trig.append(([c[:, i] for i in range(lmax + 1)], [s[:, i] for i in range(lmax + 1)]))
    for l in range(lmax + 1):
        j = jd[l].to(dtype=alpha.dtype)
        blk = _zrot(*trig[0], l, 1.0) @ j @ _zrot(*trig[1], l, 1.0) @ j @ _zrot(*trig[2], l, 1.0)
        out[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = blk
    return out


# ----------------------------------------------------------------------------------------
# radial front end, envelope
# ----------------------------------------------------------------------------------------


def gauss_offsets(cutoff: float, nb: int) -> torch.Tensor:
    """fp32 linspace, as the reference builds it (eso2_ref.py:165)."""
    return torch.linspace(0.0, cutoff, nb)


def gauss_coeff(cutoff: float, nb: int) -> float:
    off = gauss_offsets(cutoff, nb)
    return -0.5 / (off[1] - off[0]).item() ** 2


def radial_mlp(params: dict, x_edge: torch.Tensor) -> torch.Tensor:
    """Linear-LN-SiLU, Linear-LN-SiLU, Linear (eso2_ref.py:169-182)."""
    f = torch.nn.functional
    h = x_edge
    for lin, ln in ((0, 1), (3, 4)):
        h = f.linear(h, params[f"rad_func.{lin}.weight"], params[f"rad_func.{lin}.bias"])
        h = f.layer_norm(h, h.shape[-1:], params[f"rad_func.{ln}.weight"],
                         params[f"rad_func.{ln}.bias"], 1e-5)
        h = f.silu(h)
    return f.linear(h, params["rad_func.6.weight"], params["rad_func.6.bias"])


def radial_features(params, dist, z_src, z_dst, cutoff: float, nb: int) -> torch.Tensor:
    off = gauss_offsets(cutoff, nb).to(dist.dtype)
    d = dist[:, None] - off[None, :]
    gauss = torch.exp(gauss_coeff(cutoff, nb) * d * d)
    emb = params["elem_emb.weight"]
    return radial_mlp(params, torch.cat([gauss, emb[z_src], emb[z_dst]], dim=-1))


def envelope(d_scaled: torch.Tensor, p: float = 5.0) -> torch.Tensor:
    """Polynomial cutoff, zero at and beyond d_scaled = 1 (eso2_ref.py:242-246)."""
    a, b, c = -(p + 1) * (p + 2) / 2, p * (p + 2), -p * (p + 1) / 2
    val = 1 + d_scaled ** p * (a + d_scaled * (b + c * d_scaled))
    return torch.where(d_scaled < 1, val, torch.zeros_like(val))


# ----------------------------------------------------------------------------------------
# SO(2) convolution and gate
# ----------------------------------------------------------------------------------------


def so2_conv(x, w0, b0, wm: list, lmax: int, mmax: int, c_out: int, radial, n_gate: int):
    """Per-m linear mixing in m'-major order (eso2_ref.py:252-293).

    ``x`` [E, Km, Cin]; ``w0`` [out0, m_size0*Cin] with bias; ``wm[m-1]`` [2*km*c_out, km*Cin].
    ``radial`` [E, sum_m km*Cin] scales the inputs (same gain for the +m and -m rows).
    Returns (y [E, Km, c_out], gate [E, n_gate] | None).
    """
    e, cin = x.shape[0], x.shape[2]
    ms, split = m_sizes(lmax, mmax), m_splits(lmax, mmax)
    by_m = x.split(split, dim=1)
    rad_m = radial.split([k * cin for k in ms], dim=1) if radial is not None else None

    x0 = by_m[0].reshape(e, -1)
    if rad_m is not None:
        x0 = x0 * rad_m[0]
    y0 = torch.nn.functional.linear(x0, w0, b0)
    gate = None
    if n_gate:
        gate, y0 = y0[:, :n_gate], y0[:, n_gate:]
    out = [y0.reshape(e, -1, c_out)]
    for m in range(1, mmax + 1):
        xm = by_m[m].reshape(e, 2, -1)
        if rad_m is not None:
            xm = xm * rad_m[m][:, None, :]
        ym = torch.nn.functional.linear(xm, wm[m - 1])          # [E, 2, 2*km*c_out]
        half = ym.shape[-1] // 2
        wa_re, wb_re = ym[:, 0, :half], ym[:, 0, half:]
        wa_im, wb_im = ym[:, 1, :half], ym[:, 1, half:]
        out.append((wa_re - wb_im).reshape(e, -1, c_out))
        out.append((wa_im + wb_re).reshape(e, -1, c_out))
    return torch.cat(out, dim=1), gate


def gate_activation(gate, x, lmax: int, mmax: int):
    """SiLU on row 0, sigmoid(gate[l-1]) on the others (eso2_ref.py:295-301)."""
    e, h = x.shape[0], x.shape[2]
    g = torch.sigmoid(gate).reshape(e, lmax, h)[:, gate_expand_index(lmax, mmax)]
    return torch.cat([torch.nn.functional.silu(x[:, :1]), x[:, 1:] * g], dim=1)


# ----------------------------------------------------------------------------------------
# the block
# ----------------------------------------------------------------------------------------


def edge_geometry(pos, edge_index, shifts):
    src, dst = edge_index[0], edge_index[1]
    edge_vec = pos[dst] - pos[src] + shifts
    dist = edge_vec.pow(2).sum(-1).clamp_min(1e-24).sqrt()
    return edge_vec, dist


def edge_conv(params, x_node, edge_index, rot, radial, env, lmax, mmax, c, h):
    """The kernel path proper: gather, rotate in, conv1, gate, conv2, envelope, rotate back,
    scatter-add.  ``rot`` [E, Km, K], ``radial`` [E, R], ``env`` [E].  Returns node_out [N, K, C]
    (eso2_ref.py:334-349)."""
    src, dst = edge_index[0], edge_index[1]
    msg = torch.cat([x_node[src], x_node[dst]], dim=2)
    msg = torch.bmm(rot, msg)
    c1m = [params[f"c1_m.{m}.weight"] for m in range(mmax)]
    c2m = [params[f"c2_m.{m}.weight"] for m in range(mmax)]
    msg, gate = so2_conv(msg, params["c1_m0.weight"], params["c1_m0.bias"], c1m,
                         lmax, mmax, h, radial, lmax * h)
    msg = gate_activation(gate, msg, lmax, mmax)
    msg, _ = so2_conv(msg, params["c2_m0.weight"], params["c2_m0.bias"], c2m,
                      lmax, mmax, c, None, 0)
    msg = msg * env[:, None, None]
    msg = torch.bmm(rot.transpose(1, 2), msg)
    node_out = torch.zeros(x_node.shape[0], msg.shape[1], msg.shape[2], dtype=msg.dtype)
    node_out.index_add_(0, dst, msg)
    return node_out


def block_node_out(params, cfg: dict, pos, atomic_numbers, x_node, edge_index, shifts,
                   cos_gamma_k, sin_gamma_k, jd) -> torch.Tensor:
    """pos -> node_out [N, K, C], everything position-dependent included."""
    lmax, mmax = cfg["lmax"], cfg["mmax"]
    edge_vec, dist = edge_geometry(pos, edge_index, shifts)
    radial = radial_features(params, dist, atomic_numbers[edge_index[0]],
                             atomic_numbers[edge_index[1]], cfg["cutoff"],
                             cfg["num_distance_basis"])
    rot = edge_rotation(edge_vec, cos_gamma_k, sin_gamma_k, lmax, mmax, jd)
    env = envelope(dist / cfg["cutoff"], float(cfg.get("envelope_exponent", 5)))
    return edge_conv(params, x_node, edge_index, rot, radial, env, lmax, mmax,
                     cfg["sphere_channels"], cfg["hidden_channels"])


def node_invariants(node_out, lmax: int):
    feats = [node_out[:, 0, :]]
    for l in range(1, lmax + 1):
        feats.append(node_out[:, l * l:(l + 1) ** 2, :].pow(2).sum(dim=1))
    return torch.cat(feats, dim=-1)


def block_energy(params, cfg, pos, atomic_numbers, x_node, edge_index, shifts,
                 cos_gamma_k, sin_gamma_k, jd) -> torch.Tensor:
    """Scalar E, the reference's ``ESO2RefBlock.forward`` return value (eso2_ref.py:305-351)."""
    f = torch.nn.functional
    node_out = block_node_out(params, cfg, pos, atomic_numbers, x_node, edge_index, shifts,
                              cos_gamma_k, sin_gamma_k, jd)
    inv = node_invariants(node_out, cfg["lmax"])
    hid = f.silu(f.linear(inv, params["readout.0.weight"], params["readout.0.bias"]))
    return f.linear(hid, params["readout.2.weight"], params["readout.2.bias"]).sum()


# ----------------------------------------------------------------------------------------
# parameters
# ----------------------------------------------------------------------------------------


def param_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Shapes of the reference module's 23 parameter tensors (eso2_ref.py:157-238)."""
    lmax, mmax = cfg["lmax"], cfg["mmax"]
    c, h, ec = cfg["sphere_channels"], cfg["hidden_channels"], cfg["edge_channels"]
    nb = cfg["num_distance_basis"]
    ms = m_sizes(lmax, mmax)
    r = 2 * c * sum(ms)
    shapes = {
        "elem_emb.weight": (cfg.get("max_num_elements", 100), ec),
        "rad_func.0.weight": (ec, nb + 2 * ec), "rad_func.0.bias": (ec,),
        "rad_func.1.weight": (ec,), "rad_func.1.bias": (ec,),
        "rad_func.3.weight": (ec, ec), "rad_func.3.bias": (ec,),
        "rad_func.4.weight": (ec,), "rad_func.4.bias": (ec,),
        "rad_func.6.weight": (r, ec), "rad_func.6.bias": (r,),
        "c1_m0.weight": (h * (lmax + 1) + lmax * h, ms[0] * 2 * c),
        "c1_m0.bias": (h * (lmax + 1) + lmax * h,),
    }
    for m in range(1, mmax + 1):
        shapes[f"c1_m.{m - 1}.weight"] = (2 * h * ms[m], ms[m] * 2 * c)
    shapes["c2_m0.weight"] = (c * (lmax + 1), ms[0] * h)
    shapes["c2_m0.bias"] = (c * (lmax + 1),)
    for m in range(1, mmax + 1):
        shapes[f"c2_m.{m - 1}.weight"] = (2 * c * ms[m], ms[m] * h)
    shapes |= {
        "readout.0.weight": (c, c * (lmax + 1)), "readout.0.bias": (c,),
        "readout.2.weight": (1, c), "readout.2.bias": (1,),
    }
    return shapes


def init_params(cfg: dict, seed: int = 0, dtype=torch.float64) -> dict[str, torch.Tensor]:
    """Seeded parameters: Xavier-uniform matrices, small uniform biases, LayerNorm gains near
    one; m > 0 SO(2) weights carry the reference's 1/sqrt(2) (eso2_ref.py:191-192, 201-202).
    Values are irrelevant to parity -- the same tensors go to the oracle and to the kernels."""
    g = torch.Generator("cpu").manual_seed(seed)
    out = {}
    for name, shape in param_shapes(cfg).items():
        if name.startswith("elem_emb"):
            t = torch.randn(shape, generator=g, dtype=torch.float64)
        elif len(shape) == 2:
            bound = math.sqrt(6.0 / (shape[0] + shape[1]))
            t = (torch.rand(shape, generator=g, dtype=torch.float64) * 2 - 1) * bound
            if name.startswith(("c1_m.", "c2_m.")):
                t = t / math.sqrt(2.0)
        elif name in ("rad_func.1.weight", "rad_func.4.weight"):
            t = 1.0 + 0.1 * (torch.rand(shape, generator=g, dtype=torch.float64) * 2 - 1)
        else:
            t = 0.1 * (torch.rand(shape, generator=g, dtype=torch.float64) * 2 - 1)
        out[name] = t.to(dtype)
    return out


def load_jd(path, lmax: int) -> list[torch.Tensor]:
    import numpy as np
    z = np.load(path)
    return [torch.from_numpy(z[f"J{l}"]).to(torch.float64) for l in range(lmax + 1)]
