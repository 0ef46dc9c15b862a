"""Binds a block's parameters and a batch dict to the input names of the IR programs.

Same contract as the reference's ``blocks/ir_bind.py:26-103``: ``bind(block, batch, jd_list, cfg)
-> (inputs, sizes)`` with every value tensor carrying a leading segment axis (length 1 for shared
parameters), FP64 on the CPU.  ``block`` may be an ``ESO2Block`` or a reference ``ESO2RefBlock``
(same parameter names).  ``to_m`` is the rectangular ``[1, Km, K]`` selection.
"""

from __future__ import annotations

import torch

from .eso2 import BlockConfig, Layout

DT = torch.float64


def pack_jd(jd_list, lmax: int) -> torch.Tensor:
    k = (lmax + 1) ** 2
    out = torch.zeros(1, k, k, dtype=DT)
    for l in range(lmax + 1):
        out[0, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = jd_list[l].to(DT)
    return out


def bind(block, batch, jd_list, cfg: BlockConfig | None = None):
    cfg = cfg or block.cfg
    L, C, H, mmax = cfg.lmax, cfg.sphere_channels, cfg.hidden_channels, cfg.mmax
    EC, NB, C2 = cfg.edge_channels, cfg.num_distance_basis, 2 * cfg.sphere_channels
    layout = Layout.make(L, mmax)
    n, e = batch["pos"].shape[0], batch["edge_index"].shape[1]
    src, dst = batch["edge_index"][0].cpu(), batch["edge_index"][1].cpu()
    z = batch["atomic_numbers"].cpu()
    t = lambda x: x.detach().to("cpu", DT)                                     # noqa: E731
    one = lambda *shape: torch.ones(*shape, dtype=DT)                           # noqa: E731
    emb = t(block.elem_emb.weight)
    inputs = {
        "pos": t(batch["pos"]), "x_node": t(batch["x_node"]), "shifts": t(batch["shifts"]),
        "cos_g": t(batch["cos_gamma_k"]), "sin_g": t(batch["sin_gamma_k"]),
        "emb_src": emb[z[src]], "emb_dst": emb[z[dst]], "src": src, "dst": dst,
        "zn": torch.zeros(n, dtype=torch.long), "ze": torch.zeros(e, dtype=torch.long),
        "jd": pack_jd(jd_list, L), "to_m": layout.to_m("cpu", DT).unsqueeze(0),
        "gauss_offset": t(block.gauss_offset).unsqueeze(0), "ones_g": one(1, NB), "ones": one(e),
        "unit": one(1, 1), "unit_mat": one(1, 1, 1), "unit_m": one(1, 1), "ones_ec": one(1, EC),
    }
    rad = block.rad_func
    for tag, i_lin, i_ln in (("0", 0, 1), ("1", 3, 4)):
        inputs[f"rad_w{tag}"] = t(rad[i_lin].weight).unsqueeze(0)
        inputs[f"rad_b{tag}"] = t(rad[i_lin].bias).unsqueeze(0)
        inputs[f"rad_g{tag}"] = t(rad[i_ln].weight).unsqueeze(0)
        inputs[f"rad_be{tag}"] = t(rad[i_ln].bias).unsqueeze(0)
    fw, fb, off = t(rad[6].weight), t(rad[6].bias), 0
    for m in range(mmax + 1):
        width = layout.m_size[m] * C2
        inputs[f"rad_wm{m}"] = fw[off:off + width].reshape(1, layout.m_size[m], C2, EC)
        inputs[f"rad_bm{m}"] = fb[off:off + width].reshape(1, layout.m_size[m], C2)
        off += width
    inputs["c1_w0"] = t(block.c1_m0.weight).reshape(1, -1, layout.m_size[0], C2)
    inputs["c1_b0"] = t(block.c1_m0.bias).unsqueeze(0)
    inputs["c2_w0"] = t(block.c2_m0.weight).reshape(1, -1, layout.m_size[0], H)
    inputs["c2_b0"] = t(block.c2_m0.bias).unsqueeze(0)
    for m in range(1, mmax + 1):
        km = layout.m_size[m]
        for tag, mod, cin, cout in (("c1", block.c1_m[m - 1], C2, H), ("c2", block.c2_m[m - 1], H, C)):
            w = t(mod.weight)                       # rows (half, j, o), columns (k, c)
            half = w.shape[0] // 2
            inputs[f"{tag}_w{m}a"] = w[:half].reshape(1, km, cout, km, cin)
            inputs[f"{tag}_w{m}b"] = w[half:].reshape(1, km, cout, km, cin)
    inputs["ro_w0"] = t(block.readout[0].weight).unsqueeze(0)
    inputs["ro_b0"] = t(block.readout[0].bias).unsqueeze(0)
    inputs["ro_w1"] = t(block.readout[2].weight).unsqueeze(0)
    inputs["ro_b1"] = t(block.readout[2].bias).unsqueeze(0)
    return inputs, {"node": n, "edge": e, "graph": 1}
