"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED reference.

Run where the reference checkout is importable (it is not on the GPU machines):

    python tests/golden/make_golden.py /path/to/reference

For every case it builds seeded inputs, runs ``blocks.eso2_ref.ESO2RefBlock`` and
``blocks.wigner.wigner_from_edge_vec`` in FP64 on CPU, and stores inputs, parameters and
outputs (E, node_out, Wigner-D, dE/dpos, and the VJP of <node_out, g> w.r.t. x_node, pos and
every parameter) in one ``.npz`` per case.  The reference only supports ``mmax == lmax``, so
every case has that shape; ``node_out`` is captured by wrapping the instance's
``node_invariants`` method (the reference's ``forward`` returns only E).
"""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
DT = torch.float64

CASES = {
    # name: (cfg kwargs, nodes, edges, seed)
    "ref_l2m2_c8": (dict(lmax=2, mmax=2, sphere_channels=8, hidden_channels=8, edge_channels=8,
                         num_distance_basis=8, cutoff=5.0), 10, 48, 11),
    "ref_l2m2_c16h8": (dict(lmax=2, mmax=2, sphere_channels=16, hidden_channels=8,
                            edge_channels=12, num_distance_basis=10, cutoff=6.0), 9, 40, 12),
    "ref_l4m4_c8": (dict(lmax=4, mmax=4, sphere_channels=8, hidden_channels=8, edge_channels=4,
                         num_distance_basis=6, cutoff=6.0), 8, 24, 13),
    "ref_l3m3_c8h16": (dict(lmax=3, mmax=3, sphere_channels=8, hidden_channels=16, edge_channels=4,
                         num_distance_basis=5, cutoff=4.0), 7, 30, 14),
}


def make_inputs(cfg, n, e, seed):
    g = torch.Generator("cpu").manual_seed(seed)
    box = 0.8 * cfg.cutoff
    pos = torch.rand(n, 3, generator=g, dtype=DT) * box
    src = torch.randint(0, n, (e,), generator=g)
    dst = (src + 1 + torch.randint(0, n - 1, (e,), generator=g)) % n
    # a few periodic-image shifts, scaled so that most edges stay inside the cutoff
    shifts = torch.randint(-1, 2, (e, 3), generator=g).to(DT) * (0.35 * box)
    shifts[: e // 2] = 0.0
    gamma = torch.rand(e, generator=g, dtype=DT) * 2 * torch.pi
    x_node = torch.randn(n, (cfg.lmax + 1) ** 2, cfg.sphere_channels, generator=g, dtype=DT)
    z = torch.randint(1, 30, (n,), generator=g)
    upstream = torch.randn(n, (cfg.lmax + 1) ** 2, cfg.sphere_channels, generator=g, dtype=DT)
    return pos, torch.stack([src, dst]), shifts, gamma, x_node, z, upstream


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from blocks.eso2_ref import BlockConfig, ESO2RefBlock
    from blocks.wigner import gamma_harmonics, wigner_from_edge_vec

    jd = [j.to(DT) for j in torch.load(pathlib.Path(ref_root) / "blocks" / "Jd.pt",
                                       weights_only=False)]
    for name, (kw, n, e, seed) in CASES.items():
        cfg = BlockConfig(**kw)
        torch.manual_seed(seed)
        block = ESO2RefBlock(cfg).to("cpu", DT)
        # default init leaves biases/LayerNorm at trivial values; perturb so they are live
        with torch.no_grad():
            g = torch.Generator("cpu").manual_seed(seed + 100)
            for p_name, p in block.named_parameters():
                if p.dim() == 1:
                    p.add_(0.1 * torch.randn(p.shape, generator=g, dtype=DT))
        pos, edge_index, shifts, gamma, x_node, z, upstream = make_inputs(cfg, n, e, seed)
        cos_g, sin_g = gamma_harmonics(gamma, cfg.lmax)
        pos.requires_grad_(True)
        x_node.requires_grad_(True)

        captured = []
        orig = block.node_invariants
        block.node_invariants = lambda t: (captured.append(t), orig(t))[1]
        energy = block(pos, z, x_node, edge_index, shifts, cos_g, sin_g, jd)
        node_out = captured[0]

        params = dict(block.named_parameters())
        (de_dpos,) = torch.autograd.grad(energy, pos, retain_graph=True)
        wrt = [x_node, pos, *params.values()]
        grads = torch.autograd.grad((node_out * upstream).sum(), wrt, allow_unused=True)
        edge_vec = (pos[edge_index[1]] - pos[edge_index[0]] + shifts).detach()
        wigner = wigner_from_edge_vec(edge_vec, cos_g, sin_g, cfg.lmax, jd)

        out = {
            "cfg_keys": np.array(list(kw.keys())),
            "cfg_vals": np.array([float(v) for v in kw.values()]),
            "pos": pos.detach().numpy(), "edge_index": edge_index.numpy(),
            "shifts": shifts.numpy(), "gamma": gamma.numpy(),
            "cos_gamma_k": cos_g.numpy(), "sin_gamma_k": sin_g.numpy(),
            "x_node": x_node.detach().numpy(), "atomic_numbers": z.numpy(),
            "upstream": upstream.numpy(),
            "energy": energy.detach().numpy(), "node_out": node_out.detach().numpy(),
            "de_dpos": de_dpos.numpy(), "wigner": wigner.numpy(),
            "vjp_x_node": grads[0].numpy(), "vjp_pos": grads[1].numpy(),
        }
        for (p_name, p), gp in zip(params.items(), grads[2:]):
            out["param:" + p_name] = p.detach().numpy()
            out["vjp_param:" + p_name] = (torch.zeros_like(p) if gp is None else gp).numpy()
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, "E =", float(energy), "edges", e, "bytes",
              (HERE / f"{name}.npz").stat().st_size)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
