"""Back end for IR programs: the reference's ``compile_program`` / ``allocate`` / ``run_program``
(``codegen/compose.py:113-239``) over the hand-written kernels.

The reference compiles *any* program by emitting one kernel per fusion group.  This back end
does the opposite for the one program family the kernels implement: ``compile_program`` checks
that the program IS the eSEN SO(2) block as ``blocks.eso2_ir.build_forward`` / ``build_force``
state it -- it reads the configuration off the input types, rebuilds the program for that
configuration and compares every op's structural key, coefficients included -- and refuses
anything else (``UnsupportedProgram``).  ``run_program`` then evaluates the block with the CUDA
kernels (``EdgeConvFunction``) plus the small torch ops around them and stores the program's
outputs in the environment.  There is no interpreter fallback.
"""

from __future__ import annotations

import dataclasses

import torch

from ..blocks.eso2 import BlockConfig, EdgeConvFunction, Plan, Readout, radial_mlp
from ..blocks.eso2_ir import build_force, build_forward
from ..graph import EdgeGraph
from ..zippel.ir import BufferType, Program


class UnsupportedProgram(ValueError):
    """The program is not the SO(2) block this back end has kernels for."""


@dataclasses.dataclass
class CompiledProgram:
    prog: Program
    cfg: BlockConfig
    kind: str                      # "forward" | "force"
    meta: dict
    sizes: dict
    label: str = ""
    dtype: str = "f32"


def _axis(prog: Program, name: str, axis: int) -> int:
    t = prog.inputs.get(name)
    if not isinstance(t, BufferType) or axis >= t.rank:
        raise UnsupportedProgram(f"input {name!r} missing or of unexpected rank")
    return t.sizes[axis]


def _infer(prog: Program):
    lmax = _axis(prog, "cos_g", 0) - 1
    mmax = max(int(n[6:]) for n in prog.inputs if n.startswith("rad_wm"))
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=_axis(prog, "x_node", 1),
               hidden_channels=_axis(prog, "c2_w0", 2), edge_channels=_axis(prog, "emb_src", 0),
               num_distance_basis=_axis(prog, "gauss_offset", 0))
    cutoff = gauss = None
    for op in prog.ops.values():
        if op.kind != "scalar_map" or op.inputs[0] not in prog.ops:
            continue
        feeder = prog.ops[op.inputs[0]]
        if op.fn == "poly_envelope" and op.order == 0 and len(feeder.paths) == 1:
            cutoff = 1.0 / feeder.paths[0].coeff
        if op.fn == "exp" and len(feeder.paths) == 1 and feeder.paths[0].operands == (0, 0):
            gauss = feeder.paths[0].coeff
    if cutoff is None or gauss is None:
        raise UnsupportedProgram("no envelope / Gaussian basis found")
    return BlockConfig(cutoff=cutoff, **cfg), gauss


def compile_program(prog: Program, sizes: dict, label: str = "", dtype: str = "f32",
                    max_volume=None) -> CompiledProgram:
    """Recognises the block program; ``max_volume`` is accepted for signature compatibility."""
    del max_volume
    try:
        cfg, gauss = _infer(prog)
    except (KeyError, ValueError) as exc:
        raise UnsupportedProgram(f"not an SO(2) block program: {exc}") from exc
    kind = "force" if "seed_E" in prog.inputs else "forward"
    want, meta = (build_force if kind == "force" else build_forward)(cfg, gauss)
    if list(want.inputs.items()) != list(prog.inputs.items()) or len(want.ops) != len(prog.ops):
        raise UnsupportedProgram("inputs or op count differ from the SO(2) block program")
    for (n1, a), (n2, b) in zip(want.ops.items(), prog.ops.items()):
        if n1 != n2 or a.key() != b.key():
            raise UnsupportedProgram(f"op {n2!r} differs from the SO(2) block program")
    if want.outputs != prog.outputs:
        raise UnsupportedProgram("outputs differ from the SO(2) block program")
    return CompiledProgram(prog, cfg, kind, meta, dict(sizes), label, dtype)


def allocate(cp: CompiledProgram, inputs: dict, dtype: str | None = None, device="cuda") -> dict:
    """Copies every program input to the device (values as fp32, indices as int64)."""
    del dtype
    env = {}
    for name, t in cp.prog.inputs.items():
        if name not in inputs:
            raise KeyError(f"missing input {name!r}")
        a = inputs[name]
        env[name] = (a.to(device, torch.float32) if isinstance(t, BufferType)
                     else a.to(device, torch.long))
    return env


def _block_energy(cp: CompiledProgram, env: dict, pos: torch.Tensor):
    cfg = cp.cfg
    L, C, H, mmax, EC = cfg.lmax, cfg.sphere_channels, cfg.hidden_channels, cfg.mmax, cfg.edge_channels
    n = pos.shape[0]
    graph = EdgeGraph.build(torch.stack([env["src"], env["dst"]]), n)
    perm, src, dst = graph.perm64, graph.src.long(), graph.dst.long()
    edge_vec = pos[dst] - pos[src] + env["shifts"][perm]
    dist = edge_vec.pow(2).sum(-1).sqrt()
    gauss_coeff = next(op.paths[0].coeff for op in cp.prog.ops.values()
                       if op.kind == "segmented_contraction" and len(op.paths) == 1
                       and op.paths[0].operands == (0, 0) and op.paths[0].subscripts == "g,g->g")
    d = dist[:, None] - env["gauss_offset"][0][None, :]
    x_edge = torch.cat([torch.exp(gauss_coeff * d * d), env["emb_src"][perm], env["emb_dst"][perm]], -1)
    # the radial MLP on the library's kernels, as the module path runs it
    w6 = torch.cat([env[f"rad_wm{m}"][0].reshape(-1, EC) for m in range(mmax + 1)])
    b6 = torch.cat([env[f"rad_bm{m}"][0].reshape(-1) for m in range(mmax + 1)])
    plan = Plan.get(L, mmax, C, H, pos.device)
    layers = []
    for tag in ("0", "1"):
        layers += [("linear", env[f"rad_w{tag}"][0], env[f"rad_b{tag}"][0]),
                   ("ln_silu", env[f"rad_g{tag}"][0], env[f"rad_be{tag}"][0], 1e-5)]
    radial = radial_mlp(plan, x_edge, [*layers, ("linear", w6, b6)])
    ds = dist / cfg.cutoff
    p = float(cfg.envelope_exponent)
    env_e = 1 + ds ** p * (-(p + 1) * (p + 2) / 2 + ds * (p * (p + 2) - p * (p + 1) / 2 * ds))
    env_e = torch.where(ds < 1, env_e, torch.zeros_like(env_e))
    fold = lambda tag, m: torch.cat([env[f"{tag}_w{m}a"][0].flatten(0, 1).flatten(1),      # noqa: E731
                                     env[f"{tag}_w{m}b"][0].flatten(0, 1).flatten(1)])
    node_out = EdgeConvFunction.apply(
        plan, graph, env["x_node"], edge_vec, env["cos_g"][perm], env["sin_g"][perm], radial, env_e,
        None, None, env["c1_w0"][0].flatten(1), env["c1_b0"][0], env["c2_w0"][0].flatten(1), env["c2_b0"][0],
        *[fold("c1", m) for m in range(1, mmax + 1)], *[fold("c2", m) for m in range(1, mmax + 1)])
    energy = Readout.apply(plan, node_out, env["ro_w0"][0], env["ro_b0"][0], env["ro_w1"][0],
                           env["ro_b1"][0])
    return energy, node_out


def run_program(cp: CompiledProgram, env: dict) -> dict:
    """Runs the block on the kernels, stores the program outputs (and ``node_out``) in ``env``
    under their buffer names, synchronises, and returns ``env``."""
    need_force = cp.kind == "force"
    pos = env["pos"].detach().requires_grad_(need_force)
    with torch.enable_grad() if need_force else torch.no_grad():
        energy, node_out = _block_energy(cp, env, pos)
        if need_force:
            (de,) = torch.autograd.grad(energy * env["seed_E"].reshape(()), pos)
            env[cp.meta["dE_dpos"]] = de
            env[cp.meta["force"]] = -de
    env[cp.meta["energy"]] = energy.detach().reshape(1)
    env[cp.meta["node_out"]] = node_out.detach()
    torch.cuda.synchronize(pos.device)
    return env
