"""The block in the IR: interpreter == oracle, IR force == autograd, symmetries, clean-up
(after the reference's tests/test_ir_block.py:53-222 and tests/test_ir_wigner.py:84-127)."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc
from oracle import ir_interp as interp
from tests.helpers import random_case
from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
from zippel_b200.blocks.eso2_ir import build_force, build_forward
from zippel_b200.blocks.ir_bind import bind
from zippel_b200.zippel.simplify import op_stats, simplify

DT = torch.float64


def setup(lmax, mmax, c=4, h=4, seed=0):
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=4,
               num_distance_basis=5, cutoff=5.0)
    params = orc.init_params(cfg, seed=seed)
    block = ESO2Block(BlockConfig(**cfg)).double()
    block.load_state_dict(params)
    case = random_case(cfg, 7, 20, seed=seed + 1)
    batch = {k: case[k] for k in ("pos", "x_node", "edge_index", "shifts", "atomic_numbers",
                                  "cos_gamma_k", "sin_gamma_k")}
    return cfg, params, block, batch


@pytest.mark.parametrize("lmax,mmax", [(2, 2), (3, 1), (4, 2)])
def test_interpreter_energy_and_force_match_oracle(lmax, mmax, jd64):
    cfg, params, block, batch = setup(lmax, mmax)
    prog, meta = build_force(BlockConfig(**cfg), block.gauss_coeff)
    inputs, sizes = bind(block, batch, jd64)
    inputs["seed_E"] = torch.ones(1, dtype=DT)
    env = interp.run(prog, inputs, sizes)
    pos = batch["pos"].clone().requires_grad_(True)
    e = orc.block_energy(params, cfg, pos, batch["atomic_numbers"], batch["x_node"],
                         batch["edge_index"], batch["shifts"], batch["cos_gamma_k"],
                         batch["sin_gamma_k"], jd64)
    (de,) = torch.autograd.grad(e, pos)
    assert abs(env[meta["energy"]].item() - e.item()) < 1e-11 * max(1.0, abs(e.item()))
    assert (env[meta["force"]] + de).abs().max().item() < 1e-10 * max(1.0, de.abs().max().item())
    assert env[meta["force"]].sum(0).abs().max().item() < 1e-10          # no net force
    want_nodes = orc.block_node_out(params, cfg, batch["pos"], batch["atomic_numbers"],
                                    batch["x_node"], batch["edge_index"], batch["shifts"],
                                    batch["cos_gamma_k"], batch["sin_gamma_k"], jd64)
    assert (env[meta["node_out"]] - want_nodes).abs().max().item() < 1e-11


def test_simplify_keeps_outputs_and_shrinks_force_program(jd64):
    cfg, params, block, batch = setup(2, 2, seed=3)
    prog, meta = build_force(BlockConfig(**cfg), block.gauss_coeff)
    small = simplify(prog)
    assert len(small.ops) < len(prog.ops)
    inputs, sizes = bind(block, batch, jd64)
    inputs["seed_E"] = torch.ones(1, dtype=DT)
    a, b = interp.run(prog, inputs, sizes), interp.run(small, inputs, sizes)
    for x, y in zip(prog.outputs, small.outputs):
        assert torch.equal(a[x], b[y])
    assert op_stats(small)["contractions"] > 0


def test_only_declared_transcendentals_on_the_position_path():
    prog, _ = build_force(BlockConfig(lmax=2, mmax=2, sphere_channels=4, hidden_channels=4,
                                      edge_channels=4, num_distance_basis=5))
    fns = {op.fn for op in prog.ops.values() if op.kind == "scalar_map"}
    assert "sin" not in fns and "cos" not in fns
    assert fns <= {"exp", "sigmoid", "silu", "rsqrt", "reciprocal", "poly_envelope"}


def test_bind_accepts_reference_shaped_layouts(jd64):
    cfg, params, block, batch = setup(4, 2, c=8, h=4)
    inputs, sizes = bind(block, batch, jd64)
    assert inputs["to_m"].shape == (1, 19, 25) and sizes == {"node": 7, "edge": 20, "graph": 1}
    assert inputs["c1_w1a"].shape == (1, 4, 4, 4, 16) and inputs["rad_wm2"].shape == (1, 3, 16, 4)
    prog, _ = build_forward(BlockConfig(**cfg))
    assert set(prog.inputs) <= set(inputs)


def _training_step_oracle(params, cfg, batch, jd, pos, x_node, e_ref, f_ref, w_e=1.0, w_f=1.0):
    """E, F = -dE/dpos kept differentiable, L = w_e (E - e_ref)^2 + w_f mean((F - f_ref)^2): the
    reference's conservative_training_step (blocks/eso2_ref.py:365-385) on the oracle."""
    e = orc.block_energy(params, cfg, pos, batch["atomic_numbers"], x_node, batch["edge_index"],
                         batch["shifts"], batch["cos_gamma_k"], batch["sin_gamma_k"], jd)
    (de,) = torch.autograd.grad(e, pos, create_graph=True)
    f = -de
    return e, f, w_e * (e - e_ref).pow(2).mean() + w_f * (f - f_ref).pow(2).mean()


@pytest.mark.parametrize("lmax,mmax", [(2, 2), (3, 1)])
def test_double_backward_program_three_ways(lmax, mmax, jd64):
    """build_dbwd evaluated by the interpreter == double autograd through the oracle == central
    differences of the loss (after the reference's tests/test_ir_block.py:106-137)."""
    from zippel_b200.blocks.eso2_ir import build_dbwd
    cfg, params, block, batch = setup(lmax, mmax, seed=5)
    n = batch["pos"].shape[0]
    g = torch.Generator("cpu").manual_seed(9)
    e_ref = torch.randn(1, generator=g, dtype=DT)
    f_ref = torch.randn(n, 3, generator=g, dtype=DT)
    prog, meta = build_dbwd(BlockConfig(**cfg), block.gauss_coeff, w_e=0.7, w_f=1.3)
    inputs, sizes = bind(block, batch, jd64)
    inputs |= {"seed_E": torch.ones(1, dtype=DT), "seed_L": torch.ones(1, dtype=DT), "e_ref": e_ref,
               "f_ref": f_ref, "inv_nf": torch.full((1,), 1.0 / (3 * n), dtype=DT)}
    env = interp.run(prog, inputs, sizes)

    p = {k: v.clone().requires_grad_(True) for k, v in params.items()}
    pos = batch["pos"].clone().requires_grad_(True)
    x = batch["x_node"].clone().requires_grad_(True)
    e, f, loss = _training_step_oracle(p, cfg, batch, jd64, pos, x, e_ref[0], f_ref, 0.7, 1.3)
    names = ["c1_m0.weight", "c2_m0.bias", "rad_func.0.weight", "readout.2.weight", "rad_func.4.bias"]
    grads = torch.autograd.grad(loss, [pos, x, *[p[k] for k in names]])

    rel = lambda a, b: ((a - b).norm() / b.norm().clamp_min(1e-300)).item()      # noqa: E731
    assert abs(env[meta["loss"]].item() - loss.item()) < 1e-11 * max(1.0, abs(loss.item()))
    assert rel(env[meta["force"]], f.detach()) < 1e-10
    assert rel(env[meta["grads"]["pos"]], grads[0]) < 1e-9
    assert rel(env[meta["grads"]["x_node"]], grads[1]) < 1e-9
    ir_names = {"c1_m0.weight": "c1_w0", "c2_m0.bias": "c2_b0", "rad_func.0.weight": "rad_w0",
                "readout.2.weight": "ro_w1", "rad_func.4.bias": "rad_be1"}
    for k, want in zip(names, grads[2:]):
        got = env[meta["grads"][ir_names[k]]].reshape(want.shape)
        assert rel(got, want) < 1e-9, k

    # third leg: central differences of L along a random direction in position space
    def loss_at(q):
        q = q.clone().requires_grad_(True)
        return _training_step_oracle(params, cfg, batch, jd64, q, batch["x_node"], e_ref[0], f_ref,
                                     0.7, 1.3)[2].item()

    d = torch.randn(n, 3, generator=g, dtype=DT)
    h = 1e-6
    fd = (loss_at(batch["pos"] + h * d) - loss_at(batch["pos"] - h * d)) / (2 * h)
    got = (env[meta["grads"]["pos"]] * d).sum().item()
    assert abs(got - fd) < 1e-6 * max(abs(fd), 1e-9)
