"""Helpers shared by the GPU parity tests: run the CUDA block and the oracle on one case."""

from __future__ import annotations

import torch

from oracle import eso2_oracle as orc
from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()


def make_block(cfg: dict, params: dict, device="cuda", dtype=torch.float32,
               precision: str = "fp32") -> ESO2Block:
    block = ESO2Block(BlockConfig(**cfg), precision=precision)
    block.load_state_dict({k: v.clone() for k, v in params.items()})
    return block.to(device=device, dtype=dtype)


def gpu_node_out_and_vjp(block, case, upstream, dtype=torch.float32, device="cuda"):
    """node_out and the VJP of <node_out, upstream> w.r.t. x_node, pos and all parameters."""
    pos = case["pos"].to(device, dtype).requires_grad_(True)
    x_node = case["x_node"].to(device, dtype).requires_grad_(True)
    node_out = block.node_output(
        pos, case["atomic_numbers"].to(device), x_node, case["edge_index"].to(device),
        case["shifts"].to(device, dtype), case["cos_gamma_k"].to(device, dtype),
        case["sin_gamma_k"].to(device, dtype))
    names = [n for n, _ in block.named_parameters()]
    grads = torch.autograd.grad((node_out * upstream.to(device, dtype)).sum(),
                                [x_node, pos, *block.parameters()], allow_unused=True)
    pg = {n: g for n, g in zip(names, grads[2:])}
    return node_out.detach(), grads[0], grads[1], pg


def oracle_node_out_and_vjp(cfg: dict, params: dict, case, upstream, jd):
    pos = case["pos"].double().clone().requires_grad_(True)
    x_node = case["x_node"].double().clone().requires_grad_(True)
    p = {k: v.double().clone().requires_grad_(True) for k, v in params.items()}
    node_out = orc.block_node_out(p, cfg, pos, case["atomic_numbers"], x_node, case["edge_index"],
                                  case["shifts"].double(), case["cos_gamma_k"].double(),
                                  case["sin_gamma_k"].double(), jd)
    grads = torch.autograd.grad((node_out * upstream.double()).sum(), [x_node, pos, *p.values()],
                                allow_unused=True)
    pg = {n: g for n, g in zip(p, grads[2:])}
    return node_out.detach(), grads[0], grads[1], pg


def random_case(cfg: dict, n: int, e: int, seed: int, box: float = 4.0) -> dict:
    """Random multigraph without self loops; some nodes may have no incoming edges."""
    g = torch.Generator("cpu").manual_seed(seed)
    lmax = cfg["lmax"]
    src = torch.randint(0, n, (e,), generator=g)
    dst = (src + 1 + torch.randint(0, max(n - 1, 1), (e,), generator=g)) % n
    gamma = torch.rand(e, generator=g, dtype=torch.float64) * 2 * torch.pi
    cg, sg = orc.gamma_harmonics(gamma, lmax)
    shifts = torch.randint(-1, 2, (e, 3), generator=g).double() * 0.5
    return {
        "pos": torch.rand(n, 3, generator=g, dtype=torch.float64) * box,
        "atomic_numbers": torch.randint(1, 30, (n,), generator=g),
        "x_node": torch.randn(n, (lmax + 1) ** 2, cfg["sphere_channels"], generator=g,
                              dtype=torch.float64),
        "edge_index": torch.stack([src, dst]), "shifts": shifts,
        "cos_gamma_k": cg, "sin_gamma_k": sg,
        "upstream": torch.randn(n, (lmax + 1) ** 2, cfg["sphere_channels"], generator=g,
                                dtype=torch.float64),
    }


def check_against(node_out, gx, gpos, pg, want_out, want_gx, want_gpos, want_pg, tol=1e-5, rows=None):
    """Relative-L2 comparison of outputs and all gradients; unused parameters must have zero/None."""
    if rows is None:
        assert rel_l2(node_out, want_out) < tol
    else:
        assert rel_l2(node_out[rows], want_out[rows]) < tol
    assert rel_l2(gx, want_gx) < tol
    assert rel_l2(gpos, want_gpos) < tol
    for name, want in want_pg.items():
        got = pg[name]
        if want is None or want.abs().max().item() == 0.0:
            assert got is None or got.abs().max().item() == 0.0, name
            continue
        assert rel_l2(got, want) < tol, name
