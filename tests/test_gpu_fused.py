"""The fused epilogues of the SO(2) contractions (gate activation inside conv1; envelope,
rotation back and the per-node sums inside conv2) against the oracle, the stand-alone kernels
they replace, and the no-gradient entry point that keeps nothing for a backward."""

from __future__ import annotations

import os
import pathlib
import subprocess
import sys

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                           oracle_node_out_and_vjp, random_case, rel_l2)

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]


def _forward(block, case, grad: bool):
    dev = "cuda"
    pos = case["pos"].to(dev, torch.float32)
    x = case["x_node"].to(dev, torch.float32)
    if grad:
        pos, x = pos.requires_grad_(True), x.requires_grad_(True)
    with torch.set_grad_enabled(grad):
        return block.node_output(pos, case["atomic_numbers"].to(dev), x, case["edge_index"].to(dev),
                                 case["shifts"].to(dev, torch.float32),
                                 case["cos_gamma_k"].to(dev, torch.float32),
                                 case["sin_gamma_k"].to(dev, torch.float32)).detach()


@pytest.mark.parametrize("precision,tol", [("fp32", 1e-5), ("bf16", 2e-2), ("fp32_bf16x3", 1e-5)])
@pytest.mark.parametrize("lmax,mmax,c,h,n,e", [(4, 2, 128, 128, 50, 700), (2, 2, 32, 16, 9, 70),
                                               (6, 2, 16, 24, 20, 333), (1, 0, 8, 8, 6, 40)])
def test_inference_entry_matches_training_forward(lmax, mmax, c, h, n, e, precision, tol, jd64):
    """zp_eso2_forward_inference (taken under no_grad) returns what zp_eso2_forward returns, bit
    for bit: both run the same arithmetic, one of them without storing the activations."""
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=61)
    case = random_case(cfg, n, e, seed=62)
    block = make_block(cfg, params, precision=precision)
    kept = _forward(block, case, grad=True)
    lean = _forward(block, case, grad=False)
    assert torch.equal(kept, lean)
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)[0]
    assert rel_l2(lean, want) < tol
    assert block.plan("cuda").device_status() == 0


def test_runs_of_edges_across_32_edge_blocks(jd64):
    """Destination nodes whose edges start and end anywhere relative to the 32-edge blocks the
    rotate-back epilogue works in: degrees 0, 1, 31, 32, 33, 64, 65 and 200 in one graph."""
    cfg = dict(lmax=3, mmax=2, sphere_channels=32, hidden_channels=16, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    degrees = [1, 0, 31, 32, 0, 0, 33, 64, 1, 65, 200, 2, 0, 30]
    n = len(degrees)
    dst = torch.cat([torch.full((d,), i) for i, d in enumerate(degrees)])
    g = torch.Generator("cpu").manual_seed(5)
    src = (dst + 1 + torch.randint(0, n - 1, dst.shape, generator=g)) % n
    case = random_case(cfg, n, dst.numel(), seed=71)
    perm = torch.randperm(dst.numel(), generator=g)
    case["edge_index"] = torch.stack([src, dst])[:, perm]
    params = orc.init_params(cfg, seed=72)
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    block = make_block(cfg, params)
    got = gpu_node_out_and_vjp(block, case, case["upstream"])
    check_against(*got, *want)
    again = gpu_node_out_and_vjp(block, case, case["upstream"])
    assert torch.equal(got[0], again[0])                     # fixed summation order
    assert got[0][[1, 4, 5, 12]].abs().max().item() == 0.0
    assert torch.equal(_forward(block, case, grad=False), got[0])


_CHILD = r"""
import sys, torch
sys.path.insert(0, {root!r})
from oracle import eso2_oracle as orc
from tests.helpers import gpu_node_out_and_vjp, make_block, oracle_node_out_and_vjp, random_case, check_against
cfg = dict(lmax=4, mmax=2, sphere_channels=32, hidden_channels=32, edge_channels=8,
           num_distance_basis=6, cutoff=5.0)
params = orc.init_params(cfg, seed=81)
case = random_case(cfg, 25, 300, seed=82)
jd = orc.load_jd({root!r} + "/zippel_b200/data/jd.npz", 8)
want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd)
got = gpu_node_out_and_vjp(make_block(cfg, params), case, case["upstream"])
check_against(*got, *want)
torch.save(got[0].cpu(), sys.argv[1])
print("child ok")
"""


def test_stand_alone_kernels_still_serve(tmp_path):
    """With ZP_FUSED_EPILOGUE=0 the gate and rotate-back/scatter kernels run as launches of their
    own (the path the three-plane format always takes): same tolerance, and the two paths agree."""
    outs = []
    for flag in ("0", "1"):
        out = tmp_path / f"node_out_{flag}.pt"
        env = dict(os.environ, ZP_FUSED_EPILOGUE=flag)
        res = subprocess.run([sys.executable, "-c", _CHILD.format(root=str(ROOT)), str(out)],
                             env=env, capture_output=True, text=True, timeout=600)
        assert res.returncode == 0 and "child ok" in res.stdout, res.stdout + res.stderr
        outs.append(torch.load(out))
    assert rel_l2(outs[0], outs[1]) < 2e-6
