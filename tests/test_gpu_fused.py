"""The opt-in fused epilogues of the SO(2) contractions (ZP_FUSED_EPILOGUE=1: gate activation
inside conv1; envelope, rotation back and the per-node sums inside conv2) against the oracle and
against the stand-alone kernels, and the no-gradient entry point that keeps nothing for a backward.

The library reads the switch once per process, so every case runs in a child process with the
switch set; this file doubles as the child's program (``python tests/test_gpu_fused.py CASE``)."""

from __future__ import annotations

import os
import pathlib
import subprocess
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


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


def _jd():
    from oracle import eso2_oracle as orc
    return orc.load_jd(ROOT / "zippel_b200" / "data" / "jd.npz", 8)


def case_inference(out_path: str) -> None:
    """zp_eso2_forward_inference (taken under no_grad) returns what zp_eso2_forward returns, bit
    for bit -- same arithmetic, one of them without storing the activations -- within the oracle's
    tolerance, in all three operand formats (the three-plane one never fuses)."""
    from oracle import eso2_oracle as orc
    from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                               oracle_node_out_and_vjp, random_case, rel_l2)
    jd = _jd()
    for lmax, mmax, c, h, n, e in [(4, 2, 128, 128, 50, 700), (2, 2, 32, 16, 9, 70),
                                   (6, 2, 16, 24, 20, 333), (1, 0, 8, 8, 6, 40)]:
        cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=8,
                   num_distance_basis=6, cutoff=5.0)
        params = orc.init_params(cfg, seed=61)
        case = random_case(cfg, n, e, seed=62)
        want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd)
        for precision, tol in (("fp32", 1e-5), ("bf16", 2e-2), ("fp32_bf16x3", 1e-5)):
            block = make_block(cfg, params, precision=precision)
            kept = _forward(block, case, grad=True)
            lean = _forward(block, case, grad=False)
            assert torch.equal(kept, lean), (cfg, precision)
            assert rel_l2(lean, want[0]) < tol, (cfg, precision)
            got = gpu_node_out_and_vjp(block, case, case["upstream"])     # and the VJP after it
            check_against(*got, *want, tol=tol)
            assert block.plan("cuda").device_status() == 0
    torch.save(torch.zeros(1), out_path)


def case_runs(out_path: str) -> None:
    """Destination nodes whose edges start and end anywhere relative to the 32-edge blocks the
    rotate-back epilogue works in: degrees 0, 1, 31, 32, 33, 64, 65 and 200 in one graph."""
    from oracle import eso2_oracle as orc
    from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                               oracle_node_out_and_vjp, random_case)
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
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], _jd())
    block = make_block(cfg, params)
    got = gpu_node_out_and_vjp(block, case, case["upstream"])
    check_against(*got, *want)
    again = gpu_node_out_and_vjp(block, case, case["upstream"])
    assert torch.equal(got[0], again[0])                     # fixed summation order
    assert got[0][[1, 4, 5, 12]].abs().max().item() == 0.0
    assert torch.equal(_forward(block, case, grad=False), got[0])
    torch.save(torch.zeros(1), out_path)


def case_ab(out_path: str) -> None:
    """One mid-size case, result saved: the parent compares fused and stand-alone runs."""
    from oracle import eso2_oracle as orc
    from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                               oracle_node_out_and_vjp, random_case)
    cfg = dict(lmax=4, mmax=2, sphere_channels=32, hidden_channels=32, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=81)
    case = random_case(cfg, 25, 300, seed=82)
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], _jd())
    got = gpu_node_out_and_vjp(make_block(cfg, params), case, case["upstream"])
    check_against(*got, *want)
    torch.save(got[0].cpu(), out_path)


def _child(case: str, out: pathlib.Path, fused: str):
    env = dict(os.environ, ZP_FUSED_EPILOGUE=fused)
    res = subprocess.run([sys.executable, str(pathlib.Path(__file__).resolve()), case, str(out)],
                         env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0 and "child ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
    return torch.load(out)


@pytest.mark.parametrize("case", ["inference", "runs"])
def test_fused_epilogues(case, tmp_path):
    _child(case, tmp_path / "out.pt", "1")


def test_fused_and_stand_alone_paths_agree(tmp_path):
    """Same tolerance against the oracle on both paths, and the two node outputs agree."""
    from tests.helpers import rel_l2
    a = _child("ab", tmp_path / "a.pt", "0")
    b = _child("ab", tmp_path / "b.pt", "1")
    assert rel_l2(a, b) < 2e-6


def test_inference_entry_without_fusion(jd64):
    """In the default build the no-gradient entry point runs the stand-alone kernels."""
    from oracle import eso2_oracle as orc
    from tests.helpers import make_block, random_case
    cfg = dict(lmax=4, mmax=2, sphere_channels=16, hidden_channels=16, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=91)
    case = random_case(cfg, 30, 400, seed=92)
    block = make_block(cfg, params)
    assert torch.equal(_forward(block, case, grad=True), _forward(block, case, grad=False))


if __name__ == "__main__":
    {"inference": case_inference, "runs": case_runs, "ab": case_ab}[sys.argv[1]](sys.argv[2])
    print("child ok")
