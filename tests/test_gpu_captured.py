"""CapturedStep (the module's forward + VJP replayed as one CUDA graph) against the module path
it records, on the recording data and on new data of the same sizes."""

import pytest
import torch

from tests.helpers import gpu_node_out_and_vjp, random_case
from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
from zippel_b200.captured import HOST_KEYS, CapturedStep

pytestmark = pytest.mark.gpu

CFG = dict(lmax=3, mmax=2, sphere_channels=32, hidden_channels=32, edge_channels=32,
           num_distance_basis=16, cutoff=5.0)


def _f32(case):
    return {k: (v.float() if v.is_floating_point() else v) for k, v in case.items()}


def _same(a, b):
    if a is None or b is None:
        return a is None and b is None
    return torch.equal(a, b)


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_replay_equals_module_path(precision):
    torch.manual_seed(0)
    block = ESO2Block(BlockConfig(**CFG), precision=precision).to("cuda")
    first, second = _f32(random_case(CFG, 40, 500, 1)), _f32(random_case(CFG, 40, 500, 2))
    step = CapturedStep(block, first, "cuda")
    assert step.h2d_bytes == sum(first[k].numel() * first[k].element_size() for k in HOST_KEYS)
    for case in (first, second, first):
        for k in HOST_KEYS:
            step.host[k].copy_(case[k])
        step.run()
        out, gx, gpos, pg = gpu_node_out_and_vjp(block, case, case["upstream"])
        # the same kernels in the same order on the same data: equal bit for bit
        assert torch.equal(step.node_out, out)
        assert torch.equal(step.grads["x_node"], gx) and torch.equal(step.grads["pos"], gpos)
        assert torch.equal(step.grad_pos_host, gpos.cpu())
        assert torch.equal(step.loss_host, (out * case["upstream"].cuda()).sum().cpu())
        for name, want in pg.items():
            assert _same(step.grads["params"][name], want), name
    assert block.plan("cuda").device_status() == 0


def test_frozen_block_records_a_force_evaluation():
    """With every parameter frozen the recorded step forms the gradients of x_node and pos only;
    they equal those of the step recorded with trainable parameters."""
    torch.manual_seed(2)
    block = ESO2Block(BlockConfig(**CFG)).to("cuda")
    case = _f32(random_case(CFG, 40, 500, 4))
    full = CapturedStep(block, case, "cuda")
    full.run()
    block.requires_grad_(False)
    frozen = CapturedStep(block, case, "cuda")
    block.requires_grad_(True)
    frozen.run()
    assert frozen.grads["params"] == {} and len(full.grads["params"]) > 0
    assert torch.equal(frozen.node_out, full.node_out)
    assert torch.equal(frozen.grads["pos"], full.grads["pos"])
    assert torch.equal(frozen.grads["x_node"], full.grads["x_node"])
    assert torch.equal(frozen.grad_pos_host, full.grad_pos_host)


def test_parameter_updates_are_seen():
    torch.manual_seed(1)
    block = ESO2Block(BlockConfig(**CFG)).to("cuda")
    case = _f32(random_case(CFG, 30, 300, 3))
    step = CapturedStep(block, case, "cuda")
    step.run()
    before = step.node_out.clone()
    with torch.no_grad():
        block.c2_m0.weight.mul_(2.0)
        block.c2_m0.bias.mul_(2.0)
        for lin in block.c2_m:
            lin.weight.mul_(2.0)
    step.run()
    out = gpu_node_out_and_vjp(block, case, case["upstream"])[0]
    assert torch.equal(step.node_out, out)
    assert (step.node_out - 2.0 * before).abs().max() <= 1e-5 * before.abs().max()


def test_needs_cuda():
    block = ESO2Block(BlockConfig(**CFG))
    with pytest.raises(RuntimeError):
        CapturedStep(block, _f32(random_case(CFG, 8, 20, 0)), "cpu")
