"""The energy head on the library's kernels (zp_readout_forward / zp_readout_backward through
``Readout``) against the oracle's readout in FP64: energy, parameter gradients and the gradient
with respect to the node output (the upstream gradient of the edge convolution's backward)."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lmax,c,n", [(4, 128, 2000), (2, 32, 64), (6, 16, 37), (1, 8, 1)])
def test_readout_forward_and_vjp(lmax, c, n):
    from zippel_b200.blocks.eso2 import Plan, Readout
    g = torch.Generator("cpu").manual_seed(lmax * 100 + c)
    k = (lmax + 1) ** 2
    node_out = torch.randn(n, k, c, generator=g, dtype=torch.float64)
    w0 = torch.randn(c, (lmax + 1) * c, generator=g, dtype=torch.float64) / ((lmax + 1) * c) ** 0.5
    b0 = torch.randn(c, generator=g, dtype=torch.float64) * 0.1
    w1 = torch.randn(1, c, generator=g, dtype=torch.float64) / c ** 0.5
    b1 = torch.randn(1, generator=g, dtype=torch.float64)
    ref = [t.clone().requires_grad_(True) for t in (node_out, w0, b0, w1, b1)]
    inv = orc.node_invariants(ref[0], lmax)
    e_ref = (torch.nn.functional.silu(inv @ ref[1].T + ref[2]) @ ref[3].T + ref[4]).sum()
    grads_ref = torch.autograd.grad(e_ref * 0.7, ref)

    plan = Plan.get(lmax, min(lmax, 2), c, c, "cuda")
    dev = [t.float().cuda().requires_grad_(True) for t in (node_out, w0, b0, w1, b1)]
    e = Readout.apply(plan, *dev)
    grads = torch.autograd.grad(e * 0.7, dev)
    assert abs(e.item() - e_ref.item()) < 1e-5 * max(1.0, abs(e_ref.item()), inv.abs().sum().item() ** 0.5)
    for name, got, want in zip(("node_out", "w0", "b0", "w1", "b1"), grads, grads_ref):
        assert rel_l2(got, want) < 1e-5, name
    e2 = Readout.apply(plan, *dev)
    assert e2.item() == e.item()                     # fixed summation order
    assert plan.device_status() == 0


def test_readout_with_no_atoms():
    from zippel_b200.blocks.eso2 import Plan, Readout
    plan = Plan.get(2, 2, 8, 8, "cuda")
    z = lambda *s: torch.zeros(*s, device="cuda", requires_grad=True)         # noqa: E731
    args = [z(0, 9, 8), z(8, 24), z(8), z(1, 8), z(1)]
    e = Readout.apply(plan, *args)
    assert e.item() == 0.0
    grads = torch.autograd.grad(e, args[1:], allow_unused=True)
    assert all(g is None or g.abs().max().item() == 0.0 for g in grads)
