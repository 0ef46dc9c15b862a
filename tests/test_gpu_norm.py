"""LayerNorm + SiLU of the radial MLP's hidden layers (zp_layernorm_silu_forward/backward through
the autograd wrapper) against fp64 torch: 2e-6 relative L2 on the output and every gradient."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, r):
    return ((a.double().cpu() - r).norm() / r.norm().clamp_min(1e-300)).item()


@pytest.mark.parametrize("rows,width", [(1000, 128), (77, 32), (513, 200), (64, 1024), (5, 8),
                                        (60000, 128)])
def test_layernorm_silu_and_vjp(rows, width):
    from zippel_b200.blocks.eso2 import LayerNormSiLU
    g = torch.Generator("cpu").manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g, dtype=torch.float64) * 2.0 + 0.3
    gamma = torch.randn(width, generator=g, dtype=torch.float64)
    beta = torch.randn(width, generator=g, dtype=torch.float64)
    up = torch.randn(rows, width, generator=g, dtype=torch.float64)
    xr, gr, br = (t.clone().requires_grad_(True) for t in (x, gamma, beta))
    want = torch.nn.functional.silu(torch.nn.functional.layer_norm(xr, (width,), gr, br, 1e-5))
    wx, wg, wb = torch.autograd.grad((want * up).sum(), [xr, gr, br])
    xc, gc, bc = (t.float().cuda().requires_grad_(True) for t in (x, gamma, beta))
    got = LayerNormSiLU.apply(xc, gc, bc, 1e-5)
    hx, hg, hb = torch.autograd.grad((got * up.float().cuda()).sum(), [xc, gc, bc])
    assert rel(got, want.detach()) < 2e-6
    assert rel(hx, wx) < 2e-6 and rel(hg, wg) < 2e-6 and rel(hb, wb) < 2e-6
    # fixed summation order: a second backward gives the same bits
    got2 = LayerNormSiLU.apply(xc, gc, bc, 1e-5)
    hx2, hg2, hb2 = torch.autograd.grad((got2 * up.float().cuda()).sum(), [xc, gc, bc])
    assert torch.equal(hg, hg2) and torch.equal(hb, hb2) and torch.equal(hx, hx2)


def test_layernorm_silu_empty_and_rejections():
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import LayerNormSiLU
    x = torch.zeros(0, 16, device="cuda", requires_grad=True)
    gm = torch.ones(16, device="cuda", requires_grad=True)
    bt = torch.zeros(16, device="cuda", requires_grad=True)
    y = LayerNormSiLU.apply(x, gm, bt, 1e-5)
    assert y.shape == (0, 16)
    dg, = torch.autograd.grad(y.sum(), [gm])
    assert dg.abs().max().item() == 0.0
    lib = _lib.load()
    assert lib.zp_layernorm_silu_forward(4, 6, None, None, None, 1e-5, None, None, None, None) == 2
    assert lib.zp_layernorm_silu_forward(4, 2048, None, None, None, 1e-5, None, None, None, None) == 2
