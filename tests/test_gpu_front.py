"""The fused per-edge front end (zp_edge_features_forward/backward through EdgeFeatures) against
the same formulas in fp64 torch: outputs 2e-6, gradients 1e-5 relative L2; sorted copies exact."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, r):
    return ((a.double().cpu() - r).norm() / r.norm().clamp_min(1e-300)).item()


@pytest.mark.parametrize("n,e,nb,ec,lmax,p", [(50, 700, 64, 128, 4, 5), (9, 40, 10, 12, 2, 5),
                                               (30, 200, 7, 4, 6, 3), (2000, 60000, 64, 128, 4, 5)])
def test_edge_features_and_vjp(n, e, nb, ec, lmax, p):
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import EdgeFeatures
    from zippel_b200.graph import EdgeGraph
    g = torch.Generator("cpu").manual_seed(n + e)
    cutoff = 6.0
    pos = torch.rand(n, 3, generator=g, dtype=torch.float64) * 5.0
    src = torch.randint(0, n, (e,), generator=g)
    dst = (src + 1 + torch.randint(0, n - 1, (e,), generator=g)) % n
    shifts = torch.randint(-1, 2, (e, 3), generator=g).double() * 2.0
    z = torch.randint(1, 20, (n,), generator=g)
    emb = torch.randn(24, ec, generator=g, dtype=torch.float64)
    off = torch.linspace(0.0, cutoff, nb, dtype=torch.float64)
    coeff = -0.5 / (off[1] - off[0]).item() ** 2
    cg = torch.randn(e, lmax + 1, generator=g, dtype=torch.float64)
    sg = torch.randn(e, lmax + 1, generator=g, dtype=torch.float64)
    ei = torch.stack([src, dst])
    graph = EdgeGraph.build(ei.cuda(), n)
    perm = graph.perm64.cpu()
    # fp64 statement in the sorted order
    pr, er = pos.clone().requires_grad_(True), emb.clone().requires_grad_(True)
    s_, d_ = src[perm], dst[perm]
    vec = pr[d_] - pr[s_] + shifts[perm]
    dist = vec.pow(2).sum(-1).clamp_min(1e-24).sqrt()
    t = dist.unsqueeze(1) - off.unsqueeze(0)
    x_edge = torch.cat([torch.exp(coeff * t * t), er[z[s_]], er[z[d_]]], dim=-1)
    sc = dist / cutoff
    a, b, c = -(p + 1) * (p + 2) / 2, p * (p + 2), -p * (p + 1) / 2
    env = torch.where(sc < 1, 1 + sc ** p * (a + sc * (b + c * sc)), torch.zeros_like(sc))
    u1 = torch.randn(e, 3, generator=g, dtype=torch.float64)
    u2 = torch.randn(x_edge.shape, generator=g, dtype=torch.float64)
    u3 = torch.randn(e, generator=g, dtype=torch.float64)
    wp, we = torch.autograd.grad((vec * u1).sum() + (x_edge * u2).sum() + (env * u3).sum(), [pr, er])

    front = _lib.ZpFrontConfig(lmax, nb, ec, 24, p, cutoff, coeff)
    pc = pos.float().cuda().requires_grad_(True)
    ec_ = emb.float().cuda().requires_grad_(True)
    out = EdgeFeatures.apply(graph, graph.perm, front, pc, shifts.float().cuda(), z.cuda(), ec_,
                             off.float().cuda(), cg.float().cuda(), sg.float().cuda())
    gv, gx, ge, cs, ss = out
    assert rel(gv, vec.detach()) < 2e-6 and rel(gx, x_edge.detach()) < 2e-6
    assert rel(ge, env.detach()) < 2e-5          # 1 - O(1) terms cancel near the cutoff
    assert torch.equal(cs.cpu(), cg.float()[perm]) and torch.equal(ss.cpu(), sg.float()[perm])
    hp, he = torch.autograd.grad((gv * u1.float().cuda()).sum() + (gx * u2.float().cuda()).sum()
                                 + (ge * u3.float().cuda()).sum(), [pc, ec_])
    assert rel(hp, wp) < 1e-5 and rel(he, we) < 1e-5
    # fixed summation order: the same bits on a second run
    out2 = EdgeFeatures.apply(graph, graph.perm, front, pc, shifts.float().cuda(), z.cuda(), ec_,
                              off.float().cuda(), cg.float().cuda(), sg.float().cuda())
    hp2, he2 = torch.autograd.grad((out2[0] * u1.float().cuda()).sum()
                                   + (out2[1] * u2.float().cuda()).sum()
                                   + (out2[2] * u3.float().cuda()).sum(), [pc, ec_])
    assert torch.equal(hp, hp2) and torch.equal(he, he2)


def test_front_config_rejections():
    import ctypes
    from zippel_b200 import _lib
    lib = _lib.load()
    bad = _lib.ZpFrontConfig(2, 8, 6, 10, 5, 6.0, -1.0)          # edge_channels not a multiple of 4
    assert lib.zp_edge_features_work_bytes(ctypes.byref(bad), 10, 10) == 0
    ok = _lib.ZpFrontConfig(2, 8, 8, 10, 5, 6.0, -1.0)
    assert lib.zp_edge_features_work_bytes(ctypes.byref(ok), 10, 10) > 0
