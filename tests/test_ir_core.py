"""The IR layer: type checking, evaluation, the VJP transform, CSE/DCE (after the reference's
tests/test_ir_core.py:95-328)."""

from __future__ import annotations

import pytest
import torch

from oracle import ir_interp as interp
from zippel_b200.zippel.ir import BufferType, ContractionPath, IndexType, Program
from zippel_b200.zippel.simplify import cse, dce, op_stats, simplify
from zippel_b200.zippel.vjp import ClosureError, assert_closed, vjp

S = slice(None)
DT = torch.float64


def linear_prog():
    p = Program()
    p.add_input("x", BufferType("edge", (("i", 4),)))
    p.add_input("w", BufferType("none", (("o", 3), ("i", 4))))
    p.add_input("b", BufferType("none", (("o", 3),)))
    y = p.contract(["x", "w", "b"], BufferType("edge", (("o", 3),)),
                   [ContractionPath(1.0, "i,oi->o", (0, 1), ((S,), (S, S)), (S,)),
                    ContractionPath(1.0, "o->o", (2,), ((S,),), (S,))])
    return p, y


def test_type_checker_rejections():
    with pytest.raises(ValueError):
        BufferType("atom", ())
    with pytest.raises(ValueError):
        BufferType("edge", (("a", 2), ("a", 3)))
    with pytest.raises(ValueError):
        BufferType("edge", (("a", 0),))
    p = Program()
    p.add_input("x", BufferType("edge", (("i", 4),)))
    p.add_input("n", BufferType("node", (("i", 4),)))
    p.add_input("g", BufferType("none", (("i", 4),)))
    p.add_input("idx", IndexType("edge"))
    with pytest.raises(ValueError):
        p.add_input("x", BufferType("edge", ()))
    t = BufferType("edge", (("i", 4),))
    ok = ContractionPath(1.0, "i->i", (0,), ((S,),), (S,))
    with pytest.raises(ValueError):
        p.contract(["x"], t, [])
    with pytest.raises(TypeError):
        p.contract(["idx"], t, [ok])                         # index buffer as operand
    with pytest.raises(TypeError):
        p.contract(["n"], t, [ok], index_maps=["x"])         # gather map is not an index buffer
    with pytest.raises(TypeError):
        p.contract(["g"], t, [ok], index_maps=["idx"])       # gather from a 'none' buffer
    with pytest.raises(TypeError):
        p.contract(["n"], t, [ok])                           # node -> edge without a map
    with pytest.raises(ValueError):
        p.contract(["x"], BufferType("edge", ()), [ContractionPath(1.0, "i->", (0,), ((S,),), ())])
    with pytest.raises(ValueError):
        p.contract(["x"], t, [ContractionPath(1.0, "i->j", (0,), ((S,),), (S,))])
    with pytest.raises(ValueError):
        p.contract(["x", "g"], t, [ContractionPath(1.0, "i,i->i", (0,), ((S,),), (S,))])
    with pytest.raises(ValueError):
        p.contract(["x"], t, [ContractionPath(1.0, "i->i", (3,), ((S,),), (S,))])
    with pytest.raises(ValueError):
        p.contract(["x"], t, [ContractionPath(1.0, "i->i", (0,), ((slice(0, 2),),), (S,))])
    with pytest.raises(ValueError):
        p.scalar("x", "tanh")
    with pytest.raises(ValueError):
        p.scalar("x", "exp", order=1)
    with pytest.raises(TypeError):
        p.scalar("idx", "exp")
    assert p.contract(["n"], t, [ok], index_maps=["idx"]) in p.ops        # gather is fine


def test_interpreter_matches_torch():
    p, y = linear_prog()
    g = torch.Generator().manual_seed(0)
    x, w, b = (torch.randn(s, generator=g, dtype=DT) for s in ((7, 4), (1, 3, 4), (1, 3)))
    env = interp.run(p, {"x": x, "w": w, "b": b}, {"edge": 7})
    assert torch.allclose(env[y], x @ w[0].T + b[0])
    with pytest.raises(ValueError):
        interp.run(p, {"x": x[:, :3], "w": w, "b": b}, {"edge": 7})
    with pytest.raises(KeyError):
        interp.run(p, {"x": x, "w": w}, {"edge": 7})


def test_vjp_matches_autograd_with_gather_scatter_and_diamond():
    p = Program()
    p.add_input("h", BufferType("node", (("c", 3),)))
    p.add_input("w", BufferType("none", (("c", 3),)))
    p.add_input("src", IndexType("edge"))
    p.add_input("dst", IndexType("edge"))
    p.add_input("zn", IndexType("node"))
    p.add_input("ze", IndexType("edge"))
    p.add_input("seed", BufferType("graph", ()))
    et = BufferType("edge", (("c", 3),))
    a = p.contract(["h", "w"], et, [ContractionPath(1.0, "c,c->c", (0, 1), ((S,), (S,)), (S,))],
                   index_maps=["src", None])
    s = p.scalar(a, "silu")
    d = p.contract([s, a, "h"], et,                          # diamond: a used twice, h twice
                   [ContractionPath(2.0, "c,c->c", (0, 1), ((S,), (S,)), (S,)),
                    ContractionPath(1.0, "c,c->c", (2, 2), ((S,), (S,)), (S,))],
                   index_maps=[None, None, "dst"])
    n = p.contract([d], BufferType("node", (("c", 3),)),
                   [ContractionPath(1.0, "c->c", (0,), ((S,),), (S,))], out_index_map="dst")
    e = p.contract([n, n], BufferType("graph", ()),
                   [ContractionPath(1.0, "c,c->", (0, 1), ((S,), (S,)), ())], out_index_map="zn")
    grads = vjp(p, e, ["h", "w"], "seed", zero_index={"node": "zn", "edge": "ze"})
    assert_closed(p)
    g = torch.Generator().manual_seed(1)
    h = torch.randn(5, 3, generator=g, dtype=DT, requires_grad=True)
    w = torch.randn(1, 3, generator=g, dtype=DT, requires_grad=True)
    src, dst = torch.randint(0, 5, (9,), generator=g), torch.randint(0, 5, (9,), generator=g)
    env = interp.run(p, {"h": h.detach(), "w": w.detach(), "src": src, "dst": dst,
                         "zn": torch.zeros(5, dtype=torch.long), "ze": torch.zeros(9, dtype=torch.long),
                         "seed": torch.ones(1, dtype=DT)}, {"node": 5, "edge": 9, "graph": 1})
    a_t = h[src] * w
    d_t = 2.0 * torch.nn.functional.silu(a_t) * a_t + h[dst] * h[dst]
    n_t = torch.zeros(5, 3, dtype=DT).index_add(0, dst, d_t)
    e_t = (n_t * n_t).sum()
    gh, gw = torch.autograd.grad(e_t, [h, w])
    assert torch.allclose(env[e], e_t.detach().reshape(1))
    assert torch.allclose(env[grads["h"]], gh, atol=1e-12)
    assert torch.allclose(env[grads["w"]], gw, atol=1e-12)


@pytest.mark.parametrize("fn", ["exp", "sigmoid", "silu", "rsqrt", "reciprocal", "sin", "cos",
                                "poly_envelope"])
def test_scalar_derivatives(fn):
    p = Program()
    p.add_input("x", BufferType("edge", (("c", 2),)))
    p.add_input("seed", BufferType("edge", (("c", 2),)))
    y = p.scalar("x", fn)
    grads = vjp(p, y, ["x"], "seed")
    x = torch.rand(6, 2, dtype=DT) * 0.8 + 0.1
    env = interp.run(p, {"x": x, "seed": torch.ones(6, 2, dtype=DT)}, {"edge": 6})
    xr = x.clone().requires_grad_(True)
    (want,) = torch.autograd.grad(interp.apply_scalar(fn, xr).sum(), xr)
    assert torch.allclose(env[grads["x"]], want, atol=1e-12)


def test_envelope_is_twice_differentiable_at_the_cutoff():
    one = torch.tensor([1.0 - 1e-9, 1.0, 1.0 + 1e-9], dtype=DT)
    for order in (0, 1, 2):
        assert interp.apply_scalar("poly_envelope", one, order).abs().max().item() < 1e-6


def test_closure_check_fires():
    p, y = linear_prog()
    assert_closed(p)
    import dataclasses
    p.ops[y] = dataclasses.replace(p.ops[y], kind="reshape")
    with pytest.raises(ClosureError):
        assert_closed(p)


def test_cse_dce_are_exact():
    p, y = linear_prog()
    y2 = p.contract(["x", "w", "b"], p.ops[y].out_type, p.ops[y].paths)     # duplicate of y
    dead = p.scalar(y2, "exp")
    z = p.add(y, y2)
    p.outputs = (z,)
    q = simplify(p)
    assert len(cse(p).ops) == len(p.ops) - 1 and dead not in dce(p).ops
    assert len(q.ops) == 2 and op_stats(q)["ops"] == 2
    g = torch.Generator().manual_seed(2)
    ins = {"x": torch.randn(4, 4, generator=g, dtype=DT), "w": torch.randn(1, 3, 4, generator=g, dtype=DT),
           "b": torch.randn(1, 3, generator=g, dtype=DT)}
    a = interp.run(p, ins, {"edge": 4})[z]
    b = interp.run(q, ins, {"edge": 4})[q.outputs[0]]
    assert torch.equal(a, b)
