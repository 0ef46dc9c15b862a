"""GPU parity: the CUDA path (through the C ABI) against the golden vectors of the reference
and against the CPU oracle on seeded inputs.  Tolerance: 1e-5 relative L2 for fp32 outputs and
gradients; sort order, CSR offsets and index maps bit-exact."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import eso2_oracle as orc
from tests.conftest import golden_names, load_golden
from tests.helpers import (check_against, gpu_node_out_and_vjp, make_block,
                           oracle_node_out_and_vjp, random_case, rel_l2)

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.mark.parametrize("name", golden_names())
def test_golden_reference_vectors(name):
    c = load_golden(name)
    block = make_block(c["cfg"], c["params"])
    out = gpu_node_out_and_vjp(block, c, c["upstream"])
    check_against(*out, c["node_out"], c["vjp_x_node"], c["vjp_pos"], c["vjp_params"])
    # and the scalar E with its force through the reference call signature
    pos = c["pos"].cuda().float().requires_grad_(True)
    e = block(pos, c["atomic_numbers"].cuda(), c["x_node"].cuda().float(), c["edge_index"].cuda(),
              c["shifts"].cuda().float(), c["cos_gamma_k"].cuda().float(),
              c["sin_gamma_k"].cuda().float(), None)
    (f,) = torch.autograd.grad(e, pos)
    assert abs(e.item() - c["energy"].item()) < 1e-5 * max(1.0, abs(c["energy"].item()))
    assert rel_l2(f, c["de_dpos"]) < TOL


ORACLE_CASES = [
    # lmax, mmax, C, H, EC, NB, nodes, edges
    (4, 2, 8, 8, 8, 6, 12, 60),
    (6, 2, 8, 16, 4, 5, 9, 40),
    (3, 1, 24, 8, 8, 4, 7, 33),
    (2, 2, 32, 32, 32, 32, 20, 150),
    (5, 3, 16, 8, 4, 4, 6, 25),
    (1, 0, 8, 8, 4, 4, 5, 12),
    (4, 2, 128, 128, 32, 16, 40, 300),
]


@pytest.mark.parametrize("scale", [1.0, 1e-4, 30.0])
@pytest.mark.parametrize("lmax,mmax,c,h,ec,nb,n,e", ORACLE_CASES[:4] + ORACLE_CASES[-1:])
def test_oracle_parity_bf16x3_and_scaled_inputs(lmax, mmax, c, h, ec, nb, n, e, scale, jd64):
    """Both fp32-accurate operand formats (two scaled fp16 terms = the default, three bf16 terms)
    hold the fp32 tolerance, also when embeddings and upstream gradient are far from unit
    magnitude (the fp16 scales are derived from device-side magnitude bounds)."""
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=ec,
               num_distance_basis=nb, cutoff=5.0)
    params = orc.init_params(cfg, seed=lmax * 10 + mmax)
    case = random_case(cfg, n, e, seed=100 + lmax)
    case["x_node"] = case["x_node"] * scale
    case["upstream"] = case["upstream"] / scale
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    for precision in ("fp32", "fp32_bf16x3"):
        block = make_block(cfg, params, precision=precision)
        got = gpu_node_out_and_vjp(block, case, case["upstream"])
        check_against(*got, *want)
        assert block.plan("cuda").device_status() == 0


@pytest.mark.parametrize("lmax,mmax,c,h,ec,nb,n,e", ORACLE_CASES)
def test_oracle_parity_small(lmax, mmax, c, h, ec, nb, n, e, jd64):
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=ec,
               num_distance_basis=nb, cutoff=5.0)
    params = orc.init_params(cfg, seed=lmax * 10 + mmax)
    case = random_case(cfg, n, e, seed=100 + lmax)
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    got = gpu_node_out_and_vjp(make_block(cfg, params), case, case["upstream"])
    check_against(*got, *want)


@pytest.mark.parametrize("lmax,mmax,c,h,n,e", [(4, 2, 32, 32, 16, 120), (2, 2, 64, 32, 12, 80)])
def test_bf16_operands_fp32_accumulate(lmax, mmax, c, h, n, e, jd64):
    """bf16 embeddings/weights in the SO(2) contraction, fp32 accumulation: 2e-2 relative L2."""
    cfg = dict(lmax=lmax, mmax=mmax, sphere_channels=c, hidden_channels=h, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=21)
    case = random_case(cfg, n, e, seed=22)
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    block = make_block(cfg, params, precision="bf16")
    got = gpu_node_out_and_vjp(block, case, case["upstream"])
    check_against(*got, *want, tol=2e-2)
    assert block.plan("cuda").device_status() == 0


def test_chunked_execution_matches(jd64, monkeypatch):
    """Graphs larger than the per-call edge budget run as destination-node chunks with the
    forward recomputed in the backward; results must not change beyond summation order."""
    from zippel_b200.blocks import eso2
    cfg = dict(lmax=4, mmax=2, sphere_channels=16, hidden_channels=8, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=31)
    case = random_case(cfg, 30, 400, seed=32)
    case["edge_index"][1, :90] = 11                      # one node above the budget on its own
    case["edge_index"][0, :90] = (torch.arange(90) % 29 + 12) % 30
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    block = make_block(cfg, params)
    monkeypatch.setattr(eso2, "MAX_EDGES_PER_CALL", 64)
    from zippel_b200.graph import EdgeGraph
    graph = EdgeGraph.build(case["edge_index"].cuda(), 30)
    pieces = graph.chunks(64)
    assert len(pieces) > 4 and pieces[0].n0 == 0 and pieces[-1].n1 == 30
    assert all(a.n1 == b.n0 and a.e1 == b.e0 for a, b in zip(pieces, pieces[1:]))
    got = gpu_node_out_and_vjp(block, case, case["upstream"])
    check_against(*got, *want)


def test_nodes_without_edges_and_empty_graph(jd64):
    cfg = dict(lmax=2, mmax=1, sphere_channels=8, hidden_channels=8, edge_channels=4,
               num_distance_basis=4, cutoff=5.0)
    params = orc.init_params(cfg, seed=3)
    block = make_block(cfg, params)
    case = random_case(cfg, 10, 6, seed=5)
    case["edge_index"][1] = torch.tensor([2, 2, 2, 7, 7, 2])     # ragged: most nodes empty
    case["edge_index"][0] = torch.tensor([0, 1, 3, 0, 9, 5])
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    got = gpu_node_out_and_vjp(block, case, case["upstream"])
    check_against(*got, *want)
    assert got[0][[0, 1, 3, 4, 5, 6, 8, 9]].abs().max().item() == 0.0
    # no edges at all: zero output, zero gradients
    empty = dict(case, edge_index=torch.zeros(2, 0, dtype=torch.long),
                 shifts=torch.zeros(0, 3, dtype=torch.float64),
                 cos_gamma_k=torch.zeros(0, 3, dtype=torch.float64),
                 sin_gamma_k=torch.zeros(0, 3, dtype=torch.float64))
    node_out, gx, gpos, pg = gpu_node_out_and_vjp(block, empty, case["upstream"])
    assert node_out.abs().max().item() == 0.0 and gx.abs().max().item() == 0.0
    assert pg["c1_m0.weight"].abs().max().item() == 0.0


def test_high_degree_node(jd64):
    """One destination with far more than 30 incoming edges (the reference applies no cap)."""
    cfg = dict(lmax=2, mmax=2, sphere_channels=8, hidden_channels=8, edge_channels=4,
               num_distance_basis=4, cutoff=6.0)
    params = orc.init_params(cfg, seed=8)
    case = random_case(cfg, 40, 300, seed=9)
    case["edge_index"][1, :200] = 17
    case["edge_index"][0, :200] = torch.arange(200) % 39
    case["edge_index"][0, :200][case["edge_index"][0, :200] >= 17] += 1
    want = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    got = gpu_node_out_and_vjp(make_block(cfg, params), case, case["upstream"])
    check_against(*got, *want)


@pytest.mark.parametrize("lmax,mmax", [(2, 2), (4, 2), (6, 2), (3, 3)])
def test_wigner_kernel_forward_backward(lmax, mmax, jd64):
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import Plan
    plan = Plan.get(lmax, mmax, 8, 8, "cuda")
    lib, s = _lib.load(), plan.sizes
    g = torch.Generator("cpu").manual_seed(lmax)
    e = 257
    ev = torch.randn(e, 3, generator=g, dtype=torch.float64)
    ev[0] = torch.tensor([0.0, 1.3, 0.0])            # on the pole: clamp path
    ev[1] = torch.tensor([1e-4, -2.0, 1e-4])
    gamma = torch.rand(e, generator=g, dtype=torch.float64) * 6.28
    cg, sg = orc.gamma_harmonics(gamma, lmax)
    ev32 = ev.float()
    evd = ev32.double().requires_grad_(True)          # oracle sees the same rounded inputs
    rot = orc.edge_rotation(evd, cg.float().double(), sg.float().double(), lmax, mmax, jd64)
    tabs = plan.tables()
    d_ev, d_cg, d_sg = ev32.cuda(), cg.float().cuda(), sg.float().cuda()
    out = torch.zeros(e, s.nnz_pad, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.zp_wigner_forward(plan.handle, e, d_ev.data_ptr(), d_cg.data_ptr(),
                                     d_sg.data_ptr(), out.data_ptr(), st), "fwd")
    dense = torch.zeros(e, s.Km, s.K, dtype=torch.float64)
    up = torch.randn(e, s.Km, s.K, generator=g, dtype=torch.float64)
    gpacked = torch.zeros(e, s.nnz_pad)
    mask = torch.zeros(s.Km, s.K, dtype=torch.float64)
    for r in range(s.Km):
        l, off = int(tabs["row_l"][r]), int(tabs["rot_off"][r])
        dense[:, r, l * l:(l + 1) ** 2] = out[:, off:off + 2 * l + 1].double().cpu()
        gpacked[:, off:off + 2 * l + 1] = up[:, r, l * l:(l + 1) ** 2].float()
        mask[r, l * l:(l + 1) ** 2] = 1.0
    assert (dense - rot.detach()).abs().max().item() < 2e-7
    (want,) = torch.autograd.grad((rot * up.float().double() * mask).sum(), evd)
    gev = torch.zeros(e, 3, device="cuda")
    d_g = gpacked.cuda()
    _lib.check(lib.zp_wigner_backward(plan.handle, e, d_ev.data_ptr(), d_cg.data_ptr(),
                                      d_sg.data_ptr(), d_g.data_ptr(), gev.data_ptr(), st), "bwd")
    # the two near-pole edges have huge, ill-conditioned derivatives; compare them separately
    assert rel_l2(gev[2:], want[2:]) < 1e-6
    assert rel_l2(gev[:2], want[:2]) < 1e-3


@pytest.mark.parametrize("n,e,seed", [(1, 0, 0), (5, 1, 1), (50, 1000, 2), (3000, 50000, 3),
                                      (7, 400, 4)])
def test_csr_build_bit_exact(n, e, seed):
    from zippel_b200.graph import EdgeGraph, csr_reference
    g = torch.Generator("cpu").manual_seed(seed)
    ei = torch.randint(0, n, (2, e), generator=g)
    want = csr_reference(ei.numpy(), n)
    got = EdgeGraph.build(ei.cuda(), n)
    for key in ("perm", "src", "dst", "row_ptr", "perm_src", "row_ptr_src"):
        assert np.array_equal(getattr(got, key).cpu().numpy(), want[key]), key


def test_csr_build_rejects_node_indices_out_of_range():
    """What torch indexing does for the reference (IndexError), without any out-of-range access."""
    from zippel_b200.graph import EdgeGraph
    ei = torch.tensor([[0, 1, 2, 5], [1, 2, 0, 1]], dtype=torch.int64, device="cuda")
    # free blocks of the caching allocator hold large values from here on: the sort's scratch and
    # outputs start from them, so a slot that an omitted edge leaves unwritten would show
    junk = torch.full((8 << 20,), 0x7F7F7F7F, dtype=torch.int32, device="cuda")
    del junk
    with pytest.raises(IndexError):
        EdgeGraph.build(ei, 5)                       # src 5 >= N
    ei[0, 3] = -1
    with pytest.raises(IndexError):
        EdgeGraph.build(ei, 5)
    # the arrays of a flagged sort still index inside [0, N) and [0, E) everywhere (a caller that
    # replays a recorded step never reads the flag): the omitted edge's slot is an edge 0 -> 0
    g = EdgeGraph.build(ei, 5, validate=False)
    assert g.row_ptr.cpu().tolist() == [0, 1, 2, 3, 3, 3]
    assert g.row_ptr_src.cpu().tolist() == [0, 2, 3, 4, 4, 4]
    assert g.src.cpu().tolist() == [2, 0, 1, 0] and g.dst.cpu().tolist() == [0, 1, 2, 0]
    assert g.perm.cpu().tolist() == [2, 0, 1, 0] and g.perm_src.cpu().tolist() == [1, 3, 2, 0]
    ei[0, 3] = 4
    assert EdgeGraph.build(ei, 5).row_ptr.cpu().tolist() == [0, 1, 3, 4, 4, 4]


def test_chunks_keep_leading_nodes_without_edges():
    """Edge-less nodes at the start, followed by a node above the budget: every row must be covered."""
    from zippel_b200.graph import EdgeGraph
    dst = torch.cat([torch.full((100,), 2), torch.full((20,), 3)])
    src = torch.arange(120) % 2
    graph = EdgeGraph.build(torch.stack([src, dst]).cuda(), 5)
    pieces = graph.chunks(10)
    assert pieces[0].n0 == 0 and pieces[-1].n1 == 5
    assert all(a.n1 == b.n0 and a.e1 == b.e0 for a, b in zip(pieces, pieces[1:]))
    assert sum(p.n_edges for p in pieces) == 120


def test_abi_rejects_bad_arguments():
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import Plan
    lib = _lib.load()
    cfg = _lib.ZpConfig(7, 2, 8, 8, 0)
    h = ctypes.c_void_p()
    jd = (ctypes.c_double * 4)()
    assert lib.zp_plan_create(ctypes.byref(cfg), jd, ctypes.byref(h)) == 2      # lmax too large
    cfg = _lib.ZpConfig(2, 3, 8, 8, 0)
    assert lib.zp_plan_create(ctypes.byref(cfg), jd, ctypes.byref(h)) == 2      # mmax > lmax
    cfg = _lib.ZpConfig(2, 2, 12, 8, 0)
    assert lib.zp_plan_create(ctypes.byref(cfg), jd, ctypes.byref(h)) == 2      # C % 8
    assert lib.zp_plan_create(None, jd, ctypes.byref(h)) == 1
    plan = Plan.get(2, 2, 8, 8, "cuda")
    assert lib.zp_workspace_bytes(plan.handle, 4, -1, 0) == 0
    assert lib.zp_wigner_forward(plan.handle, 5, None, None, None, None, None) == 1


def test_ir_program_dispatch(jd64):
    """compile_program / allocate / run_program on the force program: kernels vs FP64 interpreter."""
    from oracle import ir_interp as interp
    from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
    from zippel_b200.blocks.eso2_ir import build_force
    from zippel_b200.blocks.ir_bind import bind
    from zippel_b200.codegen.compose import UnsupportedProgram, allocate, compile_program, run_program
    cfg = dict(lmax=4, mmax=2, sphere_channels=16, hidden_channels=8, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=51)
    block = ESO2Block(BlockConfig(**cfg)).double()
    block.load_state_dict(params)
    case = random_case(cfg, 14, 90, seed=52)
    prog, meta = build_force(BlockConfig(**cfg), block.gauss_coeff)
    inputs, sizes = bind(block, case, jd64)
    inputs["seed_E"] = torch.ones(1, dtype=torch.float64)
    want = interp.run(prog, inputs, sizes)
    cp = compile_program(prog, sizes, label="force")
    assert cp.kind == "force" and cp.cfg.lmax == 4 and cp.cfg.mmax == 2 and cp.cfg.cutoff == 5.0
    env = run_program(cp, allocate(cp, inputs))
    e_want = want[meta["energy"]].item()
    assert abs(env[meta["energy"]].item() - e_want) < 1e-5 * max(1.0, abs(e_want))
    assert rel_l2(env[meta["force"]], want[meta["force"]]) < TOL
    assert rel_l2(env[meta["node_out"]], want[meta["node_out"]]) < TOL
    # anything that is not the block program is refused
    other, _ = build_force(BlockConfig(**cfg), block.gauss_coeff)
    other.scale(meta["energy"], 2.0)
    with pytest.raises(UnsupportedProgram):
        compile_program(other, sizes)


def test_streamed_vjp_without_recompute(monkeypatch):
    """`node_output_vjp` (chunk forward, then at once chunk backward) against `node_output` +
    autograd, for a fixed upstream tensor and for a per-row callable (loss = sum node_out^2)."""
    from zippel_b200.blocks import eso2
    from zippel_b200.graph import EdgeGraph
    cfg = dict(lmax=3, mmax=2, sphere_channels=16, hidden_channels=8, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=41)
    case = random_case(cfg, 60, 3000, seed=42)
    block = make_block(cfg, params)
    dev = "cuda"
    args = [case["pos"].to(dev, torch.float32), case["atomic_numbers"].to(dev),
            case["x_node"].to(dev, torch.float32), case["edge_index"].to(dev),
            case["shifts"].to(dev, torch.float32), case["cos_gamma_k"].to(dev, torch.float32),
            case["sin_gamma_k"].to(dev, torch.float32)]
    up = case["upstream"].to(dev, torch.float32)

    def reference(loss_fn):
        pos, x = args[0].clone().requires_grad_(True), args[2].clone().requires_grad_(True)
        out = block.node_output(pos, args[1], x, *args[3:])
        grads = torch.autograd.grad(loss_fn(out), [x, pos, *block.parameters()], allow_unused=True)
        return out.detach(), grads

    want_t, grads_t = reference(lambda o: (o * up).sum())
    want_c, grads_c = reference(lambda o: (o * o).sum())

    monkeypatch.setattr(eso2, "MAX_EDGES_PER_CALL", 2048)      # module-level pieces of <= 1024 edges
    # Free blocks of the caching allocator hold huge values from here on: a magnitude scan that
    # strays beyond the rows a chunk call holds would pick them up and flush the operands to zero.
    junk = torch.full((32 << 20,), 1e30, device=dev)
    del junk
    graph = EdgeGraph.build(args[3], 60)
    assert len(graph.chunks(1024)) >= 3
    for upstream, want, grads in ((up, want_t, grads_t),
                                  (lambda rows, n0, n1: 2.0 * rows, want_c, grads_c)):
        out, gx, gpos, gp = block.node_output_vjp(*args, upstream, graph=graph)
        assert rel_l2(out, want) < 1e-5
        assert rel_l2(gx, grads[0]) < 1e-5 and rel_l2(gpos, grads[1]) < 1e-5
        for got_p, want_p, (name, _) in zip(gp, grads[2:], block.named_parameters()):
            if want_p is None:
                assert got_p is None, name
            else:
                assert rel_l2(got_p, want_p) < 1e-5, name


def test_runner_with_the_last_radial_layer_inside_the_call():
    """`EdgeConvRunner` with `edge_channels` set takes the hidden activations of the radial MLP and
    the last layer's parameters; results equal the runner fed with `radial` = that layer applied
    by torch, and the extra gradients equal the layer's VJP of `grad_radial`."""
    from zippel_b200.graph import EdgeGraph
    from zippel_b200.runner import EdgeConvRunner
    cfg = dict(lmax=4, mmax=2, sphere_channels=32, hidden_channels=32, edge_channels=32,
               num_distance_basis=16, cutoff=5.0)
    params = orc.init_params(cfg, seed=51)
    case = random_case(cfg, 40, 900, seed=52)
    block = make_block(cfg, params)
    dev = torch.device("cuda")
    graph = EdgeGraph.build(case["edge_index"].to(dev), 40)
    e, r = 900, block.plan(dev).sizes.R
    g = torch.Generator().manual_seed(53)
    f32 = lambda t: t.to(dev, torch.float32).contiguous()                      # noqa: E731
    perm = graph.perm64
    pos = f32(case["pos"])
    ev = (pos[graph.dst.long()] - pos[graph.src.long()] + f32(case["shifts"])[perm]).contiguous()
    cg, sg = f32(case["cos_gamma_k"])[perm].contiguous(), f32(case["sin_gamma_k"])[perm].contiguous()
    h_rad = f32(torch.randn(e, 32, generator=g))
    rw, rb = f32(torch.randn(r, 32, generator=g) * 0.2), f32(torch.randn(r, generator=g) * 0.1)
    env = f32(torch.rand(e, generator=g))
    radial = (h_rad @ rw.T + rb).contiguous()
    up = f32(case["upstream"])
    w = (block.c1_m0.weight.detach(), block.c1_m0.bias.detach(),
         [l.weight.detach() for l in block.c1_m], block.c2_m0.weight.detach(),
         block.c2_m0.bias.detach(), [l.weight.detach() for l in block.c2_m])
    a = EdgeConvRunner(block.plan(dev), graph)
    a.bind(f32(case["x_node"]), ev, cg, sg, radial, env, *w)
    out_a = a.forward().clone()
    gx_a, gev_a, grad_a, genv_a, gw_a = a.backward(up)
    b = EdgeConvRunner(block.plan(dev), graph, edge_channels=32)
    b.bind(f32(case["x_node"]), ev, cg, sg, h_rad, env, *w, rad_layer=(rw, rb))
    out_b = b.forward().clone()
    gx_b, gev_b, gh_b, genv_b, gw_b = b.backward(up)
    assert rel_l2(out_b, out_a) < 1e-5
    assert rel_l2(gx_b, gx_a) < 1e-5 and rel_l2(gev_b, gev_a) < 1e-5 and rel_l2(genv_b, genv_a) < 1e-5
    assert rel_l2(gw_b[0], gw_a[0]) < 1e-5 and rel_l2(gw_b[2][1], gw_a[2][1]) < 1e-5
    assert rel_l2(gh_b, grad_a @ rw) < 1e-5
    assert rel_l2(b.grad_rad_w, grad_a.T @ h_rad) < 1e-5
    assert rel_l2(b.grad_rad_b, grad_a.sum(0)) < 1e-5
    with pytest.raises(ValueError):
        a.bind(f32(case["x_node"]), ev, cg, sg, radial, env, *w, rad_layer=(rw, rb))
    # frozen parameters (gw = NULL): the other gradients are the same numbers, the weight-gradient
    # buffers are not touched
    for run, ref in ((a, (gx_a, gev_a, grad_a, genv_a)), (b, (gx_b, gev_b, gh_b, genv_b))):
        ref = [t.clone() for t in ref]
        run.grad_w_flat.fill_(7.0)
        run.forward()
        got = run.backward(up, weight_grads=False)
        for g_, r_ in zip(got[:4], ref):
            assert torch.equal(g_, r_)
        assert bool((run.grad_w_flat == 7.0).all())
        run.grad_x.fill_(7.0)                  # no gradient of x_node either
        got = run.backward(up, weight_grads=False, x_grad=False)
        for g_, r_ in zip(got[1:4], ref[1:]):
            assert torch.equal(g_, r_)
        assert bool((run.grad_x == 7.0).all())


def test_frozen_parameters_give_the_same_forces(jd64, monkeypatch):
    """With `requires_grad_(False)` on the block the backward skips every parameter-gradient
    product (SO(2) weights, radial MLP, readout); E and dE/dpos do not change."""
    cfg = dict(lmax=3, mmax=2, sphere_channels=16, hidden_channels=16, edge_channels=16,
               num_distance_basis=8, cutoff=5.0)
    params = orc.init_params(cfg, seed=61)
    case = random_case(cfg, 30, 500, seed=62)
    block = make_block(cfg, params)
    dev = "cuda"
    args = [case["atomic_numbers"].to(dev), case["x_node"].to(dev, torch.float32),
            case["edge_index"].to(dev), case["shifts"].to(dev, torch.float32),
            case["cos_gamma_k"].to(dev, torch.float32), case["sin_gamma_k"].to(dev, torch.float32)]

    def energy_and_forces(x_grad: bool):
        pos = case["pos"].to(dev, torch.float32).requires_grad_(True)
        x = args[1].clone().requires_grad_(x_grad)
        e = block(pos, args[0], x, *args[2:])
        de = torch.autograd.grad(e, [pos, x] if x_grad else [pos])[0]
        return e.detach(), de

    e0, f0 = energy_and_forces(True)           # every gradient formed
    block.requires_grad_(False)
    e1, f1 = energy_and_forces(True)           # frozen parameters
    e2, f2 = energy_and_forces(False)          # ... and embeddings without a gradient
    from zippel_b200.blocks import eso2
    monkeypatch.setattr(eso2, "MAX_EDGES_PER_CALL", 256)       # the same in destination chunks
    e3, f3 = energy_and_forces(False)
    e4, f4 = energy_and_forces(True)
    block.requires_grad_(True)
    assert torch.equal(e0, e1) and torch.equal(e0, e2)
    assert rel_l2(f1, f0) < 1e-6 and rel_l2(f2, f0) < 1e-6
    assert rel_l2(e3, e0) < 1e-6 and rel_l2(f3, f0) < 1e-5 and rel_l2(f4, f0) < 1e-5
