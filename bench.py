"""Benchmark of the eSEN SO(2) edge-convolution block (forward + first-order VJP).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step" = one forward + VJP pass of the block over one batch): a periodic cube
of 2 000 atoms at 0.1 atoms/A^3, 6 A cutoff, 30 nearest incoming neighbours per atom
(60 000 directed edges), lmax 4 / mmax 2 / C = H = EC = 128, 64 Gaussian RBFs, fp32,
gradients w.r.t. node embeddings, positions (through the Wigner-D derivative, the radial MLP
and the envelope) and the SO(2) weights, upstream gradient ~ N(0,1).  Data are seeded
synthetic tensors of those shapes; weights are Xavier-uniform.  With N > 1 every rank runs its
own independent structure of that size (weak scaling, no data-path exchange) and the SO(2)
weight gradients are all-reduced once per step.

The line printed by rank 0 carries
    value      edges/s of the kernel path with everything resident in HBM (C ABI forward +
               backward; radial features and envelope precomputed, CSR built beforehand)
    e2e        edges/s through the public module API from pinned HOST buffers: host->device
               copies, CSR build, radial MLP, forward, autograd backward, device->host read,
               recorded once as a CUDA graph (CapturedStep) and replayed per step; `e2e_eager`
               is the same step enqueued from Python every time
    radial_in_call  the resident step again with the last radial layer (EC -> R) inside the call
    roofline   the dominant kernel class, timed live with CUDA events inside the library
    kernels    per kernel class: ms, launches and share of the step; the HBM-bound classes also
               carry their algorithmic bytes, GB/s and fraction of the measured copy bandwidth
    cpu_baseline  the CPU oracle timed on this machine's host cores on a bounded sample
`--impl reference` times the reference algorithm's CPU restatement (the oracle) instead.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

CFG = dict(lmax=4, mmax=2, sphere_channels=128, hidden_channels=128, edge_channels=128,
           num_distance_basis=64, cutoff=6.0)
N_ATOMS, MAX_NEIGHBORS, DENSITY = 2000, 30, 0.1
METRIC = "edges/s per eSEN SO(2) block fwd+bwd (lmax4,C128)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def gemm_macs_per_edge(cfg) -> int:
    """Multiply-adds of the six SO(2) contractions for one edge (folded form = reference form)."""
    L, M, C, H = cfg["lmax"], cfg["mmax"], cfg["sphere_channels"], cfg["hidden_channels"]
    total = (L + 1) * 2 * C * (H * (L + 1) + L * H) + (L + 1) * H * C * (L + 1)
    for m in range(1, M + 1):
        km = L + 1 - m
        total += (2 * km * 2 * C) * (2 * km * H) + (2 * km * H) * (2 * km * C)
    return total


def hbm_bytes_per_step(block, n: int, e: int) -> dict:
    """Algorithmic bytes one step moves in each HBM-bound kernel class (timing class names of the
    library): fp32 arrays 4 bytes per value, 16-bit operand planes 2 bytes per value and plane."""
    c = block.cfg
    lay = block.layout
    K, Km = (c.lmax + 1) ** 2, lay.m_size[0] + 2 * sum(lay.m_size[1:])
    C, H, R = c.sphere_channels, c.hidden_channels, block.num_channels_rad
    w1 = c.lmax * H + Km * H                     # gate head + rows of conv1's output
    P = {2: 2, 0: 3, 1: 1}[block.precision]      # planes per operand
    # with the opt-in fused epilogues (ZP_FUSED_EPILOGUE=1, one- and two-plane formats) the gate
    # activation and the rotation back run inside the contractions; what is left of the scatter is
    # the sum of the per-row partial sums (one slab of nnz x C values per node and per 32-edge block)
    fused = P != 3 and os.environ.get("ZP_FUSED_EPILOGUE", "0") == "1"
    nnz = sum((2 * min(l, c.mmax) + 1) * (2 * l + 1) for l in range(c.lmax + 1))
    per_edge = {
        "rotate_in": R * 4 + Km * 2 * C * 2 * P,
        **({} if fused else {"gate_fwd": w1 * 4 + Km * H * 2 * P}),
        "rotate_back_scatter": nnz * C * 4 / 32 if fused else Km * C * 4,
        "rotate_grad_out": Km * C * 4 + Km * C * 2 * P,
        "gate_bwd": w1 * 4 + Km * H * 4 + w1 * 2 * P,
        "rotate_in_bwd": Km * 2 * C * 4 + 2 * R * 4 + 2 * K * C * 4,
        "src_reduce": 2 * K * C * 4,
    }
    per_node = {"rotate_back_scatter": K * C * 4 + (nnz * C * 4 if fused else 0),
                "src_reduce": K * C * 4}
    return {k: int(e * v + n * per_node.get(k, 0)) for k, v in per_edge.items()}


def xavier_(block, seed: int) -> None:
    g = torch.Generator("cpu").manual_seed(seed)
    with torch.no_grad():
        for name, p in block.named_parameters():
            if p.dim() == 2 and not name.startswith("elem_emb"):
                bound = (6.0 / (p.shape[0] + p.shape[1])) ** 0.5
                p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * bound)
                if name.startswith(("c1_m.", "c2_m.")):
                    p.mul_(2 ** -0.5)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        try:
            rows = [r.split(",") for r in open(self.path).read().strip().splitlines() if r]
            os.unlink(self.path)
        except Exception:
            return out
        sm, reasons = [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            try:
                sm.append(float(r[0])); out["sm_max_mhz"] = float(r[1])
            except Exception:
                continue
            for nm, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(nm)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
        out["reasons"], out["samples"] = sorted(reasons), len(sm)
        return out


def make_workload(seed: int, n_atoms: int = N_ATOMS):
    from zippel_b200.graph import synthetic_batch
    batch = synthetic_batch(n_atoms, CFG["lmax"], CFG["sphere_channels"], CFG["cutoff"],
                            density=DENSITY, max_neighbors=MAX_NEIGHBORS, seed=seed)
    g = torch.Generator("cpu").manual_seed(seed + 7)
    batch["upstream"] = torch.randn(batch["x_node"].shape, generator=g)
    return batch


# ------------------------------------------------------------------------------------------
# CPU leg (oracle): used for cpu_baseline and for --impl reference
# ------------------------------------------------------------------------------------------

def cpu_step_factory(batch, sample_nodes: int, threads: int):
    """Forward + VJP of the oracle on the edges into the first `sample_nodes` atoms."""
    from oracle import eso2_oracle as orc
    torch.set_num_threads(threads)
    params = orc.init_params(CFG, seed=0, dtype=torch.float32)
    jd = orc.load_jd(ROOT / "zippel_b200" / "data" / "jd.npz", CFG["lmax"])
    ei = batch["edge_index"]
    keep = ei[1] < sample_nodes
    ei_s = ei[:, keep]
    shifts, cg, sg = batch["shifts"][keep], batch["cos_gamma_k"][keep], batch["sin_gamma_k"][keep]
    so2 = [k for k in params if k.startswith(("c1_", "c2_"))]

    def step():
        pos = batch["pos"].clone().requires_grad_(True)
        x = batch["x_node"].clone().requires_grad_(True)
        p = {k: (v.clone().requires_grad_(True) if k in so2 else v) for k, v in params.items()}
        out = orc.block_node_out(p, CFG, pos, batch["atomic_numbers"], x, ei_s, shifts, cg, sg, jd)
        torch.autograd.grad((out * batch["upstream"]).sum(), [x, pos, *[p[k] for k in so2]])

    return step, int(keep.sum())


def interp_baseline(threads: int) -> dict:
    """The second CPU comparator: the FP64 IR interpreter (the reference's zippel/interp.py:135 run,
    restated under oracle/) evaluating the force program -- energy and F = -dE/dpos -- on the
    CPU-runnable configuration: 64 atoms in a 10 A cube, 5 A cutoff, lmax 2, C 32."""
    from oracle import eso2_oracle as orc
    from oracle import ir_interp as interp
    from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
    from zippel_b200.blocks.eso2_ir import build_force
    from zippel_b200.blocks.ir_bind import bind
    from zippel_b200.graph import synthetic_batch
    torch.set_num_threads(threads)
    cfg = dict(lmax=2, mmax=2, sphere_channels=32, hidden_channels=32, edge_channels=32,
               num_distance_basis=32, cutoff=5.0)
    batch = synthetic_batch(64, 2, 32, 5.0, box=10.0, max_neighbors=None, seed=0, dtype=torch.float64)
    block = ESO2Block(BlockConfig(**cfg)).double()
    jd = orc.load_jd(ROOT / "zippel_b200" / "data" / "jd.npz", 2)
    prog, _meta = build_force(BlockConfig(**cfg), block.gauss_coeff)
    inputs, sizes = bind(block, batch, jd)
    inputs["seed_E"] = torch.ones(1, dtype=torch.float64)
    interp.run(prog, inputs, sizes)
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        interp.run(prog, inputs, sizes)
        times.append(time.perf_counter() - t0)
    dt, e = statistics.median(times), batch["meta"]["n_edges"]
    return {"value": e / dt, "unit": "edges/s", "cores": threads, "kind": "port",
            "sample": f"IR interpreter, force program (E and dE/dpos), FP64, {e} edges, median of 3 "
                      "runs after 1 warm-up"}


def run_reference(args) -> dict:
    threads = os.cpu_count() or 1
    batch = make_workload(0, args.atoms)
    step, n_edges = cpu_step_factory(batch, args.cpu_sample_nodes, threads)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = n_edges / dt
    sample = (f"edges into the first {args.cpu_sample_nodes} of {N_ATOMS} atoms "
              f"({n_edges} of {batch['meta']['n_edges']} edges) per step, fp32 torch CPU")
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(batch),
        "notes": {"l2": "host cores only"},
        "cpu_baseline": {"value": val, "unit": "edges/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": "edges/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def workload_config(batch) -> dict:
    """The same dict in both arms (what differs between them is said under `notes`)."""
    m = batch["meta"]
    return {"workload": f"eSEN SO(2) block fwd+VJP, {m['n_atoms']} atoms periodic cube 0.1/A^3, 6 A cutoff, "
                        "30 neighbours, lmax4 mmax2 C128 H128 EC128 64 RBF, fp32",
            "atoms_per_gpu": m["n_atoms"], "edges_per_gpu": m["n_edges"], "lmax": CFG["lmax"],
            "mmax": CFG["mmax"], "channels": CFG["sphere_channels"]}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

def run_ours(args) -> dict | None:
    import torch.distributed as dist

    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
    from zippel_b200.graph import EdgeGraph
    from zippel_b200.partition import all_reduce_grads
    from zippel_b200.runner import EdgeConvRunner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    batch = make_workload(rank, args.atoms)
    n, e = batch["meta"]["n_atoms"], batch["meta"]["n_edges"]
    block = ESO2Block(BlockConfig(**CFG), precision=args.precision)
    xavier_(block, 0)
    block = block.to(dev)
    so2_params = [block.c1_m0.weight, block.c1_m0.bias, *[l.weight for l in block.c1_m],
                  block.c2_m0.weight, block.c2_m0.bias, *[l.weight for l in block.c2_m]]

    # ---- resident inputs for the kernel-path timing ----------------------------------------
    d = {k: v.to(dev) for k, v in batch.items() if torch.is_tensor(v)}
    graph = EdgeGraph.build(d["edge_index"], n)
    with torch.no_grad():
        perm, src, dst = graph.perm64, graph.src.long(), graph.dst.long()
        edge_vec = (d["pos"][dst] - d["pos"][src] + d["shifts"][perm]).contiguous()
        dist_e = edge_vec.pow(2).sum(-1).clamp_min(1e-24).sqrt()
        x_edge = torch.cat([block.gaussian_basis(dist_e), block.elem_emb(d["atomic_numbers"][src]),
                            block.elem_emb(d["atomic_numbers"][dst])], dim=-1)
        radial = block.rad_func(x_edge).contiguous()
        env = block.envelope(dist_e / CFG["cutoff"]).contiguous()
        cg, sg = d["cos_gamma_k"][perm].contiguous(), d["sin_gamma_k"][perm].contiguous()
    runner = EdgeConvRunner(block.plan(dev), graph, with_backward=True)
    runner.bind(d["x_node"].contiguous(), edge_vec, cg, sg, radial, env,
                block.c1_m0.weight.detach(), block.c1_m0.bias.detach(),
                [l.weight.detach() for l in block.c1_m], block.c2_m0.weight.detach(),
                block.c2_m0.bias.detach(), [l.weight.detach() for l in block.c2_m])
    upstream = d["upstream"].contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def kernel_step():
        runner.forward()
        runner.backward(upstream)
        if world > 1:          # every weight gradient is a view of this one buffer
            dist.all_reduce(runner.grad_w_flat, op=dist.ReduceOp.SUM)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        kernel_step()
    barrier()
    ev = [(torch.cuda.Event(True), torch.cuda.Event(True)) for _ in range(args.steps)]
    clocks = ClockSampler(local)
    clocks.__enter__()                  # sampled through the timed kernel region AND the e2e region
    if True:
        barrier()
        t_wall = time.perf_counter()
        for a, b in ev:
            flush.zero_()                       # evict L2 between steps (not inside the events)
            a.record()
            kernel_step()
            b.record()
        barrier()
        t_wall = time.perf_counter() - t_wall
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = total_ms.item() / args.steps
    # per-kernel-class times: a second pass with the library's timer on, which puts every launch
    # on one stream (the timed pass above lets independent launches share the device, so the
    # classes there overlap); shares and per-class rates come from this pass
    runner.timing(True)
    runner.read_timing()
    for _ in range(args.steps):
        flush.zero_()
        kernel_step()
    torch.cuda.synchronize()
    timing = runner.read_timing()
    runner.timing(False)

    # forward-only timing (same resident inputs)
    fa, fb = torch.cuda.Event(True), torch.cuda.Event(True)
    barrier()
    fwd_ms = 0.0
    for _ in range(args.steps):
        flush.zero_()
        fa.record(); runner.forward(); fb.record()
        fb.synchronize()
        fwd_ms += fa.elapsed_time(fb)
    fwd_ms /= args.steps

    # the same resident step with the LAST radial layer (EC -> R) inside the call: the op takes the
    # 128-wide hidden activations and that layer's parameters instead of `radial` [E, R]
    with torch.no_grad():
        h_rad = block.rad_func[:-1](x_edge).contiguous()
    last = block.rad_func[-1]
    runner_r = EdgeConvRunner(block.plan(dev), graph, with_backward=True,
                              edge_channels=CFG["edge_channels"])
    runner_r.bind(d["x_node"].contiguous(), edge_vec, cg, sg, h_rad, env,
                  block.c1_m0.weight.detach(), block.c1_m0.bias.detach(),
                  [l.weight.detach() for l in block.c1_m], block.c2_m0.weight.detach(),
                  block.c2_m0.bias.detach(), [l.weight.detach() for l in block.c2_m],
                  rad_layer=(last.weight.detach().contiguous(), last.bias.detach().contiguous()))
    for _ in range(3):
        runner_r.forward(); runner_r.backward(upstream)
    ra, rb = torch.cuda.Event(True), torch.cuda.Event(True)
    barrier()
    rad_ms = 0.0
    for _ in range(args.steps):
        flush.zero_()
        ra.record(); runner_r.forward(); runner_r.backward(upstream); rb.record()
        rb.synchronize()
        rad_ms += ra.elapsed_time(rb)
    rad_ms /= args.steps
    del runner_r, h_rad
    # ... and with frozen parameters (a force evaluation: gradients w.r.t. x_node and positions only)
    barrier()
    frozen_ms = 0.0
    for i in range(3 + args.steps):
        flush.zero_()
        ra.record(); runner.forward(); runner.backward(upstream, weight_grads=False); rb.record()
        rb.synchronize()
        if i >= 3:
            frozen_ms += ra.elapsed_time(rb)
    frozen_ms /= args.steps

    # ---- end to end through the module API from pinned host memory -------------------------
    host = {k: batch[k].pin_memory() for k in ("pos", "x_node", "edge_index", "shifts",
                                               "cos_gamma_k", "sin_gamma_k", "atomic_numbers",
                                               "upstream")}
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    out_host = torch.empty(n, 3, pin_memory=True)
    loss_host = torch.empty((), pin_memory=True)
    d2h = out_host.numel() * 4 + 4

    copy_stream = torch.cuda.Stream(dev)

    def e2e_step():
        # the two [N, K, C] arrays travel on a second stream beside the edge sort, the front end
        # and the radial MLP (x_node) and beside the forward (the upstream gradient); their
        # device buffers are allocated on the compute stream, which also outlives their use
        main = torch.cuda.current_stream(dev)
        big = ("x_node", "upstream")
        t = {k: v.to(dev, non_blocking=True) for k, v in host.items() if k not in big}
        ready = {}
        for k in big:
            t[k] = torch.empty(host[k].shape, dtype=host[k].dtype, device=dev)
        copy_stream.wait_stream(main)
        with torch.cuda.stream(copy_stream):
            for k in big:
                t[k].copy_(host[k], non_blocking=True)
                ready[k] = torch.cuda.Event()
                ready[k].record(copy_stream)
        pos = t["pos"].requires_grad_(True)
        x = t["x_node"].requires_grad_(True)
        node_out = block.node_output(pos, t["atomic_numbers"], x, t["edge_index"], t["shifts"],
                                     t["cos_gamma_k"], t["sin_gamma_k"], x_ready=ready["x_node"])
        main.wait_event(ready["upstream"])
        loss = (node_out * t["upstream"]).sum()
        grads = torch.autograd.grad(loss, [x, pos, *block.parameters()], allow_unused=True)
        if world > 1:
            all_reduce_grads([g for g, p in zip(grads[2:], block.parameters())
                              if g is not None and any(p is q for q in so2_params)])
        out_host.copy_(grads[1], non_blocking=True)
        loss_host.copy_(loss.detach(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def time_e2e(fn) -> float:
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        barrier()
        return (time.perf_counter() - t0) / args.steps

    e2e_eager_s = time_e2e(e2e_step) if not args.no_e2e else float("nan")

    # the same step recorded once as a CUDA graph (zippel_b200.captured.CapturedStep): pinned
    # host inputs -> device, edge sort, front end, radial MLP, edge convolution, VJP, results
    # back to pinned host memory (the benchmark replays the same host inputs every step)
    from zippel_b200.captured import CapturedStep
    e2e_path = ("zippel_b200.captured.CapturedStep.run: the module forward + VJP from pinned host "
                "inputs to pinned host results, replayed as one CUDA graph")
    try:
        if args.no_e2e:
            raise RuntimeError("--no-e2e")
        cap = CapturedStep(block, batch, dev)
    except RuntimeError as err:                 # recording refused: report the eager path
        cap, e2e_path = None, f"eager module path (recording failed: {str(err)[:120]})"
        print(f"bench: CapturedStep failed, e2e falls back to the eager path: {err}",
              file=sys.stderr)
    if cap is not None:
        cap_grads = [cap.grads["params"][n_] for n_, p in block.named_parameters()
                     if any(p is q for q in so2_params)]

        def e2e_captured():
            cap.run(sync=False)
            if world > 1:
                all_reduce_grads(cap_grads)
            torch.cuda.current_stream().synchronize()

        e2e_s = torch.tensor([time_e2e(e2e_captured)], dtype=torch.float64, device=dev)
        assert cap.h2d_bytes == h2d and cap.d2h_bytes == d2h
    else:
        e2e_s = torch.tensor([e2e_eager_s], dtype=torch.float64, device=dev)
    clocks.__exit__(None, None, None)
    clk = clocks.summary()
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    total_edges = torch.tensor([e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_edges)
    total_edges = total_edges.item()

    # ---- roofline of the dominant kernel class ---------------------------------------------
    pk, pk_src = peaks()
    macs = gemm_macs_per_edge(CFG)
    total_kernel_ms = sum(v[0] for v in timing.values())
    kernels = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps,
                   "share": v[0] / total_kernel_ms if total_kernel_ms else 0.0}
               for k, v in timing.items() if v[1]}
    launches = sum(v[1] for v in timing.values()) / args.steps
    # HBM-side kernel classes: algorithmic bytes per step (each operand once; gathered node rows
    # come from L2 and are not counted) against the measured copy bandwidth
    for k, nbytes in hbm_bytes_per_step(block, n, e).items():
        if k in kernels and kernels[k]["ms_per_step"] > 0:
            gbs = nbytes / (kernels[k]["ms_per_step"] * 1e-3) / 1e9
            kernels[k]["hbm"] = {"algorithmic_bytes": nbytes, "gbs": gbs,
                                 "frac_of_measured_copy": gbs / peaks()[0]["hbm_gbs"]}
    # The dominant kernel is the tensor-core contraction: one kernel (gemm_tc_kernel) serving the
    # forward, input-gradient and weight-gradient products, 18 launches per step.
    gemm = [k for k in kernels if k.startswith("gemm")]
    gemm_ms = sum(kernels[k]["ms_per_step"] for k in gemm)
    gemm_launches = sum(kernels[k]["launches_per_step"] for k in gemm)
    gemm_share = sum(kernels[k]["share"] for k in gemm)
    flops_step = 3 * 2.0 * macs * e            # fwd, dgrad and wgrad each do the same MACs
    ach = flops_step / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    peak = pk["bf16_tflops_sustained"]
    passes = {"fp32": 3, "fp32_bf16x3": 6, "bf16": 1}[args.precision]   # tensor-core passes per product
    # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of three forward launches
    # captured by ncu on an 18 000-edge case of this configuration (fp32 precision), averaged
    # and scaled by edges (operand and output bytes grow in proportion to the edge count)
    traffic = 172.9e6 * (e / 18000.0) if args.precision == "fp32" and args.atoms == N_ATOMS else None
    roof = {"bound": "tensor",
            "kernel": "gemm_tc_pair_kernel / gemm_tc_kernel (fwd + dgrad + wgrad launches)",
            "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
            "traffic": traffic, "share_of_step": gemm_share,
            "peak_source": f"{pk_src} bf16 dense sustained (no fp32/tf32 peak is measured)",
            "ms_per_launch": gemm_ms / max(gemm_launches, 1), "launches_per_step": gemm_launches,
            "mma_passes": passes, "mma_tflops": ach * passes, "mma_frac": ach * passes / peak,
            "algorithmic_flops_per_launch": flops_step / max(gemm_launches, 1),
            "note": "achieved counts algorithmic FLOPs (2*MAC of the six per-m SO(2) products, "
                    "forward + two gradients) once; the operand format costs mma_passes 16-bit "
                    "tensor-core passes per product, so mma_tflops = mma_passes x achieved is "
                    "what the tensor pipe executes"}

    # whole-step bounds: streaming bytes (gathered node rows counted per edge, no reuse) against
    # the copy bandwidth, algorithmic FLOPs against the tensor peak; the larger time binds
    K = (CFG["lmax"] + 1) ** 2
    n_weights = sum(p.numel() for p in so2_params)
    bytes_fwd = (e * (2 * K * CFG["sphere_channels"] * 4 + 12 + 8 * (CFG["lmax"] + 1) + 8)
                 + n * K * CFG["sphere_channels"] * 4 + n_weights * 4)
    bytes_step = 2 * bytes_fwd + e * 12
    t_hbm = bytes_step / (pk["hbm_gbs"] * 1e9) * 1e3
    t_tensor = flops_step / (peak * 1e12) * 1e3
    roof["whole_step"] = {
        "streaming_bytes": bytes_step, "t_hbm_ms": t_hbm, "algorithmic_flops": flops_step,
        "t_tensor_ms": t_tensor, "binds": "tensor" if t_tensor >= t_hbm else "hbm",
        "frac_of_bound": max(t_hbm, t_tensor) / ms_per_step,
        "hbm_frac_streaming": bytes_step / (ms_per_step * 1e-3) / (pk["hbm_gbs"] * 1e9),
        "note": "t_tensor counts each product once at the bf16 peak; the fp32 operand format "
                "needs mma_passes passes, so frac_of_bound <= 1/mma_passes for the GEMM part"}
    q = statistics.quantiles(step_ms, n=4) if len(step_ms) >= 4 else [min(step_ms)] * 3

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": total_edges / (ms_per_step * 1e-3), "unit": "edges/s",
            "ms_per_step_median": q[1], "ms_per_step_iqr": q[2] - q[0],
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if args.precision == "bf16" else "f32",
            "precision": args.precision, "data": "synthetic",
            "config": workload_config(batch),
            "notes": {"l2": "256 MiB L2 flush between steps, outside the per-step events; "
                            "per-step activations are >5 GB",
                      "radial": "value: radial features and envelope are precomputed inputs of "
                                "the C-ABI step; e2e: computed inside the step (radial MLP on "
                                "the library's kernels)"},
            "fwd_only": {"value": e / (fwd_ms * 1e-3), "unit": "edges/s (this rank)",
                         "ms_per_step": fwd_ms},
            "radial_in_call": {"value": e / (rad_ms * 1e-3), "unit": "edges/s (this rank)",
                               "ms_per_step": rad_ms,
                               "what": "the resident step with the last radial layer (EC -> R) and "
                                       "its VJP inside the call (zp_eso2_forward_radial / "
                                       "zp_eso2_backward_radial); `value` has `radial` precomputed"},
            "frozen_parameters": {"value": e / (frozen_ms * 1e-3), "unit": "edges/s (this rank)",
                                  "ms_per_step": frozen_ms,
                                  "what": "forward + VJP w.r.t. x_node, edge vectors, radial "
                                          "features and envelope only (gw = NULL: no "
                                          "weight-gradient products), the force evaluation of an "
                                          "MD loop; not the headline workload"},
            "wall_ms_per_step_incl_flush": t_wall * 1e3 / args.steps,
            "roofline": roof, "kernels": kernels, "gpu_launches": launches,
            "e2e": {"value": total_edges / e2e_s.item(), "unit": "edges/s",
                    "ms_per_step": e2e_s.item() * 1e3, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h,
                    "path": e2e_path},
            "e2e_eager": {"ms_per_step": e2e_eager_s * 1e3,
                          "path": "ESO2Block.node_output + torch.autograd.grad, enqueued from "
                                  "Python every step (this rank)"},
            "clocks": clk,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            step, n_s = cpu_step_factory(batch, args.cpu_sample_nodes, threads)
            step()
            reps, times = 3, []
            for _ in range(reps):
                t0 = time.perf_counter()
                step()
                times.append(time.perf_counter() - t0)
            dt = statistics.median(times)
            line["cpu_baseline"] = {
                "value": n_s / dt, "unit": "edges/s", "cores": threads, "kind": "port",
                "sample": f"oracle fwd+VJP on the {n_s} edges into the first "
                          f"{args.cpu_sample_nodes} atoms, median of {reps} repetitions after 1 "
                          "warm-up",
                "interp_cfg0": interp_baseline(threads)}
    # ---- the two larger configurations, each in child processes of their own ----------------
    if not args.no_large and args.atoms == N_ATOMS:
        del runner, flush
        cap = cap_grads = None
        torch.cuda.empty_cache()
        legs = large_legs(args, world, rank)
        if line is not None:
            line.update(legs)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


def large_legs(args, world: int, rank: int) -> dict:
    """Runs `--workload cfg3` (512 structures of 200 atoms, bf16, strong scaling over the ranks) and
    `--workload cfg4` (one 200 000-atom graph at lmax 6, destination-range partition) for a few
    steps each.  Every rank starts one child process per leg; the children form a process group of
    their own on another port, so a failure or a timeout there costs the leg, never the headline
    line.  Returns {"cfg3": ..., "cfg4": ...} (the child's result line, or {"error": ...})."""
    out = {}
    here = str(pathlib.Path(__file__).resolve())
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    for i, (name, extra) in enumerate((
            ("cfg3", ["--structures", str(args.structures), "--steps", "2", "--warmup", "2"]),
            ("cfg4", ["--atoms", str(args.large_atoms), "--steps", "1" if world == 1 else "2",
                      "--warmup", "2"]))):
        # a rendezvous of the children's own: rank 0 of them opens the store on another port
        # (the launcher's "use the agent's store" switch must not reach them)
        env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC")}
        env["MASTER_PORT"] = str(1024 + (base_port + 101 * (i + 1) - 1024) % 64000)
        cmd = [sys.executable, here, "--workload", name, "--gpus", str(world), "--parity-nodes",
               str(args.parity_nodes), *extra]
        try:
            res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.large_timeout)
            lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
            if res.returncode == 0 and (lines or rank != 0):
                out[name] = json.loads(lines[-1]) if lines else None
            else:
                out[name] = {"error": f"exit {res.returncode}: {res.stderr.strip()[-300:]}"}
        except subprocess.TimeoutExpired:
            out[name] = {"error": f"no result within {args.large_timeout} s"}
    return out


# ------------------------------------------------------------------------------------------
# the larger benchmark configurations (not the headline line): batched structures, single graph
# ------------------------------------------------------------------------------------------

def make_large_inputs(workload: str, world: int, rank: int, dev, structures: int, atoms: int):
    """Seeded inputs of the two larger configurations, on the device.

    cfg3: `structures` independent 200-atom periodic cubes (block-diagonal batch), this rank's
    contiguous share.  cfg4: one periodic cube of `atoms` atoms, lmax 6; every rank draws the same
    positions and builds the neighbour list on its own device (zp_neighbors), then keeps the edges
    into its destination-node range."""
    from zippel_b200 import partition as part
    from zippel_b200.blocks.wigner import gamma_harmonics
    from zippel_b200.graph import neighbor_list, synthetic_batch

    cfg = dict(CFG)
    if workload == "cfg3":
        a, b = part.structure_ranges(structures, world)[rank]
        batch = synthetic_batch(200, cfg["lmax"], cfg["sphere_channels"], cfg["cutoff"],
                                density=DENSITY, max_neighbors=MAX_NEIGHBORS, n_structures=b - a,
                                seed=100 + rank)
        d = {k: v.to(dev) for k, v in batch.items() if torch.is_tensor(v)}
        g = torch.Generator("cpu").manual_seed(9 + rank)
        d["upstream"] = torch.randn(batch["x_node"].shape, generator=g).to(dev)
        return cfg, d, None
    cfg["lmax"] = 6
    k = (cfg["lmax"] + 1) ** 2
    box = float((atoms / DENSITY) ** (1.0 / 3.0))
    g = torch.Generator("cpu").manual_seed(5)
    pos = (torch.rand(atoms, 3, generator=g, dtype=torch.float64) * box).to(dev)
    edge_index, shifts, _ = neighbor_list(pos, box, cfg["cutoff"], MAX_NEIGHBORS)
    e = edge_index.shape[1]
    gd = torch.Generator(dev).manual_seed(6)          # the big arrays are drawn on the device
    gamma = torch.rand(e, generator=gd, device=dev, dtype=torch.float64) * 2 * torch.pi
    cos_g, sin_g = gamma_harmonics(gamma, cfg["lmax"])
    d = {"pos": pos.float(), "edge_index": edge_index, "shifts": shifts.float(),
         "cos_gamma_k": cos_g.float(), "sin_gamma_k": sin_g.float(),
         "atomic_numbers": torch.randint(1, 30, (atoms,), generator=gd, device=dev),
         "x_node": torch.randn(atoms, k, cfg["sphere_channels"], generator=gd, device=dev),
         "upstream": torch.randn(atoms, k, cfg["sphere_channels"], generator=gd, device=dev)}
    return cfg, d, part.node_ranges(atoms, world)


def sampled_parity(block, cfg: dict, pos, z, x_full, ei, sh, cg, sg, rows, row0: int, row1: int,
                   n_sample: int, seed: int) -> float:
    """Relative L2 of `n_sample` rows of node_out (`rows` = rows row0:row1) against the CPU oracle.
    A row depends on its node's incoming edges only, so the oracle runs on the small graph made of
    the sampled destinations, their incoming edges and those edges' sources (nodes renumbered)."""
    from oracle import eso2_oracle as orc
    g = torch.Generator("cpu").manual_seed(seed)
    nodes = (torch.randperm(row1 - row0, generator=g)[:n_sample] + row0).to(ei.device)
    keep = torch.isin(ei[1], nodes)
    e_sub = ei[:, keep]
    used, inverse = torch.unique(torch.cat([nodes, e_sub.reshape(-1)]), return_inverse=True)
    where, e_new = inverse[:nodes.numel()], inverse[nodes.numel():].reshape(2, -1)
    f64 = lambda t: t.detach().cpu().double()                 # noqa: E731
    params = {k: f64(v) for k, v in block.state_dict().items()}
    jd = orc.load_jd(ROOT / "zippel_b200" / "data" / "jd.npz", cfg["lmax"])
    want = orc.block_node_out(params, cfg, f64(pos[used]), z[used].cpu(), f64(x_full[used]),
                              e_new.cpu(), f64(sh[keep]), f64(cg[keep]), f64(sg[keep]), jd)[where.cpu()]
    got = f64(rows[nodes - row0])
    return ((got - want).norm() / want.norm().clamp_min(1e-300)).item()


def measure_large(workload: str, world: int, rank: int, dev, *, precision: str, structures: int,
                  atoms: int, steps: int, warmup: int, recompute: bool = False,
                  parity_nodes: int = 0) -> dict | None:
    """One of the two larger configurations inside an initialised process group (or alone).
    Returns the result dict on rank 0, None elsewhere."""
    import torch.distributed as dist

    from zippel_b200 import partition as part
    from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
    from zippel_b200.graph import EdgeGraph

    t_setup = time.perf_counter()
    cfg, d, nranges = make_large_inputs(workload, world, rank, dev, structures, atoms)
    block = ESO2Block(BlockConfig(**cfg), precision=precision)
    xavier_(block, 0)
    block = block.to(dev)
    n = d["pos"].shape[0]
    ei, sh, cg, sg = d["edge_index"], d["shifts"], d["cos_gamma_k"], d["sin_gamma_k"]
    x_in, up = d["x_node"], d["upstream"]
    partitioned = workload == "cfg4" and world > 1
    if partitioned:
        a, b = nranges[rank]
        keep = part.local_edges(ei, nranges[rank])
        ei, sh, cg, sg = ei[:, keep], sh[keep], cg[keep], sg[keep]
        x_in, up = x_in[a:b].clone(), up[a:b].clone()
    graph = EdgeGraph.build(ei, n)
    e_local = ei.shape[1]
    t_setup = time.perf_counter() - t_setup
    streamed = not recompute

    def step():
        if streamed and partitioned:
            out, gx, gpos, gp = part.partitioned_node_output_vjp(
                block, d["pos"], d["atomic_numbers"], x_in, ei, sh, cg, sg, up, nranges, rank,
                graph=graph)
            return out, gx, gpos, gp
        if streamed:
            # chunk forward, then at once chunk backward: no forward is computed twice
            out, gx, gpos, gp = block.node_output_vjp(d["pos"], d["atomic_numbers"], x_in, ei, sh,
                                                      cg, sg, up, graph=graph)
            if world > 1:
                part.all_reduce_grads([gpos, *[g_ for g_ in gp if g_ is not None]])
            return out, gx, gpos, gp
        pos = d["pos"].detach().requires_grad_(True)
        x = x_in.detach().requires_grad_(True)
        if partitioned:
            fn = lambda p_, z_, xf, e_, s_, c_, g_: block.node_output(p_, z_, xf, e_, s_, c_, g_, graph=graph)  # noqa: E731
            out = part.partitioned_node_output(fn, pos, d["atomic_numbers"], x, ei, sh, cg, sg, nranges, rank)
        else:
            out = block.node_output(pos, d["atomic_numbers"], x, ei, sh, cg, sg, graph=graph)
        grads = torch.autograd.grad((out * up).sum(), [x, pos, *block.parameters()], allow_unused=True)
        if world > 1:
            part.all_reduce_grads([grads[1], *[g_ for g_ in grads[2:] if g_ is not None]])
        return out.detach(), grads[0], grads[1], grads[2:]

    torch.cuda.reset_peak_memory_stats(dev)
    res = None
    for _ in range(max(warmup, 1)):
        res = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    marks = [torch.cuda.Event(True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        res = step()
        marks[i + 1].record()
    torch.cuda.synchronize()
    each = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]    # this rank's steps
    ms = torch.tensor([marks[0].elapsed_time(marks[-1]) / steps], dtype=torch.float64, device=dev)
    edges = torch.tensor([float(e_local)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(edges)
    chunks = max((len(v) for v in graph.__dict__.get("_chunk_cache", {}).values()), default=1)
    status = block.plan(dev).device_status()
    line = None
    if rank == 0:
        parity = None
        if parity_nodes:
            r0, r1 = nranges[0] if partitioned else (0, n)   # rank 0's rows; its edges hold all into them
            parity = sampled_parity(block, cfg, d["pos"], d["atomic_numbers"], d["x_node"], ei, sh, cg,
                                    sg, res[0], r0, r1, parity_nodes, seed=11)
        line = {"workload": workload, "value": edges.item() / (ms.item() * 1e-3), "unit": "edges/s",
                "n_gpus": world, "steps": steps, "ms_per_step": ms.item(), "ms_each_step_rank0": each,
                "precision": precision,
                "scaling": "strong",
                "config": {"atoms_total": n if workload == "cfg4" else 200 * structures,
                           "edges_total": edges.item(), "lmax": cfg["lmax"], "mmax": cfg["mmax"],
                           "channels": cfg["sphere_channels"], "chunks_per_rank": chunks,
                           "path": ("ESO2Block.node_output_vjp, inputs resident: per destination "
                                    "chunk the forward and at once the backward, no recompute"
                                    if streamed else
                                    "module API forward + autograd VJP, inputs resident; chunked "
                                    "runs recompute the forward in the backward")},
                "device_status": status, "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
                "setup_s": t_setup, "parity_rel_l2_sampled_rows": parity}
    del res
    return line


def run_large(args) -> dict | None:
    """`--workload cfg3`: `--structures` independent 200-atom structures (bf16 precision unless
    --precision is given), sharded over the ranks with no data-path exchange.  `--workload cfg4`:
    one graph of `--atoms` atoms at lmax 6, partitioned by destination-node range over the ranks
    (all-gather of embedding shards forward, reduce-scatter backward).  Inputs are resident on the
    device; the step is `ESO2Block.node_output_vjp` (per destination chunk the forward and at once
    the backward), or with --recompute `node_output` + autograd, whose backward recomputes each
    chunk's forward."""
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    precision = args.precision if (args.workload == "cfg4" or args.precision_given) else "bf16"
    line = measure_large(args.workload, world, rank, dev, precision=precision,
                         structures=args.structures,
                         atoms=args.atoms if args.workload == "cfg4" else 200, steps=args.steps,
                         warmup=args.warmup, recompute=args.recompute, parity_nodes=args.parity_nodes)
    if line is not None:
        line = {"metric": METRIC, "data": "synthetic", **line}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


# published by the reference on GH200 for its K4L2 configuration (lmax = mmax = 2, C = 128, fp32):
# eager PyTorch forward of the block on these fixtures (other hardware: context, not a target)
REFERENCE_PUBLISHED_FWD_MS = {"si_medium": 49.99, "si_small": 5.50}


def run_fixture(args) -> dict:
    """`--workload fixture --fixture NAME`: one of the reference's six benchmark structures
    (perturbed bulk Si / Cu, 6 A cutoff, no neighbour cap), rebuilt on the device from the
    recorded recipe, at the reference's K4L2 block configuration.  Times the module's forward to
    the scalar energy and forward + first-order VJP of the node output, inputs resident."""
    from zippel_b200 import fixtures as fx
    from zippel_b200.blocks.eso2 import BlockConfig, ESO2Block
    from zippel_b200.graph import EdgeGraph

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = BlockConfig()                                   # lmax 2, mmax 2, C = H = EC = 128, 64 RBF
    t0 = time.perf_counter()
    arrays, meta = fx.build_fixture(args.fixture, device=dev)
    build_s = time.perf_counter() - t0
    batch = fx.load_batch((arrays, meta), dev, torch.float32, cfg, requires_grad=False)
    block = ESO2Block(cfg, precision=args.precision)
    xavier_(block, 0)
    block = block.to(dev)
    n, e = meta["n_atoms"], meta["n_edges"]
    graph = EdgeGraph.build(batch["edge_index"], n)
    up = torch.randn(batch["x_node"].shape, generator=torch.Generator("cpu").manual_seed(9)).to(dev)
    a = (batch["atomic_numbers"], batch["edge_index"], batch["shifts"], batch["cos_gamma_k"],
         batch["sin_gamma_k"])

    def fwd():
        with torch.no_grad():
            return block(batch["pos"], a[0], batch["x_node"], *a[1:], graph=graph)

    def fwd_vjp():
        pos = batch["pos"].detach().requires_grad_(True)
        x = batch["x_node"].detach().requires_grad_(True)
        out = block.node_output(pos, a[0], x, *a[1:], graph=graph)
        return torch.autograd.grad((out * up).sum(), [x, pos, *block.parameters()],
                                   allow_unused=True)

    def energy_forces():
        # E and dE/dpos with frozen parameters and embeddings (the reference's force program,
        # blocks/eso2_ir.py:579-590): no parameter or embedding gradient is formed
        pos = batch["pos"].detach().requires_grad_(True)
        e_ = block(pos, a[0], batch["x_node"], *a[1:], graph=graph)
        return torch.autograd.grad(e_, pos)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        ms = []
        for _ in range(args.steps):
            ea, eb = torch.cuda.Event(True), torch.cuda.Event(True)
            ea.record(); fn(); eb.record()
            eb.synchronize()
            ms.append(ea.elapsed_time(eb))
        return statistics.median(ms)

    f_ms, b_ms = timed(fwd), timed(fwd_vjp)
    block.requires_grad_(False)
    ef_ms = timed(energy_forces)
    block.requires_grad_(True)
    pub = REFERENCE_PUBLISHED_FWD_MS.get(args.fixture)
    return {"metric": "edges/s, eSEN SO(2) block on a reference fixture (lmax2 mmax2 C128, fp32)",
            "workload": f"fixture {args.fixture}", "value": e / (b_ms * 1e-3), "unit": "edges/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": b_ms,
            "higher_is_better": True, "precision": args.precision, "data": "reference fixture rebuilt "
            "from its recipe (content hash equal to the reference manifest's)",
            "forward": {"ms": f_ms, "edges_per_s": e / (f_ms * 1e-3),
                        "reference_published_eager_ms_gh200": pub,
                        "ratio_to_published": (pub / f_ms) if pub else None},
            "energy_and_forces": {"ms": ef_ms, "edges_per_s": e / (ef_ms * 1e-3),
                                  "what": "E and dE/dpos, parameters and embeddings frozen"},
            "config": {"atoms": n, "edges": e, "avg_degree": meta["avg_degree"], "lmax": 2, "mmax": 2,
                       "channels": 128, "sha256_content": meta["sha256_content"],
                       "fixture_build_s": build_s},
            "device_status": block.plan(dev).device_status(),
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample-nodes", type=int, default=800,
                    help="CPU legs evaluate the edges into the first this-many atoms")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true",
                    help="profiling runs: skip both end-to-end legs (the line then has no valid e2e)")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "fp32_bf16x3", "bf16"],
                    help="operand format of the SO(2) contraction (see ESO2Block)")
    ap.add_argument("--fixture", default="si_medium",
                    choices=["si_small", "si_medium", "si_large", "cu_small", "cu_medium", "cu_large"],
                    help="with --workload fixture: which of the reference's structures")
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "fixture"],
                    help="cfg2 = the benchmark line; cfg3 / cfg4 = the larger configurations")
    ap.add_argument("--recompute", action="store_true",
                    help="cfg3 / cfg4: node_output + autograd (chunks recompute their forward) "
                         "instead of the streamed node_output_vjp")
    ap.add_argument("--structures", type=int, default=512, help="cfg3: number of 200-atom structures")
    ap.add_argument("--parity-nodes", type=int, default=6,
                    help="cfg3 / cfg4 legs: destination rows checked against the CPU oracle (0 = none)")
    ap.add_argument("--no-large", action="store_true",
                    help="skip the cfg3 / cfg4 legs that follow the headline measurement")
    ap.add_argument("--large-atoms", type=int, default=200000, help="atoms of the cfg4 leg")
    ap.add_argument("--large-timeout", type=int, default=200, help="seconds allowed per cfg3 / cfg4 leg")
    ap.add_argument("--atoms", type=int, default=N_ATOMS,
                    help="atoms per GPU; anything but the default is a profiling-size run, "
                         "not the benchmark workload")
    args = ap.parse_args()
    args.precision_given = any(a.startswith("--precision") for a in sys.argv[1:])
    # Library chatter (e.g. NCCL's version banner) must not share stdout with the JSON line:
    # everything else written to fd 1 during the run goes to stderr.
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    def emit(line):
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            emit(run_reference(args))
        return
    if args.workload == "fixture":
        line = run_fixture(args)
    else:
        line = run_ours(args) if args.workload == "cfg2" else run_large(args)
    if line is not None:
        emit(line)


if __name__ == "__main__":
    main()
