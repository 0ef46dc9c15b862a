"""Host logic of the multi-GPU paths on CPU: two gloo ranks, the oracle standing in for the
kernels.  Checks that the destination-range partition (all-gather of embedding shards forward,
reduce-scatter of their gradient backward, summed position/weight gradients) reproduces the
single-process result, and that structure sharding covers every structure exactly once."""

from __future__ import annotations

import os
import pathlib
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = pathlib.Path(__file__).resolve().parent.parent
WORLD = 2


def _case():
    from oracle import eso2_oracle as orc
    from tests.helpers import random_case
    cfg = dict(lmax=3, mmax=2, sphere_channels=8, hidden_channels=8, edge_channels=4,
               num_distance_basis=4, cutoff=5.0)
    params = orc.init_params(cfg, seed=5)
    case = random_case(cfg, 11, 70, seed=6)
    jd = orc.load_jd(ROOT / "zippel_b200" / "data" / "jd.npz", cfg["lmax"])
    return cfg, params, case, jd


def _worker(rank: int, port: int, out_dir: str):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    torch.set_num_threads(2)
    from oracle import eso2_oracle as orc
    from zippel_b200 import partition as part
    cfg, params, case, jd = _case()
    n = case["pos"].shape[0]
    ranges = part.node_ranges(n, WORLD)
    a, b = ranges[rank]
    keep = part.local_edges(case["edge_index"], ranges[rank])
    p = {k: v.clone().requires_grad_(k.startswith(("c1_", "c2_"))) for k, v in params.items()}
    pos = case["pos"].clone().requires_grad_(True)
    x_shard = case["x_node"][a:b].clone().requires_grad_(True)

    def node_output(pos_, z, x_full, ei, sh, cg, sg):
        return orc.block_node_out(p, cfg, pos_, z, x_full, ei, sh, cg, sg, jd)

    out = part.partitioned_node_output(node_output, pos, case["atomic_numbers"], x_shard,
                                       case["edge_index"][:, keep], case["shifts"][keep],
                                       case["cos_gamma_k"][keep], case["sin_gamma_k"][keep],
                                       ranges, rank)
    so2 = [v for k, v in p.items() if v.requires_grad]
    grads = torch.autograd.grad((out * case["upstream"][a:b]).sum(), [x_shard, pos, *so2])
    shared = [grads[1].clone(), *[g.clone() for g in grads[2:]]]
    part.all_reduce_grads(shared)
    torch.save({"out": out.detach(), "gx": grads[0], "gpos": shared[0], "gw": shared[1:],
                "range": (a, b)}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_destination_partition_matches_single_process(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    from oracle import eso2_oracle as orc
    cfg, params, case, jd = _case()
    p = {k: v.clone().requires_grad_(k.startswith(("c1_", "c2_"))) for k, v in params.items()}
    pos = case["pos"].clone().requires_grad_(True)
    x = case["x_node"].clone().requires_grad_(True)
    full = orc.block_node_out(p, cfg, pos, case["atomic_numbers"], x, case["edge_index"],
                              case["shifts"], case["cos_gamma_k"], case["sin_gamma_k"], jd)
    so2 = [v for v in p.values() if v.requires_grad]
    gx, gpos, *gw = torch.autograd.grad((full * case["upstream"]).sum(), [x, pos, *so2])
    for r in range(WORLD):
        got = torch.load(tmp_path / f"rank{r}.pt")
        a, b = got["range"]
        assert torch.allclose(got["out"], full[a:b].detach(), rtol=1e-12, atol=1e-12)
        assert torch.allclose(got["gx"], gx[a:b], rtol=1e-11, atol=1e-12)
        assert torch.allclose(got["gpos"], gpos, rtol=1e-10, atol=1e-12)
        for u, v in zip(got["gw"], gw):
            assert torch.allclose(u, v, rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("total,world", [(512, 8), (7, 3), (2, 4), (0, 2)])
def test_ranges_cover_everything_once(total, world):
    from zippel_b200.partition import node_ranges, structure_ranges
    for fn in (node_ranges, structure_ranges):
        r = fn(total, world)
        assert len(r) == world and r[0][0] == 0 and r[-1][1] == total
        assert all(x[1] == y[0] for x, y in zip(r, r[1:]))
        assert max(b - a for a, b in r) - min(b - a for a, b in r) <= 1
