"""One process per GPU: how the block's work is split, and the two collectives it needs.

* Independent structures (a batch of separate graphs) shard with no data-path exchange: every rank
  takes a contiguous range of structures (``structure_ranges``); only the SO(2) weight gradients
  are summed afterwards (``all_reduce_grads``).
* A single large graph is split by DESTINATION-node range (``node_ranges``): rank r owns the
  node rows ``n0:n1`` of ``x_node`` / ``node_out`` and every edge whose destination lies in that
  range (a contiguous slice of the destination-sorted edge list), so the forward scatter needs no
  reduction across ranks.  Sources may live anywhere: the embedding shards are all-gathered into
  the rank's own memory first (``GatherRows``), and in the backward the gradient with respect to
  the gathered copy is reduce-scattered back to the owning ranks.  Kernels only ever read local
  memory.

The reference has no multi-device code (its scope fence excludes it, PLAN.md:243-244); the
collectives go through ``torch.distributed`` (NCCL on GPUs; gloo works for CPU tests of this
logic).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _ranges(total: int, parts: int) -> list[tuple[int, int]]:
    base, extra = divmod(total, parts)
    out, start = [], 0
    for r in range(parts):
        stop = start + base + (1 if r < extra else 0)
        out.append((start, stop))
        start = stop
    return out


def node_ranges(n_nodes: int, world: int) -> list[tuple[int, int]]:
    """Contiguous, balanced destination-node ranges, one per rank."""
    return _ranges(n_nodes, world)


def structure_ranges(n_structures: int, world: int) -> list[tuple[int, int]]:
    return _ranges(n_structures, world)


def local_edges(edge_index: torch.Tensor, node_range: tuple[int, int]) -> torch.Tensor:
    """Positions (in the caller's edge order) of the edges whose destination is in the range."""
    dst = edge_index[1]
    return torch.nonzero((dst >= node_range[0]) & (dst < node_range[1]), as_tuple=False).flatten()


def gather_rows(shard: torch.Tensor, ranges, rank: int, group=None) -> torch.Tensor:
    """All-gather of row shards ``[n_r, ...]`` into the full ``[N, ...]`` array (local memory)."""
    n_max = max(b - a for a, b in ranges)
    padded = shard.new_zeros((n_max, *shard.shape[1:]))
    padded[: shard.shape[0]] = shard
    parts = [torch.empty_like(padded) for _ in ranges]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[: b - a] for p, (a, b) in zip(parts, ranges)], dim=0)


def scatter_sum_rows(grad_full: torch.Tensor, ranges, rank: int, group=None) -> torch.Tensor:
    """Sum of the ranks' full ``[N, ...]`` arrays, each rank keeping its own rows."""
    a, b = ranges[rank]
    if dist.get_backend(group) == "nccl":
        n_max = max(y - x for x, y in ranges)
        padded = grad_full.new_zeros((len(ranges), n_max, *grad_full.shape[1:]))
        for i, (x, y) in enumerate(ranges):
            padded[i, : y - x] = grad_full[x:y]
        out = torch.empty_like(padded[0])
        dist.reduce_scatter_tensor(out, padded, op=dist.ReduceOp.SUM, group=group)
        return out[: b - a]
    total = grad_full.contiguous().clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    return total[a:b]


class GatherRows(torch.autograd.Function):
    """``gather_rows`` with its VJP, the reduce-scatter (sum) of the full gradient back to the
    shards."""

    @staticmethod
    def forward(ctx, shard: torch.Tensor, ranges, rank: int, group):
        ctx.ranges, ctx.rank, ctx.group = ranges, rank, group
        return gather_rows(shard, ranges, rank, group)

    @staticmethod
    def backward(ctx, grad_full: torch.Tensor):
        return scatter_sum_rows(grad_full, ctx.ranges, ctx.rank, ctx.group), None, None, None


def partitioned_node_output(node_output_fn, pos, atomic_numbers, x_shard, edge_index, shifts,
                            cos_gamma_k, sin_gamma_k, ranges, rank: int, group=None):
    """Destination-range partition of one graph.

    ``node_output_fn(pos, Z, x_full, edge_index, shifts, cos, sin) -> [N, K, C]`` is the block's
    ``node_output``; ``edge_index`` etc. hold only this rank's edges (global node ids);
    ``x_shard`` are this rank's rows of ``x_node``.  Returns this rank's rows of ``node_out``.
    ``pos`` is replicated; its gradient is a per-rank partial to be summed with
    ``all_reduce_grads``.
    """
    x_full = GatherRows.apply(x_shard, ranges, rank, group)
    out = node_output_fn(pos, atomic_numbers, x_full, edge_index, shifts, cos_gamma_k, sin_gamma_k)
    a, b = ranges[rank]
    return out[a:b]


def partitioned_node_output_vjp(block, pos, atomic_numbers, x_shard, edge_index, shifts,
                                cos_gamma_k, sin_gamma_k, upstream_shard, ranges, rank: int,
                                graph=None, group=None):
    """Destination-range partition through ``ESO2Block.node_output_vjp``: per destination chunk
    the forward and at once the backward, nothing recomputed.

    Arguments as ``partitioned_node_output``; ``upstream_shard`` is the gradient with respect to
    this rank's rows of ``node_out``.  Returns ``(node_out rows, grad of x_shard, grad_pos,
    param_grads)``; ``grad_pos`` and ``param_grads`` are already summed over the ranks.
    """
    a, b = ranges[rank]
    x_full = gather_rows(x_shard.detach(), ranges, rank, group)

    def upstream(rows, n0, n1):                   # rows outside this rank's range carry no gradient
        g = torch.zeros_like(rows)
        lo, hi = max(n0, a), min(n1, b)
        if hi > lo:
            g[lo - n0:hi - n0] = upstream_shard[lo - a:hi - a]
        return g

    out, gx_full, gpos, gparams = block.node_output_vjp(
        pos, atomic_numbers, x_full, edge_index, shifts, cos_gamma_k, sin_gamma_k, upstream,
        graph=graph)
    gx = scatter_sum_rows(gx_full, ranges, rank, group)
    all_reduce_grads([gpos, *gparams], group)
    return out[a:b], gx, gpos, gparams


def all_reduce_grads(tensors, group=None) -> None:
    """Sums gradient tensors over ranks in place, as one flat bucket."""
    tensors = [t for t in tensors if t is not None]
    if not tensors:
        return
    flat = torch.cat([t.reshape(-1) for t in tensors])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for t in tensors:
        n = t.numel()
        t.copy_(flat[off:off + n].view_as(t))
        off += n
