"""Forward + VJP of the block for fixed array sizes, recorded once and replayed as a CUDA graph.

The module path (``ESO2Block.node_output`` + ``torch.autograd.grad``) enqueues a few hundred
kernels per step from Python; on a busy host the enqueue, not the GPU, sets the step time.
``CapturedStep`` records that very sequence — the host-to-device copies of the inputs, the edge
sort, the per-edge front end, the radial MLP, the edge convolution, its VJP and the copies of
the results back to the host — into one ``torch.cuda.CUDAGraph``.  A step is then: write the new
inputs into the pinned host arrays ``step.host[...]``, call ``step.run()``, read
``step.grad_pos_host`` / ``step.loss_host`` (and the device-side gradients in ``step.grads``).

It plays the part of the reference back end's ``allocate`` + ``run_program``
(codegen/compose.py:146-239: buffers allocated once, every run only launches) for the whole
module call (blocks/eso2_ref.py:317-349 and autograd through it).

The recording keeps every buffer of one step alive in the graph's private memory pool — inputs,
radial features, the block's workspace (about 125 KB per edge at lmax 4 / C 128 in the fp32
operand format) and all gradients — so the edge list must fit one call; graphs that need the
chunked path cannot be recorded.

Sizes are fixed at construction: the number of atoms and the number of edges (the edge list
itself, the positions and every other value may change from step to step).  The parameters are
read where they live, so in-place optimiser updates are seen by the next replay.
"""

from __future__ import annotations

import torch

from .blocks import eso2
from .blocks.eso2 import ESO2Block

HOST_KEYS = ("pos", "x_node", "edge_index", "shifts", "cos_gamma_k", "sin_gamma_k",
             "atomic_numbers", "upstream")


class CapturedStep:
    """loss = <node_output(batch), upstream>;  gradients w.r.t. x_node, pos and every parameter.

    ``example`` is a dict of CPU tensors with the keys ``HOST_KEYS`` (the reference's batch keys,
    fixtures/load.py:73-87, plus the upstream gradient [N, K, C]); it fixes the sizes and is the
    data of the recording run.
    """

    def __init__(self, block: ESO2Block, example: dict, device, warmup: int = 2):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("CapturedStep needs a CUDA device; there is no CPU path")
        self.block, self.device = block, device
        self.host = {k: example[k].detach().clone().contiguous().pin_memory() for k in HOST_KEYS}
        self.n_atoms = int(self.host["pos"].shape[0])
        self.n_edges = int(self.host["edge_index"].shape[1])
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.host.values())
        self.grad_pos_host = torch.empty(self.n_atoms, 3, pin_memory=True)
        self.loss_host = torch.empty((), pin_memory=True)
        self.d2h_bytes = self.grad_pos_host.numel() * 4 + 4
        # frozen parameters (requires_grad False) get no gradient: the recorded backward then
        # runs no weight-gradient products (a force evaluation in an MD loop)
        self.param_names = [n for n, p in block.named_parameters() if p.requires_grad]
        self.params = [p for p in block.parameters() if p.requires_grad]
        self.dev: dict = {}
        self.grads: dict = {}
        self.node_out = None
        self.graph = torch.cuda.CUDAGraph()
        self.stream = torch.cuda.Stream(device)
        self.copy_stream = torch.cuda.Stream(device)

        # chunk sizing reads the free memory of the device, which a recording must not do: the
        # whole edge list is one piece here (construction fails if its workspace does not fit)
        saved = eso2.MAX_EDGES_PER_CALL
        eso2.MAX_EDGES_PER_CALL = max(2 * self.n_edges, 4096)
        try:
            with torch.cuda.device(device):
                self.stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.stream):
                    for _ in range(max(warmup, 1)):       # plan creation, kernel attributes
                        self._enqueue()
                    self.stream.synchronize()
                    with torch.cuda.graph(self.graph, stream=self.stream):
                        self._enqueue()
                torch.cuda.current_stream().wait_stream(self.stream)
        finally:
            eso2.MAX_EDGES_PER_CALL = saved

    def _enqueue(self) -> None:
        dev = self.device
        main, side = torch.cuda.current_stream(dev), self.copy_stream
        # the small arrays first, on this stream; the two [N, K, C] arrays follow on a second
        # stream, so their transfer runs beside the edge sort, the front end and the radial MLP
        # (the embeddings) and beside the forward (the upstream gradient)
        big = ("x_node", "upstream")
        t = {k: v.to(dev, non_blocking=True) for k, v in self.host.items() if k not in big}
        side.wait_stream(main)
        ready = {}
        with torch.cuda.stream(side):
            for k in big:
                t[k] = self.host[k].to(dev, non_blocking=True)
                ready[k] = torch.cuda.Event()
                ready[k].record(side)
        pos = t["pos"].requires_grad_(True)
        x = t["x_node"].requires_grad_(True)
        node_out = self.block.node_output(pos, t["atomic_numbers"], x, t["edge_index"],
                                          t["shifts"], t["cos_gamma_k"], t["sin_gamma_k"],
                                          x_ready=ready["x_node"])
        main.wait_event(ready["upstream"])
        main.wait_stream(side)
        loss = (node_out * t["upstream"]).sum()
        g = torch.autograd.grad(loss, [x, pos, *self.params], allow_unused=True)
        self.grad_pos_host.copy_(g[1], non_blocking=True)
        self.loss_host.copy_(loss.detach(), non_blocking=True)
        self.dev, self.node_out = t, node_out.detach()
        self.grads = {"x_node": g[0], "pos": g[1],
                      "params": dict(zip(self.param_names, g[2:]))}

    def run(self, sync: bool = True) -> None:
        """Replays the recorded step on the current stream with the current contents of
        ``self.host``.  With ``sync`` the call returns when the host outputs are valid."""
        self.graph.replay()
        if sync:
            torch.cuda.current_stream(self.device).synchronize()
