"""Pre-allocated, autograd-free driver of the edge-convolution kernels.

``EdgeConvRunner`` plays the role of the reference back end's ``compile_program`` /
``allocate`` / ``run_program`` trio (codegen/compose.py:113-239) for the one program this
package runs: it sizes and allocates every device buffer once, then ``forward()`` /
``backward()`` only enqueue kernels on the current stream through the C ABI.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .blocks.eso2 import Plan, _weights_struct
from .graph import EdgeGraph


class EdgeConvRunner:
    """``edge_channels`` > 0: the last radial layer (edge_channels -> R) runs inside the call
    (``zp_eso2_forward_radial`` / ``zp_eso2_backward_radial``): ``bind`` then takes that layer's
    input ``h_rad [E, edge_channels]`` in place of ``radial`` and its weight and bias as
    ``rad_layer``; the backward returns ``grad_h_rad`` where it otherwise returns ``grad_radial``
    and fills ``grad_rad_w`` / ``grad_rad_b``."""

    def __init__(self, plan: Plan, graph: EdgeGraph, with_backward: bool = True,
                 edge_channels: int = 0):
        self.plan, self.graph, self.with_backward = plan, graph, with_backward
        self.edge_channels = int(edge_channels)
        self.lib = _lib.load()
        n, e, s, dev = graph.n_nodes, graph.n_edges, plan.sizes, plan.device
        f32 = dict(dtype=torch.float32, device=dev)
        self.ws = plan.workspace(n, e, with_backward, inference=not with_backward,
                                 edge_channels=self.edge_channels)
        self.node_out = torch.empty(n, s.K, plan.c, **f32)
        if with_backward:
            self.grad_x = torch.empty(n, s.K, plan.c, **f32)
            self.grad_edge_vec = torch.empty(e, 3, **f32)
            self.grad_radial = torch.empty(e, self.edge_channels or s.R, **f32)
            self.grad_env = torch.empty(e, **f32)
            self.grad_w = None
            if self.edge_channels:
                self.grad_rad_w = torch.empty(s.R, self.edge_channels, **f32)
                self.grad_rad_b = torch.empty(s.R, **f32)
        self._w = self._gw = None
        self._keep = []
        self.rad_layer = None

    def bind(self, x_node, edge_vec, cos_g, sin_g, radial, env, c1_w0, c1_b0, c1_wm, c2_w0,
             c2_b0, c2_wm, rad_layer=None):
        """Fixes the input tensors (fp32, contiguous, sorted-edge order); no copies are made."""
        if bool(self.edge_channels) != (rad_layer is not None):
            raise ValueError("rad_layer=(weight, bias) goes with edge_channels > 0, and only then")
        tens = [x_node, edge_vec, cos_g, sin_g, radial, env, c1_w0, c1_b0, c2_w0, c2_b0,
                *c1_wm, *c2_wm, *(rad_layer or ())]
        self.rad_layer = tuple(rad_layer) if rad_layer is not None else None
        for t in tens:
            if t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda:
                raise ValueError("EdgeConvRunner.bind needs contiguous fp32 CUDA tensors")
        self.inputs = (x_node, edge_vec, cos_g, sin_g, radial, env)
        self.weights = (c1_w0, c1_b0, list(c1_wm), c2_w0, c2_b0, list(c2_wm))
        self._w, k1 = _weights_struct(self.plan.mmax, *self.weights)
        self._keep = [k1]
        if self.with_backward:
            # all weight gradients are views of ONE buffer, so that a data-parallel caller can
            # all-reduce them in place with a single collective (no gather / copy-back)
            order = [c1_w0, c1_b0, *c1_wm, c2_w0, c2_b0, *c2_wm]
            starts, total = [], 0
            for t in order:
                starts.append(total)
                total += (t.numel() + 63) // 64 * 64          # 256-byte aligned views
            self.grad_w_flat = torch.zeros(total, dtype=torch.float32, device=c1_w0.device)
            views = [self.grad_w_flat[a:a + t.numel()].view_as(t) for a, t in zip(starts, order)]
            m = len(c1_wm)
            self.grad_w = (views[0], views[1], views[2:2 + m], views[2 + m], views[3 + m],
                           views[4 + m:])
            self._gw, k2 = _weights_struct(self.plan.mmax, *self.grad_w)
            self._keep.append(k2)

    def forward(self) -> torch.Tensor:
        x, ev, cg, sg, rad, en = self.inputs
        g = self.graph
        st = torch.cuda.current_stream().cuda_stream
        if self.rad_layer is not None:
            rw, rb = self.rad_layer
            _lib.check(self.lib.zp_eso2_forward_radial(
                self.plan.handle, g.n_nodes, g.n_edges, x.data_ptr(), ev.data_ptr(), cg.data_ptr(),
                sg.data_ptr(), rad.data_ptr(), rw.data_ptr(), rb.data_ptr(), self.edge_channels,
                en.data_ptr(), g.src.data_ptr(), g.dst.data_ptr(), g.row_ptr.data_ptr(),
                ctypes.byref(self._w), self.node_out.data_ptr(), self.ws.data_ptr(),
                self.ws.numel(), 1 if self.with_backward else 0, st), "zp_eso2_forward_radial")
            return self.node_out
        # without a backward nothing is kept: the leaner entry point
        fn = self.lib.zp_eso2_forward if self.with_backward else self.lib.zp_eso2_forward_inference
        _lib.check(fn(
            self.plan.handle, g.n_nodes, g.n_edges, x.data_ptr(), ev.data_ptr(), cg.data_ptr(),
            sg.data_ptr(), rad.data_ptr(), en.data_ptr(), g.src.data_ptr(), g.dst.data_ptr(),
            g.row_ptr.data_ptr(), ctypes.byref(self._w), self.node_out.data_ptr(),
            self.ws.data_ptr(), self.ws.numel(), st), "zp_eso2_forward")
        return self.node_out

    def backward(self, grad_node_out: torch.Tensor, weight_grads: bool = True,
                 x_grad: bool = True):
        """``weight_grads=False``: the parameters are frozen (a force evaluation): their gradient
        products are not run and ``grad_w`` / ``grad_rad_w`` / ``grad_rad_b`` keep old contents.
        ``x_grad=False``: no gradient of ``x_node`` (``grad_x`` keeps its old contents)."""
        x, ev, cg, sg, rad, en = self.inputs
        g = self.graph
        st = torch.cuda.current_stream().cuda_stream
        gw_ref = ctypes.byref(self._gw) if weight_grads else None
        gx_ptr = self.grad_x.data_ptr() if x_grad else None
        if self.rad_layer is not None:
            rw, rb = self.rad_layer
            _lib.check(self.lib.zp_eso2_backward_radial(
                self.plan.handle, g.n_nodes, g.n_edges, grad_node_out.data_ptr(), x.data_ptr(),
                ev.data_ptr(), cg.data_ptr(), sg.data_ptr(), rad.data_ptr(), rw.data_ptr(),
                rb.data_ptr(), self.edge_channels, en.data_ptr(), g.src.data_ptr(),
                g.dst.data_ptr(), g.row_ptr.data_ptr(), g.perm_src.data_ptr(),
                g.row_ptr_src.data_ptr(), ctypes.byref(self._w), gx_ptr,
                self.grad_edge_vec.data_ptr(), self.grad_radial.data_ptr(),
                self.grad_rad_w.data_ptr() if weight_grads else None,
                self.grad_rad_b.data_ptr() if weight_grads else None, self.grad_env.data_ptr(),
                gw_ref, self.ws.data_ptr(), self.ws.numel(), st),
                "zp_eso2_backward_radial")
            return self.grad_x, self.grad_edge_vec, self.grad_radial, self.grad_env, self.grad_w
        _lib.check(self.lib.zp_eso2_backward(
            self.plan.handle, g.n_nodes, g.n_edges, grad_node_out.data_ptr(), x.data_ptr(),
            ev.data_ptr(), cg.data_ptr(), sg.data_ptr(), rad.data_ptr(), en.data_ptr(),
            g.src.data_ptr(), g.dst.data_ptr(), g.row_ptr.data_ptr(), g.perm_src.data_ptr(),
            g.row_ptr_src.data_ptr(), ctypes.byref(self._w), gx_ptr,
            self.grad_edge_vec.data_ptr(), self.grad_radial.data_ptr(), self.grad_env.data_ptr(),
            gw_ref, self.ws.data_ptr(), self.ws.numel(), st), "zp_eso2_backward")
        return self.grad_x, self.grad_edge_vec, self.grad_radial, self.grad_env, self.grad_w

    # -- per-kernel-class timing ---------------------------------------------------------
    def timing(self, on: bool) -> None:
        _lib.check(self.lib.zp_timing_enable(self.plan.handle, int(on)), "zp_timing_enable")

    def read_timing(self) -> dict[str, tuple[float, int]]:
        n = _lib.N_KERNEL_CLASSES
        ms, cnt = (ctypes.c_float * n)(), (ctypes.c_int64 * n)()
        _lib.check(self.lib.zp_timing_read(self.plan.handle, ms, cnt), "zp_timing_read")
        return {self.lib.zp_kernel_class_name(i).decode(): (ms[i], cnt[i]) for i in range(n)}
