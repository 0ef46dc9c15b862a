"""The eSEN SO(2) interaction block on the B200 kernels.

Drop-in for the reference's ``blocks/eso2_ref.py``: ``BlockConfig`` and ``Layout`` carry the
same fields (``eso2_ref.py:51-146``), ``ESO2Block`` has the parameter names, ``state_dict`` and
``forward`` signature of ``ESO2RefBlock`` (``eso2_ref.py:154-351``), and
``conservative_training_step`` is *not* offered (it needs a double backward, which the kernels
do not provide).  Unlike the reference, ``mmax < lmax`` works: the l-major -> m'-major selection
is the rectangular ``[Km, K]`` matrix.

What runs where
    * the per-edge front end (geometry, Gaussian basis, element embeddings, envelope) is one
      kernel each way (``EdgeFeatures``); the radial MLP runs on the contraction engine
      (``TensorCoreLinear``) with fused LayerNorm + SiLU passes (``LayerNormSiLU``);
    * everything per edge and per (l, m, channel) -- gather, Wigner-D rotation, both SO(2)
      convolutions, the gate, rotation back and the scatter onto destination nodes, forward and
      VJP -- is one call into the C ABI (``zp_eso2_forward`` / ``zp_eso2_backward``) through
      ``EdgeConvFunction``;
    * the readout head after the node output (invariants, two dense layers, sum over atoms) is
      ``Readout`` (``zp_readout_forward`` / ``zp_readout_backward``).
There is no fallback: without the built library and a supported GPU every call raises, and
sizes the kernels do not take (``edge_channels`` not a multiple of 4 or above 1024) are refused
when the block is built.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn

from .. import _lib
from ..graph import EdgeChunk, EdgeGraph

_JD_PATH = __import__("pathlib").Path(__file__).resolve().parent.parent / "data" / "jd.npz"


def load_jd(lmax: int = 6) -> list[torch.Tensor]:
    """The J_l matrices (l = 0..lmax, FP64) shipped with the package; same values as the
    reference's ``blocks/Jd.pt``."""
    z = np.load(_JD_PATH)
    return [torch.from_numpy(z[f"J{l}"]) for l in range(lmax + 1)]


@dataclass(frozen=True)
class BlockConfig:
    lmax: int = 2
    mmax: int = 2
    sphere_channels: int = 128
    hidden_channels: int = 128
    edge_channels: int = 128
    num_distance_basis: int = 64
    cutoff: float = 6.0
    max_num_elements: int = 100
    envelope_exponent: int = 5

    @property
    def num_coeffs(self) -> int:
        return (self.lmax + 1) ** 2

    @property
    def edge_channels_list(self) -> list[int]:
        return [self.num_distance_basis + 2 * self.edge_channels, self.edge_channels,
                self.edge_channels]


@dataclass(frozen=True)
class Layout:
    """Index tables of an (lmax, mmax) pair."""

    lmax: int
    mmax: int
    m_size: tuple[int, ...]
    m_split: tuple[int, ...]

    @staticmethod
    def make(lmax: int, mmax: int) -> "Layout":
        m_size = tuple(lmax + 1 - m for m in range(mmax + 1))
        return Layout(lmax, mmax, m_size, (m_size[0],) + tuple(2 * s for s in m_size[1:]))

    @property
    def rows(self) -> list[tuple[int, int]]:
        """(l, signed m) per m'-major row."""
        out = [(l, 0) for l in range(self.lmax + 1)]
        for m in range(1, self.mmax + 1):
            out += [(l, m) for l in range(m, self.lmax + 1)]
            out += [(l, -m) for l in range(m, self.lmax + 1)]
        return out

    def to_m(self, device, dtype) -> torch.Tensor:
        """[Km, K] selection from l-major (l, m = -l..l) to m'-major rows."""
        rows = self.rows
        mat = torch.zeros(len(rows), (self.lmax + 1) ** 2, device=device, dtype=dtype)
        for r, (l, m) in enumerate(rows):
            mat[r, l * l + l + m] = 1.0
        return mat

    def gate_expand_index(self, device) -> torch.Tensor:
        return torch.tensor([l - 1 for l, _ in self.rows[1:]], dtype=torch.long, device=device)


# --------------------------------------------------------------------------------------------
# plan cache and the autograd function over the C ABI
# --------------------------------------------------------------------------------------------


class Plan:
    """Owns one ``zp_plan`` (static tables on one device)."""

    _cache: dict = {}

    def __init__(self, lmax: int, mmax: int, c: int, h: int, device: torch.device,
                 precision: int = 2):
        lib = _lib.load()
        self.precision = precision
        self.device = device
        jd = np.concatenate([j.numpy().astype(np.float64).ravel() for j in load_jd(lmax)])
        cfg = _lib.ZpConfig(lmax, mmax, c, h, precision)
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(lib.zp_plan_create(ctypes.byref(cfg),
                                          jd.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
                                          ctypes.byref(handle)), "zp_plan_create")
        self.handle = handle
        sizes = _lib.ZpSizes()
        _lib.check(lib.zp_plan_sizes(handle, ctypes.byref(sizes)), "zp_plan_sizes")
        self.sizes = sizes
        self.lmax, self.mmax, self.c, self.h = lmax, mmax, c, h

    @classmethod
    def get(cls, lmax, mmax, c, h, device, precision: int = 2) -> "Plan":
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("zippel_b200 runs on CUDA devices only; there is no CPU path")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (lmax, mmax, c, h, device.index, precision)
        if key not in cls._cache:
            cls._cache[key] = cls(lmax, mmax, c, h, device, precision)
        return cls._cache[key]

    def tables(self) -> dict[str, np.ndarray]:
        km = self.sizes.Km
        arrs = [np.zeros(km, np.int32) for _ in range(4)]
        ptrs = [a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)) for a in arrs]
        _lib.check(_lib.load().zp_plan_tables(self.handle, *ptrs), "zp_plan_tables")
        return dict(zip(("row_l", "row_m", "rot_off", "gate_idx"), arrs))

    def device_status(self) -> int:
        """Reads and clears the device status word (synchronises the device)."""
        st = ctypes.c_int(0)
        _lib.check(_lib.load().zp_plan_device_status(self.handle, ctypes.byref(st)),
                   "zp_plan_device_status")
        return st.value

    def workspace(self, n: int, e: int, with_backward: bool, inference: bool = False,
                  edge_channels: int = 0) -> torch.Tensor:
        """Workspace of one forward (+ backward) call over ``e`` edges and ``n`` node rows;
        ``inference``: for ``zp_eso2_forward_inference`` (nothing kept for a backward);
        ``edge_channels`` > 0: for the entry points that run the last radial layer themselves."""
        mode = 1 if with_backward else (2 if inference else 0)
        lib = _lib.load()
        nbytes = (lib.zp_workspace_bytes_radial(self.handle, n, e, edge_channels, mode)
                  if edge_channels else lib.zp_workspace_bytes(self.handle, n, e, mode))
        if nbytes == 0 and edge_channels:
            raise _lib.ZpError(2, "zp_workspace_bytes_radial")
        return torch.empty(max(nbytes, 16), dtype=torch.uint8, device=self.device)


def _weights_struct(mmax, c1_w0, c1_b0, c1_wm, c2_w0, c2_b0, c2_wm):
    arr_t = ctypes.c_void_p * max(mmax, 1)
    a1 = arr_t(*[t.data_ptr() for t in c1_wm]) if mmax else arr_t(0)
    a2 = arr_t(*[t.data_ptr() for t in c2_wm]) if mmax else arr_t(0)
    w = _lib.ZpWeights(c1_w0.data_ptr(), c1_b0.data_ptr(), a1, c2_w0.data_ptr(), c2_b0.data_ptr(), a2)
    return w, (a1, a2)


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float32).contiguous()


#: Upper bound on the edges handed to one forward/backward call of the C ABI.  ``None`` sizes it
#: from the device's free memory (the per-call workspace is ~123 KB per edge at lmax 4 / C 128).
#: Larger graphs are processed as destination-node chunks; the backward then recomputes each
#: chunk's forward instead of keeping every chunk's activations.
MAX_EDGES_PER_CALL: int | None = None


def _edge_budget(plan: Plan, n: int, e: int) -> int:
    if MAX_EDGES_PER_CALL is not None:
        return max(1, MAX_EDGES_PER_CALL)
    lib = _lib.load()
    probe = 4096
    per_edge = (lib.zp_workspace_bytes(plan.handle, 0, probe, 1)
                - lib.zp_workspace_bytes(plan.handle, 0, 0, 1)) / probe
    free, _total = torch.cuda.mem_get_info(plan.device)
    # memory the caching allocator holds but is not using can be re-used for the workspace
    free += torch.cuda.memory_reserved(plan.device) - torch.cuda.memory_allocated(plan.device)
    return _quantise_budget(max(1024, int(0.5 * free / max(per_edge, 1.0))))


def _quantise_budget(budget: int) -> int:
    """``budget`` rounded down to four significant bits: free memory drifts from call to call,
    and the chunking of a graph that is reused (cached per budget) should not be redone for
    every small change.  At most 1/8 of the budget is given up."""
    step = 1 << max(budget.bit_length() - 4, 0)
    return budget // step * step


def _abi_forward(plan, n_rows, e, x, ev, cg, sg, rad, en, src, dst, row_ptr, wstruct, out, ws,
                 inference: bool = False, layer=None):
    """``inference``: nothing is kept for a backward (``ws`` sized for that).  ``layer`` =
    ``(rad_w, rad_b)``: ``rad`` is then the INPUT of the last radial layer, which the call runs
    itself (``zp_eso2_forward_radial``)."""
    st = torch.cuda.current_stream().cuda_stream
    lib = _lib.load()
    if layer is not None:
        rw, rb = layer
        _lib.check(lib.zp_eso2_forward_radial(
            plan.handle, n_rows, e, x.data_ptr(), ev.data_ptr(), cg.data_ptr(), sg.data_ptr(),
            rad.data_ptr(), rw.data_ptr(), rb.data_ptr(), rw.shape[1], en.data_ptr(),
            src.data_ptr(), dst.data_ptr(), row_ptr.data_ptr(), ctypes.byref(wstruct),
            out.data_ptr(), ws.data_ptr(), ws.numel(), 0 if inference else 1, st),
            "zp_eso2_forward_radial")
        return
    fn = lib.zp_eso2_forward_inference if inference else lib.zp_eso2_forward
    _lib.check(fn(
        plan.handle, n_rows, e, x.data_ptr(), ev.data_ptr(), cg.data_ptr(), sg.data_ptr(),
        rad.data_ptr(), en.data_ptr(), src.data_ptr(), dst.data_ptr(), row_ptr.data_ptr(),
        ctypes.byref(wstruct), out.data_ptr(), ws.data_ptr(), ws.numel(), st),
        "zp_eso2_forward_inference" if inference else "zp_eso2_forward")


def _abi_backward(plan, n, e, g_ptr: int, x, ev, cg, sg, rad, en, sub: EdgeGraph, wstruct, gx, gev,
                  grad, gen, gstruct, ws, layer=None):
    """``g_ptr``: address of row 0 of grad_node_out.  The kernels read it only at the rows of the
    edges' destinations, so a caller holding rows n0:n1 alone passes its base minus n0 rows.
    ``layer`` = ``(rad_w, rad_b, grad_rad_w, grad_rad_b)``: ``rad`` / ``grad`` are the input of
    the last radial layer and its gradient (``zp_eso2_backward_radial``).  ``gstruct`` None, or
    the layer's two gradient tensors None: those parameters are frozen, their gradients are not
    computed."""
    st = torch.cuda.current_stream().cuda_stream
    lib = _lib.load()
    g_ref = ctypes.byref(gstruct) if gstruct is not None else None
    gx_ptr = gx.data_ptr() if gx is not None else None          # None: no gradient of x_node
    if layer is not None:
        rw, rb, grw, grb = layer
        grw_ptr, grb_ptr = (grw.data_ptr(), grb.data_ptr()) if grw is not None else (None, None)
        _lib.check(lib.zp_eso2_backward_radial(
            plan.handle, n, e, g_ptr, x.data_ptr(), ev.data_ptr(), cg.data_ptr(), sg.data_ptr(),
            rad.data_ptr(), rw.data_ptr(), rb.data_ptr(), rw.shape[1], en.data_ptr(),
            sub.src.data_ptr(), sub.dst.data_ptr(), sub.row_ptr.data_ptr(),
            sub.perm_src.data_ptr(), sub.row_ptr_src.data_ptr(), ctypes.byref(wstruct),
            gx_ptr, gev.data_ptr(), grad.data_ptr(), grw_ptr, grb_ptr,
            gen.data_ptr(), g_ref, ws.data_ptr(), ws.numel(), st),
            "zp_eso2_backward_radial")
        return
    _lib.check(lib.zp_eso2_backward(
        plan.handle, n, e, g_ptr, x.data_ptr(), ev.data_ptr(), cg.data_ptr(),
        sg.data_ptr(), rad.data_ptr(), en.data_ptr(), sub.src.data_ptr(), sub.dst.data_ptr(),
        sub.row_ptr.data_ptr(), sub.perm_src.data_ptr(), sub.row_ptr_src.data_ptr(),
        ctypes.byref(wstruct), gx_ptr, gev.data_ptr(), grad.data_ptr(), gen.data_ptr(),
        g_ref, ws.data_ptr(), ws.numel(), st), "zp_eso2_backward")


class EdgeConvFunction(torch.autograd.Function):
    """node_out = edge_conv(x_node, edge_vec, cos_g, sin_g, radial, env; SO(2) weights).

    Per-edge inputs are in the graph's destination-sorted order.  Differentiable w.r.t. x_node,
    edge_vec (through the rotation), radial, env and the SO(2) weights; first order only.
    With ``rad_w`` / ``rad_b`` given (weight [R, EC] and bias [R] of the radial MLP's last layer),
    ``radial`` is that layer's INPUT [E, EC] and the layer runs inside the kernel path, forward
    and VJP (the gradients then go to the input, the weight and the bias).
    """

    @staticmethod
    def forward(ctx, plan: Plan, graph: EdgeGraph, x_node, edge_vec, cos_g, sin_g, radial, env,
                rad_w, rad_b, c1_w0, c1_b0, c2_w0, c2_b0, *wm):
        mmax = plan.mmax
        n, e = graph.n_nodes, graph.n_edges
        has_layer = rad_w is not None
        s = plan.sizes
        if not has_layer:        # placeholders keep the argument positions (no gradient flows)
            rad_w, rad_b = radial.new_zeros(0), radial.new_zeros(0)
        ins = (x_node, edge_vec, cos_g, sin_g, radial, env, rad_w, rad_b, c1_w0, c1_b0, c2_w0,
               c2_b0, *wm)
        tens = [_f32(t) for t in ins]
        x, ev, cg, sg, rad, en, rw, rb, w10, b10, w20, b20 = tens[:12]
        wms = tens[12:]
        layer = (rw, rb) if has_layer else None
        ec = rw.shape[1] if has_layer else 0
        assert x.shape == (n, s.K, plan.c), (x.shape, (n, s.K, plan.c))
        assert rad.shape == ((e, ec) if has_layer else (e, s.R)) and ev.shape == (e, 3)
        assert not has_layer or (rw.shape == (s.R, ec) and rb.shape == (s.R,))
        assert en.shape == (e,) and cg.shape == (e, plan.lmax + 1) and sg.shape == cg.shape
        needs_bwd = any(ctx.needs_input_grad)
        # a graph may carry `node_range = (n0, n1)`: all its edges end in those nodes and only
        # those rows of node_out are wanted (used by the chunked module path)
        rng = getattr(graph, "node_range", None)
        n0, n1 = rng if rng is not None else (0, n)
        out = torch.empty(n1 - n0, s.K, plan.c, dtype=torch.float32, device=x.device)
        wstruct, keep = _weights_struct(mmax, w10, b10, wms[:mmax], w20, b20, wms[mmax:])
        with torch.cuda.device(x.device):
            # a node-range graph is already one piece of a chunked run: never split it again
            chunks = ([EdgeChunk(0, e, 0, n, graph)] if rng is not None
                      else graph.chunks(_edge_budget(plan, n, e)))
            if len(chunks) == 1:
                ws = plan.workspace(n1 - n0, e, needs_bwd, inference=not needs_bwd, edge_channels=ec)
                _abi_forward(plan, n1 - n0, e, x, ev, cg, sg, rad, en, graph.src, graph.dst,
                             graph.row_ptr[n0:], wstruct, out, ws, inference=not needs_bwd,
                             layer=layer)
            else:
                # the backward recomputes each chunk, so no chunk keeps anything here
                ws = plan.workspace(max(c.n1 - c.n0 for c in chunks),
                                    max(c.n_edges for c in chunks), False, inference=True,
                                    edge_channels=ec)
                for c in chunks:
                    sl = slice(c.e0, c.e1)
                    _abi_forward(plan, c.n1 - c.n0, c.n_edges, x, ev[sl], cg[sl], sg[sl], rad[sl],
                                 en[sl], c.sub.src, c.sub.dst, c.sub.row_ptr[c.n0:],
                                 wstruct, out[c.n0:c.n1], ws, inference=True, layer=layer)
                ws = None
        del keep
        if needs_bwd:
            # the workspace goes through save_for_backward like any activation, so that
            # activation checkpointing can drop it and recompute
            ctx.plan, ctx.graph, ctx.chunks, ctx.has_ws = plan, graph, chunks, ws is not None
            ctx.has_layer = has_layer
            ctx.save_for_backward(*tens, *([ws] if ws is not None else []))
            ctx.in_dtypes = [t.dtype for t in ins]
        return out.to(x_node.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        plan, graph, chunks = ctx.plan, ctx.graph, ctx.chunks
        tens = ctx.saved_tensors
        ws = tens[-1] if ctx.has_ws else None
        if ctx.has_ws:
            tens = tens[:-1]
        x, ev, cg, sg, rad, en, rw, rb, w10, b10, w20, b20 = tens[:12]
        wms = tens[12:]
        mmax = plan.mmax
        n, e = graph.n_nodes, graph.n_edges
        g = _f32(grad_out)
        gev, grad, gen = (torch.empty_like(t) for t in (ev, rad, en))
        # embeddings that need no gradient (E and dE/dpos of one block): nothing is summed per node
        gx = torch.empty_like(x) if ctx.needs_input_grad[2] else None
        # frozen parameters (an MD force evaluation): their gradient products are not run
        want_w = any(ctx.needs_input_grad[10:])
        want_lw = ctx.has_layer and (ctx.needs_input_grad[8] or ctx.needs_input_grad[9])
        grw, grb = (torch.empty_like(rw), torch.empty_like(rb)) if want_lw else (None, None)
        layer = (rw, rb, grw, grb) if ctx.has_layer else None
        ec = rw.shape[1] if ctx.has_layer else 0
        gws = [torch.empty_like(t) for t in (w10, b10, w20, b20, *wms)] if want_w else []
        wstruct, keep = _weights_struct(mmax, w10, b10, wms[:mmax], w20, b20, wms[mmax:])
        gstruct, keep2 = (_weights_struct(mmax, gws[0], gws[1], gws[4:4 + mmax], gws[2], gws[3],
                                          gws[4 + mmax:]) if want_w else (None, None))
        rng = getattr(graph, "node_range", None)
        row_bytes = plan.sizes.K * plan.c * 4
        g_ptr = g.data_ptr() - (rng[0] * row_bytes if rng is not None else 0)
        with torch.cuda.device(x.device):
            if len(chunks) == 1:
                _abi_backward(plan, n, e, g_ptr, x, ev, cg, sg, rad, en, graph, wstruct, gx, gev,
                              grad, gen, gstruct, ws, layer=layer)
            else:
                # per chunk: recompute its forward into the shared workspace, then its backward;
                # node and weight gradients add up over chunks, per-edge gradients are slices
                ws = plan.workspace(max(c.n1 - c.n0 for c in chunks),
                                    max(c.n_edges for c in chunks), True, edge_channels=ec)
                gx_c = torch.empty_like(gx) if gx is not None else None
                grw_c, grb_c = ((torch.empty_like(rw), torch.empty_like(rb)) if want_lw
                                else (None, None))
                gws_c = [torch.empty_like(t) for t in gws]
                cstruct, keep3 = (_weights_struct(mmax, gws_c[0], gws_c[1], gws_c[4:4 + mmax],
                                                  gws_c[2], gws_c[3], gws_c[4 + mmax:])
                                  if want_w else (None, None))
                scratch_out = torch.empty(max(c.n1 - c.n0 for c in chunks), plan.sizes.K, plan.c,
                                          dtype=torch.float32, device=x.device)
                for i, c in enumerate(chunks):
                    sl = slice(c.e0, c.e1)
                    _abi_forward(plan, c.n1 - c.n0, c.n_edges, x, ev[sl], cg[sl], sg[sl], rad[sl],
                                 en[sl], c.sub.src, c.sub.dst, c.sub.row_ptr[c.n0:], wstruct,
                                 scratch_out, ws, layer=layer[:2] if layer else None)
                    first = i == 0
                    lay = None if layer is None else (rw, rb, *((grw, grb) if first else (grw_c, grb_c)))
                    _abi_backward(plan, n, c.n_edges, g_ptr, x, ev[sl], cg[sl], sg[sl], rad[sl], en[sl],
                                  c.sub, wstruct, gx if first else gx_c, gev[sl], grad[sl], gen[sl],
                                  gstruct if first else cstruct, ws, layer=lay)
                    if not first:
                        for a_, b_ in zip([gx, *gws, grw, grb], [gx_c, *gws_c, grw_c, grb_c]):
                            if a_ is not None:
                                a_.add_(b_)
                del keep3
        del keep, keep2
        grads = [gx, gev, None, None, grad, gen, grw, grb,
                 *(gws if want_w else [None] * (4 + len(wms)))]
        dts = ctx.in_dtypes
        outs = []
        for i, gr in enumerate(grads):
            outs.append(None if gr is None or not ctx.needs_input_grad[i + 2] else gr.to(dts[i]))
        return (None, None, *outs)


class TensorCoreLinear(torch.autograd.Function):
    """y = x W^T + b on the contraction engine (``zp_linear_forward/backward``), in the plan's
    operand format.  Used for the widest radial layer; first order only."""

    @staticmethod
    def forward(ctx, plan: Plan, x, weight, bias):
        lib = _lib.load()
        xf, wf, bf = _f32(x), _f32(weight), _f32(bias)
        m, k = xf.shape
        n = wf.shape[0]
        y = torch.empty(m, n, dtype=torch.float32, device=xf.device)
        nbytes = lib.zp_linear_work_bytes(plan.handle, m, k, n)
        if nbytes == 0:
            raise _lib.ZpError(2, "zp_linear_work_bytes")
        work = torch.empty(nbytes, dtype=torch.uint8, device=xf.device)
        with torch.cuda.device(xf.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_linear_forward(plan.handle, m, k, n, xf.data_ptr(), wf.data_ptr(),
                                             bf.data_ptr(), y.data_ptr(), work.data_ptr(), nbytes,
                                             st), "zp_linear_forward")
        ctx.plan, ctx.dtypes = plan, (x.dtype, weight.dtype, bias.dtype)
        # what the backward reads of x and W are their 16-bit planes, which the forward has just
        # written into `work`: the buffer is kept instead of the two fp32 arrays, and the backward
        # neither scans nor re-formats them again
        ctx.shape = (m, k, n)
        ctx.work = work if any(ctx.needs_input_grad) else None
        return y.to(x.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_y):
        lib = _lib.load()
        plan, work = ctx.plan, ctx.work
        m, k, n = ctx.shape
        dy = _f32(grad_y)
        dev = dy.device
        # a frozen layer forms the input gradient only; a layer whose input needs none, the
        # parameter gradients only
        want_x = ctx.needs_input_grad[1]
        want_w = ctx.needs_input_grad[2] or ctx.needs_input_grad[3] or not want_x
        f32 = dict(dtype=torch.float32, device=dev)
        dx = torch.empty(m, k, **f32) if want_x else None
        dw = torch.empty(n, k, **f32) if want_w else None
        db = torch.empty(n, **f32) if want_w else None
        ptr = lambda t: t.data_ptr() if t is not None else None                  # noqa: E731
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_linear_backward_saved(plan.handle, m, k, n, dy.data_ptr(), ptr(dx),
                                                    ptr(dw), ptr(db), work.data_ptr(),
                                                    work.numel(), st),
                       "zp_linear_backward_saved")
        dt = ctx.dtypes
        to = lambda t, d: t.to(d) if t is not None else None                       # noqa: E731
        return None, to(dx, dt[0]), to(dw, dt[1]), to(db, dt[2])


class LayerNormSiLU(torch.autograd.Function):
    """silu(layer_norm(x) * gamma + beta) in one pass each way (``zp_layernorm_silu_forward`` /
    ``_backward``): nn.LayerNorm + nn.SiLU of the radial MLP's hidden layers (reference
    blocks/eso2_ref.py:170-180).  fp32, first order only."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps: float):
        lib = _lib.load()
        if not x.is_cuda:
            raise RuntimeError("LayerNormSiLU needs CUDA tensors: there is no CPU path")
        xf, gf, bf = _f32(x), _f32(gamma), _f32(beta)
        rows, width = xf.shape
        y = torch.empty_like(xf)
        stats = torch.empty(2, rows, dtype=torch.float32, device=xf.device)
        with torch.cuda.device(xf.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_layernorm_silu_forward(rows, width, xf.data_ptr(), gf.data_ptr(),
                                                     bf.data_ptr(), float(eps), y.data_ptr(),
                                                     stats[0].data_ptr(), stats[1].data_ptr(), st),
                       "zp_layernorm_silu_forward")
        ctx.dtypes = (x.dtype, gamma.dtype, beta.dtype)
        ctx.save_for_backward(xf, gf, bf, stats)
        return y.to(x.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_y):
        lib = _lib.load()
        xf, gf, bf, stats = ctx.saved_tensors
        rows, width = xf.shape
        dy = _f32(grad_y)
        dx = torch.empty_like(xf)
        dgb = torch.empty(2, width, dtype=torch.float32, device=xf.device)
        nbytes = lib.zp_layernorm_work_bytes(width)
        work = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=xf.device)
        with torch.cuda.device(xf.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_layernorm_silu_backward(
                rows, width, xf.data_ptr(), gf.data_ptr(), bf.data_ptr(), stats[0].data_ptr(),
                stats[1].data_ptr(), dy.data_ptr(), dx.data_ptr(), dgb[0].data_ptr(),
                dgb[1].data_ptr(), work.data_ptr(), nbytes, st), "zp_layernorm_silu_backward")
        dt = ctx.dtypes
        return dx.to(dt[0]), dgb[0].to(dt[1]), dgb[1].to(dt[2]), None


class EdgeFeatures(torch.autograd.Function):
    """Geometry, Gaussian basis, element embeddings, envelope and the re-ordering of the roll-angle
    harmonics in one pass (``zp_edge_features_forward``), with the position / embedding gradients
    summed per atom in a fixed order by ``zp_edge_features_backward``.  Takes over
    blocks/eso2_ref.py:320-327 and :343 (the envelope value).  fp32, first order only.

    Returns (edge_vec [E,3], x_edge [E, NB + 2 EC], env [E], cos_sorted, sin_sorted), all in the
    graph's sorted edge order."""

    @staticmethod
    def forward(ctx, graph: EdgeGraph, perm32, front: "_lib.ZpFrontConfig", pos, shifts,
                atomic_numbers, emb, gauss_offset, cos_g, sin_g):
        """``perm32``: int32 positions of the graph's sorted edges in the caller's per-edge arrays
        (``graph.perm`` for a whole graph, a slice of the parent's for a chunk)."""
        lib = _lib.load()
        if not pos.is_cuda:
            raise RuntimeError("EdgeFeatures needs CUDA tensors: there is no CPU path")
        dev = pos.device
        n, e = graph.n_nodes, graph.n_edges
        posf, shf, embf, off = _f32(pos), _f32(shifts), _f32(emb), _f32(gauss_offset)
        cgf, sgf = _f32(cos_g), _f32(sin_g)
        zi = atomic_numbers.to(torch.int64).contiguous()
        f32 = dict(dtype=torch.float32, device=dev)
        width = front.num_basis + 2 * front.edge_channels
        edge_vec, dist = torch.empty(e, 3, **f32), torch.empty(e, **f32)
        x_edge, env = torch.empty(e, width, **f32), torch.empty(e, **f32)
        cs, ss = torch.empty(e, front.lmax + 1, **f32), torch.empty(e, front.lmax + 1, **f32)
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_edge_features_forward(
                ctypes.byref(front), n, e, posf.data_ptr(), shf.data_ptr(), zi.data_ptr(),
                embf.data_ptr(), off.data_ptr(), cgf.data_ptr(), sgf.data_ptr(),
                perm32.data_ptr(), graph.src.data_ptr(), graph.dst.data_ptr(),
                edge_vec.data_ptr(), dist.data_ptr(), x_edge.data_ptr(), env.data_ptr(),
                cs.data_ptr(), ss.data_ptr(), st), "zp_edge_features_forward")
        ctx.graph, ctx.front = graph, front
        ctx.dtypes = (pos.dtype, emb.dtype)
        ctx.n_elem = emb.shape[0]
        ctx.save_for_backward(edge_vec, dist, x_edge, off, zi)
        ctx.mark_non_differentiable(cs, ss)
        return edge_vec, x_edge, env, cs, ss

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_edge_vec, g_x_edge, g_env, _gc, _gs):
        lib = _lib.load()
        edge_vec, dist, x_edge, off, zi = ctx.saved_tensors
        graph, front = ctx.graph, ctx.front
        n, e = graph.n_nodes, graph.n_edges
        dev = edge_vec.device
        g_pos = torch.empty(n, 3, dtype=torch.float32, device=dev)
        need_emb = ctx.needs_input_grad[6]
        g_emb = torch.empty(ctx.n_elem, front.edge_channels, dtype=torch.float32,
                            device=dev) if need_emb else None
        ptr = lambda t: None if t is None else _f32(t)            # noqa: E731
        gev, gxe, gen = ptr(g_edge_vec), ptr(g_x_edge), ptr(g_env)
        nbytes = lib.zp_edge_features_work_bytes(ctypes.byref(front), n, e)
        work = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        dp = lambda t: None if t is None else t.data_ptr()        # noqa: E731
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_edge_features_backward(
                ctypes.byref(front), n, e, edge_vec.data_ptr(), dist.data_ptr(), x_edge.data_ptr(),
                off.data_ptr(), zi.data_ptr(), dp(gev), dp(gxe), dp(gen), graph.row_ptr.data_ptr(),
                graph.perm_src.data_ptr(), graph.row_ptr_src.data_ptr(), g_pos.data_ptr(),
                dp(g_emb), work.data_ptr(), nbytes, st), "zp_edge_features_backward")
        dt = ctx.dtypes
        return (None, None, None, g_pos.to(dt[0]), None, None,
                g_emb.to(dt[1]) if need_emb else None, None, None, None)


class Readout(torch.autograd.Function):
    """E = sum_n Linear(C -> 1)(SiLU(Linear((lmax+1)C -> C)(invariants(node_out[n])))) and its VJP
    (``zp_readout_forward`` / ``zp_readout_backward``; reference blocks/eso2_ref.py:351-362).
    The gradient it returns for ``node_out`` is the upstream gradient of the edge convolution's
    backward in a force evaluation.  First order only."""

    @staticmethod
    def forward(ctx, plan: Plan, node_out, w0, b0, w1, b1):
        lib = _lib.load()
        if not node_out.is_cuda:
            raise RuntimeError("Readout needs CUDA tensors: there is no CPU path")
        x, w0f, b0f, w1f, b1f = (_f32(t) for t in (node_out, w0, b0, w1.reshape(-1), b1))
        n = x.shape[0]
        nbytes = lib.zp_readout_work_bytes(plan.handle, n)
        work = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        energy = torch.empty(1, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_readout_forward(plan.handle, n, x.data_ptr(), w0f.data_ptr(),
                                              b0f.data_ptr(), w1f.data_ptr(), b1f.data_ptr(),
                                              energy.data_ptr(), work.data_ptr(), work.numel(), st),
                       "zp_readout_forward")
        ctx.plan = plan
        ctx.shapes = (w1.shape, [t.dtype for t in (node_out, w0, b0, w1, b1)])
        ctx.save_for_backward(x, w0f, b0f, w1f, b1f, work)
        return energy.reshape(()).to(node_out.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_e):
        lib = _lib.load()
        x, w0f, b0f, w1f, b1f, work = ctx.saved_tensors
        n = x.shape[0]
        ge = _f32(grad_e).reshape(1)
        gx, gw0, gb0, gw1, gb1 = (torch.empty_like(t) for t in (x, w0f, b0f, w1f, b1f))
        with torch.cuda.device(x.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.zp_readout_backward(
                ctx.plan.handle, n, x.data_ptr(), w0f.data_ptr(), b0f.data_ptr(), w1f.data_ptr(),
                b1f.data_ptr(), ge.data_ptr(), gx.data_ptr(), gw0.data_ptr(), gb0.data_ptr(),
                gw1.data_ptr(), gb1.data_ptr(), work.data_ptr(), work.numel(), st),
                "zp_readout_backward")
        w1_shape, dts = ctx.shapes
        return (None, gx.to(dts[0]), gw0.to(dts[1]), gb0.to(dts[2]),
                gw1.reshape(w1_shape).to(dts[3]), gb1.to(dts[4]))


def tensor_core_linear(plan: Plan, x: torch.Tensor, weight: torch.Tensor, bias) -> torch.Tensor:
    """``x @ weight.T + bias`` through ``TensorCoreLinear`` for any sizes: the engine wants inner
    and outer widths in multiples of 8, so odd ones are zero-padded (and the result sliced)."""
    n_out, n_in = weight.shape
    pad_in, pad_out = (-n_in) % 8, (-n_out) % 8
    if bias is None:
        bias = weight.new_zeros(n_out)
    if pad_in or pad_out:
        # narrow, odd-sized layers keep fp32 accuracy whatever the plan's operand format is
        # (they cost next to nothing; the bf16 format is meant for the wide products)
        plan = Plan.get(plan.lmax, plan.mmax, plan.c, plan.h, plan.device, precision=2)
        x = torch.nn.functional.pad(x, (0, pad_in))
        weight = torch.nn.functional.pad(weight, (0, pad_in, 0, pad_out))
        bias = torch.nn.functional.pad(bias, (0, pad_out))
    y = TensorCoreLinear.apply(plan, x, weight, bias)
    return y[:, :n_out] if pad_out else y


def radial_mlp(plan: Plan, x_edge: torch.Tensor, layers: list) -> torch.Tensor:
    """A ``Linear / LayerNorm / SiLU`` stack (the reference's ``rad_func``) on the library's
    kernels.  ``layers``: modules, or for a functional caller tuples ``("linear", w, b)`` /
    ``("ln_silu", gamma, beta, eps)``."""
    h, i = x_edge, 0
    while i < len(layers):
        m = layers[i]
        if isinstance(m, tuple):
            h = (tensor_core_linear(plan, h, m[1], m[2]) if m[0] == "linear"
                 else LayerNormSiLU.apply(h, m[1], m[2], m[3]))
            i += 1
        elif isinstance(m, nn.Linear):
            h = tensor_core_linear(plan, h, m.weight, m.bias) if h.shape[0] else h.new_zeros(0, m.out_features)
            i += 1
        elif isinstance(m, nn.LayerNorm) and i + 1 < len(layers) and isinstance(layers[i + 1], nn.SiLU):
            h = LayerNormSiLU.apply(h, m.weight, m.bias, m.eps) if h.shape[0] else h
            i += 2
        else:
            raise _lib.ZpError(2, f"radial MLP layer {type(m).__name__} (no kernel for it)")
    return h


def edge_conv(plan: Plan, graph: EdgeGraph, x_node, edge_vec, cos_g, sin_g, radial, env,
              c1_m0: nn.Linear, c1_m, c2_m0: nn.Linear, c2_m, rad_w=None, rad_b=None) -> torch.Tensor:
    """``rad_w`` / ``rad_b``: see ``EdgeConvFunction`` (``radial`` is then the last radial
    layer's input)."""
    return EdgeConvFunction.apply(plan, graph, x_node, edge_vec, cos_g, sin_g, radial, env,
                                  rad_w, rad_b, c1_m0.weight, c1_m0.bias, c2_m0.weight, c2_m0.bias,
                                  *[l.weight for l in c1_m], *[l.weight for l in c2_m])


# --------------------------------------------------------------------------------------------
# the module
# --------------------------------------------------------------------------------------------


class ESO2Block(nn.Module):
    """One SO(2) interaction block + per-atom energy head, reference call signature."""

    PRECISIONS = {"fp32": 2, "fp32_bf16x3": 0, "bf16": 1}

    def __init__(self, cfg: BlockConfig = BlockConfig(), precision: str = "fp32"):
        """``precision`` of the SO(2) contraction's operands: "fp32" carries each value as two
        fp16 terms with per-tensor power-of-two scales derived on the device (22 bits, three
        tensor-core passes); "fp32_bf16x3" as three bf16 terms (24 bits, six passes, no scales);
        "bf16" rounds operands to bf16.  Accumulation is fp32 in all three."""
        super().__init__()
        if cfg.edge_channels % 4 or not 0 < cfg.edge_channels <= 1024:
            raise ValueError("edge_channels must be a multiple of 4 in [4, 1024]: the front-end and "
                             "LayerNorm kernels take no other width, and there is no other path")
        self.cfg = cfg
        self.precision = self.PRECISIONS[precision]
        self.layout = Layout.make(cfg.lmax, cfg.mmax)
        L, C, H = cfg.lmax, cfg.sphere_channels, cfg.hidden_channels
        ms = self.layout.m_size

        self.elem_emb = nn.Embedding(cfg.max_num_elements, cfg.edge_channels)
        offset = torch.linspace(0.0, cfg.cutoff, cfg.num_distance_basis)     # fp32, as the reference
        self.register_buffer("gauss_offset", offset, persistent=False)
        self.gauss_coeff = -0.5 / (offset[1] - offset[0]).item() ** 2

        self.edge_split = [k * 2 * C for k in ms]
        self.num_channels_rad = sum(self.edge_split)
        widths = [*cfg.edge_channels_list, self.num_channels_rad]
        layers: list[nn.Module] = []
        for i in range(1, len(widths)):
            layers.append(nn.Linear(widths[i - 1], widths[i]))
            if i < len(widths) - 1:
                layers += [nn.LayerNorm(widths[i]), nn.SiLU()]
        self.rad_func = nn.Sequential(*layers)

        self.extra_m0 = L * H
        self.c1_m0 = nn.Linear(ms[0] * 2 * C, H * (L + 1) + self.extra_m0)
        self.c1_m = nn.ModuleList(nn.Linear(ms[m] * 2 * C, 2 * H * ms[m], bias=False)
                                  for m in range(1, cfg.mmax + 1))
        self.c2_m0 = nn.Linear(ms[0] * H, C * (L + 1))
        self.c2_m = nn.ModuleList(nn.Linear(ms[m] * H, 2 * C * ms[m], bias=False)
                                  for m in range(1, cfg.mmax + 1))
        with torch.no_grad():
            for lin in (*self.c1_m, *self.c2_m):
                lin.weight.mul_(1.0 / math.sqrt(2.0))
        self.readout = nn.Sequential(nn.Linear(C * (L + 1), C), nn.SiLU(), nn.Linear(C, 1))
        self._jd_seen: set = set()
        p = float(cfg.envelope_exponent)
        self.env_p, self.env_a = p, -(p + 1) * (p + 2) / 2
        self.env_b, self.env_c = p * (p + 2), -p * (p + 1) / 2

    # -- small torch pieces ---------------------------------------------------------------
    def envelope(self, d_scaled: torch.Tensor) -> torch.Tensor:
        val = 1 + d_scaled ** self.env_p * (self.env_a + d_scaled * (self.env_b + self.env_c * d_scaled))
        return torch.where(d_scaled < 1, val, torch.zeros_like(val))

    def gaussian_basis(self, dist: torch.Tensor) -> torch.Tensor:
        d = dist.unsqueeze(1) - self.gauss_offset.to(dist.dtype).unsqueeze(0)
        return torch.exp(self.gauss_coeff * d * d)

    def node_invariants(self, node_out: torch.Tensor) -> torch.Tensor:
        feats = [node_out[:, 0, :]]
        for l in range(1, self.cfg.lmax + 1):
            feats.append(node_out[:, l * l:(l + 1) ** 2, :].pow(2).sum(dim=1))
        return torch.cat(feats, dim=-1)

    def front_config(self) -> "_lib.ZpFrontConfig":
        c = self.cfg
        return _lib.ZpFrontConfig(c.lmax, c.num_distance_basis, c.edge_channels,
                                  c.max_num_elements, c.envelope_exponent, float(c.cutoff),
                                  float(self.gauss_coeff))

    def plan(self, device) -> Plan:
        c = self.cfg
        return Plan.get(c.lmax, c.mmax, c.sphere_channels, c.hidden_channels, device,
                        self.precision)

    def radial_mlp(self, plan: Plan, x_edge: torch.Tensor) -> torch.Tensor:
        """rad_func (Linear, LayerNorm, SiLU, ..., Linear; reference eso2_ref.py:164-182) on the
        library's kernels: every Linear on the contraction engine in the plan's operand format
        (widths that are not multiples of 8 are zero-padded to the next one, which changes no
        value), every LayerNorm + SiLU pair as one fused pass."""
        return radial_mlp(plan, x_edge, list(self.rad_func))

    # -- forward --------------------------------------------------------------------------
    def _edges_to_nodes(self, plan, graph, perm, pos, atomic_numbers, x_node, shifts, cos_gamma_k,
                        sin_gamma_k, x_ready=None) -> torch.Tensor:
        """Geometry, radial features, envelope and the edge convolution for the edges of `graph`
        (whose original positions in the caller's arrays are `perm`)."""
        cfg = self.cfg

        def conv(*args):
            if x_ready is not None:        # x_node is still arriving on another stream
                torch.cuda.current_stream(pos.device).wait_event(x_ready)
            return edge_conv(*args)

        # geometry, distance basis, embeddings, envelope and the sorted copies in one pass
        edge_vec, x_edge, env, cos_s, sin_s = EdgeFeatures.apply(
            graph, perm.to(torch.int32).contiguous(), self.front_config(), pos, shifts,
            atomic_numbers, self.elem_emb.weight, self.gauss_offset, cos_gamma_k, sin_gamma_k)
        last = self.rad_func[-1]
        if isinstance(last, nn.Linear) and last.in_features % 8 == 0 and graph.n_edges > 0:
            # the last (widest) radial layer runs inside the edge-convolution call: its output
            # and that output's gradient never leave the kernel path
            h_rad = radial_mlp(plan, x_edge, list(self.rad_func)[:-1])
            return conv(plan, graph, x_node, edge_vec, cos_s, sin_s, h_rad, env,
                        self.c1_m0, self.c1_m, self.c2_m0, self.c2_m, last.weight, last.bias)
        radial = self.radial_mlp(plan, x_edge)
        return conv(plan, graph, x_node, edge_vec, cos_s, sin_s, radial, env,
                    self.c1_m0, self.c1_m, self.c2_m0, self.c2_m)

    def node_output(self, pos, atomic_numbers, x_node, edge_index, shifts, cos_gamma_k,
                    sin_gamma_k, graph: EdgeGraph | None = None,
                    x_ready: "torch.cuda.Event | None" = None) -> torch.Tensor:
        """pos -> node_out [N, K, C] (what the reference scatters at eso2_ref.py:346-349).

        ``x_ready``: an event after which ``x_node`` is valid (its host-to-device copy runs on
        another stream); the current stream waits for it only where the embeddings are first
        read, so the copy overlaps the edge sort, the front end and the radial MLP.

        Graphs whose per-edge activations (radial features included) exceed the memory budget
        are processed as destination-node chunks under activation checkpointing: each chunk's
        forward is recomputed in the backward, so memory stays bounded by one chunk."""
        n = pos.shape[0]
        if graph is None:
            # new input: node indices are range-checked by the sort, element numbers here (a
            # caller that passes a prebuilt graph has had both checked when it was built)
            graph = EdgeGraph.build(edge_index, n)
            if (atomic_numbers.numel() and not torch.cuda.is_current_stream_capturing()
                    and not bool(((atomic_numbers >= 0)
                                  & (atomic_numbers < self.cfg.max_num_elements)).all())):
                raise IndexError(f"atomic_numbers outside [0, {self.cfg.max_num_elements})")
        plan = self.plan(pos.device)
        # radial features and their gradients roughly double the per-edge footprint
        budget = max(1024, _edge_budget(plan, n, graph.n_edges) // 2)
        chunks = graph.chunks(budget)
        perm = graph.perm64
        if len(chunks) == 1:
            return self._edges_to_nodes(plan, graph, perm, pos, atomic_numbers, x_node, shifts,
                                        cos_gamma_k, sin_gamma_k, x_ready)
        if x_ready is not None:
            torch.cuda.current_stream(pos.device).wait_event(x_ready)
        from torch.utils.checkpoint import checkpoint
        outs = []
        for c in chunks:
            sub_perm = perm[c.e0:c.e1]

            def run(pos_, x_, c=c, sub_perm=sub_perm):
                return self._edges_to_nodes(plan, c.sub, sub_perm, pos_, atomic_numbers, x_, shifts,
                                            cos_gamma_k, sin_gamma_k)

            if torch.is_grad_enabled():
                outs.append(checkpoint(run, pos, x_node, use_reentrant=False))
            else:
                outs.append(run(pos, x_node))
        return torch.cat(outs, dim=0)

    def node_output_vjp(self, pos, atomic_numbers, x_node, edge_index, shifts, cos_gamma_k,
                        sin_gamma_k, upstream, graph: EdgeGraph | None = None):
        """node_out and the vector-Jacobian product of <node_out, upstream> in one sweep over
        destination-node chunks, WITHOUT recomputing any forward.

        A chunk's rows of node_out are final as soon as the chunk's forward has run (a chunk holds
        every edge into its nodes), so when the upstream gradient of a row depends on that row
        alone the chunk's backward can follow at once and its activations be dropped.  ``upstream``
        is either the gradient tensor [N, K, C] or a callable ``(rows, n0, n1) -> gradient of
        rows`` (e.g. the derivative of a per-atom readout, reference eso2_ref.py:351-362, evaluated
        on rows ``n0:n1``).  ``node_output`` + autograd has to keep or recompute every chunk
        (one extra forward per chunk); this entry point does three passes' worth of work instead
        of four on graphs that do not fit one call.

        Returns ``(node_out, grad_x_node, grad_pos, param_grads)`` with ``param_grads`` in the
        order of ``self.parameters()`` (``None`` for parameters the node output does not use).
        """
        n = pos.shape[0]
        if graph is None:
            graph = EdgeGraph.build(edge_index, n)
        plan = self.plan(pos.device)
        budget = max(1024, _edge_budget(plan, n, graph.n_edges) // 2)
        chunks = graph.chunks(budget)
        perm = graph.perm64
        params = list(self.parameters())
        gx = torch.zeros_like(x_node)
        gpos = torch.zeros_like(pos)
        gparams: list = [None] * len(params)
        outs = []
        for c in chunks:
            if len(chunks) > 1:
                sub_graph, sub_perm = c.sub, perm[c.e0:c.e1]
            else:
                sub_graph, sub_perm = graph, perm
            pos_ = pos.detach().requires_grad_(True)
            x_ = x_node.detach().requires_grad_(True)
            with torch.enable_grad():
                rows = self._edges_to_nodes(plan, sub_graph, sub_perm, pos_, atomic_numbers, x_,
                                            shifts, cos_gamma_k, sin_gamma_k)
            g_rows = (upstream(rows.detach(), c.n0, c.n1) if callable(upstream)
                      else upstream[c.n0:c.n1])
            grads = torch.autograd.grad(rows, [x_, pos_, *params], g_rows, allow_unused=True)
            gx += grads[0]
            gpos += grads[1]
            for i, g in enumerate(grads[2:]):
                if g is not None:
                    gparams[i] = g if gparams[i] is None else gparams[i].add_(g)
            outs.append(rows.detach())
            del rows, grads, g_rows
        node_out = outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)
        return node_out, gx, gpos, gparams

    def _check_jd(self, jd) -> None:
        """The kernels hold the J matrices shipped with the package; a caller's ``jd`` (the
        reference passes ``blocks/Jd.pt``) must be those same matrices.  Checked once per list."""
        if jd is None or id(jd) in self._jd_seen:
            return
        want = load_jd(self.cfg.lmax)
        if len(jd) <= self.cfg.lmax:
            raise ValueError(f"jd has {len(jd)} matrices, lmax = {self.cfg.lmax} needs {self.cfg.lmax + 1}")
        for l, w in enumerate(want):
            got = torch.as_tensor(jd[l]).detach().to("cpu", torch.float64)
            if got.shape != w.shape or not torch.allclose(got, w, rtol=0.0, atol=1e-6):
                raise ValueError(f"jd[{l}] differs from the J matrix the kernels were built with "
                                 "(zippel_b200/data/jd.npz = the reference's blocks/Jd.pt)")
        self._jd_seen.add(id(jd))

    def forward(self, pos, atomic_numbers, x_node, edge_index, shifts, cos_gamma_k, sin_gamma_k,
                jd=None, graph: EdgeGraph | None = None) -> torch.Tensor:
        """Scalar E.  ``jd`` (the reference's argument) is verified against the J matrices the
        kernels use; anything else raises ``ValueError``."""
        self._check_jd(jd)
        node_out = self.node_output(pos, atomic_numbers, x_node, edge_index, shifts,
                                    cos_gamma_k, sin_gamma_k, graph)
        return self.energy(node_out)

    def energy(self, node_out: torch.Tensor) -> torch.Tensor:
        """The readout head on the library's kernels (``Readout``): invariants, two dense layers,
        sum over atoms."""
        lin0, lin1 = self.readout[0], self.readout[2]
        return Readout.apply(self.plan(node_out.device), node_out, lin0.weight, lin0.bias,
                             lin1.weight, lin1.bias)
