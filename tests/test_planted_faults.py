"""The parity comparison must be able to fail (after the reference's
tests/test_planted_faults.py:122-221: dropped term, transposed index, off-by-one channel slice).

Each fault is planted in the ORACLE-side expectation; the 1e-5 relative-L2 check used by every
parity test must then trip -- against the reference's golden vectors on the CPU, and against the
CUDA path on a GPU -- while the unmodified oracle passes."""

from __future__ import annotations

import pytest
import torch

from oracle import eso2_oracle as orc
from tests.conftest import load_golden
from tests.helpers import oracle_node_out_and_vjp, random_case, rel_l2

TOL = 1e-5


def _drop_term(monkeypatch):
    """m > 0 blocks lose the cross term of the real part (out_re = Wa x_re - Wb x_im)."""
    real = torch.nn.functional.linear

    def so2_conv(x, w0, b0, wm, lmax, mmax, c_out, radial, n_gate):
        e, cin = x.shape[0], x.shape[2]
        ms, split = orc.m_sizes(lmax, mmax), orc.m_splits(lmax, mmax)
        by_m = x.split(split, dim=1)
        rad_m = radial.split([k * cin for k in ms], dim=1) if radial is not None else None
        x0 = by_m[0].reshape(e, -1)
        if rad_m is not None:
            x0 = x0 * rad_m[0]
        y0 = real(x0, w0, b0)
        gate = None
        if n_gate:
            gate, y0 = y0[:, :n_gate], y0[:, n_gate:]
        out = [y0.reshape(e, -1, c_out)]
        for m in range(1, mmax + 1):
            xm = by_m[m].reshape(e, 2, -1)
            if rad_m is not None:
                xm = xm * rad_m[m][:, None, :]
            ym = real(xm, wm[m - 1])
            half = ym.shape[-1] // 2
            out.append(ym[:, 0, :half].reshape(e, -1, c_out))             # "- Wb x_im" dropped
            out.append((ym[:, 1, :half] + ym[:, 0, half:]).reshape(e, -1, c_out))
        return torch.cat(out, dim=1), gate

    monkeypatch.setattr(orc, "so2_conv", so2_conv)


def _transpose_index(monkeypatch):
    """The gate scalars are looked up with the degree index reversed."""
    real = orc.gate_expand_index
    monkeypatch.setattr(orc, "gate_expand_index",
                        lambda lmax, mmax: (lmax - 1) - real(lmax, mmax))


def _shift_channel_slice(monkeypatch):
    """conv1 reads the message as [x_dst ; x_src] instead of [x_src ; x_dst]: every channel slice
    of its input is off by C (planted by exchanging the two halves of conv1's input weights)."""
    real = orc.edge_conv

    def edge_conv(params, x_node, edge_index, *rest):
        p, c = dict(params), x_node.shape[2]
        for k in [k for k in p if k.startswith("c1_") and k.endswith("weight")]:
            w = p[k].reshape(p[k].shape[0], -1, 2 * c)
            p[k] = torch.cat([w[..., c:], w[..., :c]], dim=-1).reshape(p[k].shape)
        return real(p, x_node, edge_index, *rest)

    monkeypatch.setattr(orc, "edge_conv", edge_conv)


FAULTS = {"dropped_term": _drop_term, "transposed_index": _transpose_index,
          "shifted_channel_slice": _shift_channel_slice}


def _golden_errors(c, jd):
    got = oracle_node_out_and_vjp(c["cfg"], c["params"], c, c["upstream"], jd)
    return rel_l2(got[0], c["node_out"]), rel_l2(got[1], c["vjp_x_node"]), rel_l2(got[2], c["vjp_pos"])


@pytest.mark.parametrize("fault", sorted(FAULTS))
def test_planted_fault_trips_the_golden_comparison(fault, jd64, monkeypatch):
    c = load_golden("ref_l2m2_c8")
    assert max(_golden_errors(c, jd64)) < 1e-12                 # the unmodified oracle passes
    FAULTS[fault](monkeypatch)
    errs = _golden_errors(c, jd64)
    assert min(errs[0], errs[1]) > 100 * TOL, (fault, errs)     # output AND a gradient are off


@pytest.mark.gpu
@pytest.mark.parametrize("fault", sorted(FAULTS))
def test_planted_fault_trips_the_gpu_comparison(fault, jd64, monkeypatch):
    from tests.helpers import check_against, gpu_node_out_and_vjp, make_block
    cfg = dict(lmax=4, mmax=2, sphere_channels=16, hidden_channels=16, edge_channels=8,
               num_distance_basis=6, cutoff=5.0)
    params = orc.init_params(cfg, seed=13)
    case = random_case(cfg, 14, 120, seed=14)
    got = gpu_node_out_and_vjp(make_block(cfg, params), case, case["upstream"])
    check_against(*got, *oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64))
    FAULTS[fault](monkeypatch)
    wrong = oracle_node_out_and_vjp(cfg, params, case, case["upstream"], jd64)
    with pytest.raises(AssertionError):
        check_against(*got, *wrong)
    assert rel_l2(got[0], wrong[0]) > 100 * TOL
