"""zp_csr_build_static: the edge sort for callers that may not allocate device memory (its scratch
is a fixed array inside the library instead of a caller-provided work buffer).

Collected last on purpose, so that a run stopping at the first failure has already run every
other test.  The check: called through the C ABI on two different graphs back to back (the
second call finds the first call's leftovers in the shared array), its six output arrays must be
bit-identical to those of zp_csr_build on the same input; oversize requests must be refused."""

from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_build(lib, ei: torch.Tensor, n: int):
    e = ei.shape[1]
    i32 = dict(dtype=torch.int32, device=ei.device)
    perm, src, dst, perm_src = (torch.full((max(e, 1),), -7, **i32) for _ in range(4))
    row_ptr, row_ptr_src = (torch.full((n + 1,), -7, **i32) for _ in range(2))
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.zp_csr_build_static(ei.data_ptr(), e, n, perm.data_ptr(), src.data_ptr(),
                                 dst.data_ptr(), row_ptr.data_ptr(), perm_src.data_ptr(),
                                 row_ptr_src.data_ptr(), st)
    return rc, dict(perm=perm[:e], src=src[:e], dst=dst[:e], row_ptr=row_ptr,
                    perm_src=perm_src[:e], row_ptr_src=row_ptr_src)


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    from zippel_b200 import _lib
    from zippel_b200.graph import EdgeGraph
    lib = _lib.load()
    for n, e, seed in [(4000, 90000, 1), (300, 5000, 2)]:      # larger first, then smaller
        g = torch.Generator("cpu").manual_seed(seed)
        ei = torch.randint(0, n, (2, e), generator=g).cuda()
        rc, got = _static_build(lib, ei, n)
        assert rc == 0, lib.zp_status_string(rc)
        want = EdgeGraph.build(ei, n)
        torch.cuda.synchronize()
        for key, val in got.items():
            assert np.array_equal(val.cpu().numpy(), getattr(want, key).cpu().numpy()), (key, n)


def test_static_scratch_refuses_sizes_beyond_its_capacity():
    from zippel_b200 import _lib
    lib = _lib.load()
    ei = torch.zeros(2, 8, dtype=torch.int64, device="cuda")
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    args = [dummy.data_ptr()] * 6 + [None]
    assert lib.zp_csr_build_static(ei.data_ptr(), 262145, 10, *args) == 7
    assert lib.zp_csr_build_static(ei.data_ptr(), 8, 65537, *args) == 7
    assert b"capacity" in lib.zp_status_string(7)


@pytest.mark.parametrize("n,e", [(65536, 262144), (65536, 0), (17, 0)])
def test_static_scratch_at_its_limits(n, e):
    """Exactly at the two maxima the sort's scratch fills the fixed array to the byte; an empty edge
    list is legal.  Results equal zp_csr_build's bit for bit."""
    from zippel_b200 import _lib
    from zippel_b200.graph import EdgeGraph
    lib = _lib.load()
    assert lib.zp_csr_work_bytes(262144, 65536) == 1574144            # ZP_CSR_STATIC_BYTES
    g = torch.Generator("cpu").manual_seed(n + e)
    ei = torch.randint(0, n, (2, e), generator=g).cuda()
    rc, got = _static_build(lib, ei, n)
    assert rc == 0, lib.zp_status_string(rc)
    want = EdgeGraph.build(ei, n)
    torch.cuda.synchronize()
    for key, val in got.items():
        assert np.array_equal(val.cpu().numpy(), getattr(want, key).cpu().numpy()), key


def test_static_scratch_flags_node_indices_out_of_range():
    """An index outside [0, N) must not be used as an address into the fixed array: the edge is
    left out and the status call reports it; the next, valid call is clean again."""
    import ctypes
    from zippel_b200 import _lib
    lib = _lib.load()
    ei = torch.tensor([[0, 1, 2, 3], [1, 2, 99, 0]], dtype=torch.int64, device="cuda")
    rc, got = _static_build(lib, ei, 4)
    assert rc == 0
    flag = ctypes.c_int(0)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.zp_csr_static_status(st, ctypes.byref(flag)) == 0 and flag.value == 1
    assert got["row_ptr"].cpu().tolist() == [0, 1, 2, 3, 3]           # three edges counted
    ei[1, 2] = 3
    rc, _ = _static_build(lib, ei, 4)
    assert rc == 0 and lib.zp_csr_static_status(st, ctypes.byref(flag)) == 0 and flag.value == 0
