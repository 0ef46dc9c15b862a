"""The tensor-core contraction engine on its own (zp_gemm_planes through the C ABI) against
fp64 products of the same inputs.  Tolerances: with three planes the result must match the
fp32 x fp32 product to 4e-6 relative L2 (the engine's own budget inside the 1e-5 block
tolerance); with one plane it must match the product of the bf16-rounded operands to 4e-6."""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def run_gemm(M, N, K, planes, a_mn, b_mn, variant=0, ksplit=1, kc=0, bias=True, seed=0):
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import Plan
    lib, plan = _lib.load(), Plan.get(2, 2, 8, 8, "cuda")
    g = torch.Generator("cpu").manual_seed(seed)
    A = torch.randn(M, K, generator=g)
    B = torch.randn(N, K, generator=g) * 0.1
    bvec = torch.randn(N, generator=g) if bias else None

    def planes_of(X, mn):
        Xs = (X.t() if mn else X).contiguous().cuda()
        rows, cols = Xs.shape
        ld = (cols + 7) // 8 * 8
        out = torch.zeros(planes, rows, ld, device="cuda",
                          dtype=torch.float16 if planes == 2 else torch.bfloat16)
        _lib.check(lib.zp_split_planes(rows, cols, Xs.data_ptr(), cols, out.data_ptr(), ld,
                                       rows * ld, planes, None), "zp_split_planes")
        return out, ld, rows * ld

    Ap, lda, aps = planes_of(A, a_mn)
    Bp, ldb, bps = planes_of(B, b_mn)
    ldc = (N + 3) // 4 * 4
    C = torch.full((max(ksplit, 1), M, ldc), float("nan"), device="cuda")
    bd = bvec.cuda() if bias else None
    used = ctypes.c_int(0)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.zp_gemm_planes(plan.handle, M, N, K, planes, Ap.data_ptr(), lda, aps, int(a_mn),
                                  Bp.data_ptr(), ldb, bps, int(b_mn),
                                  bd.data_ptr() if bias else None, C.data_ptr(), ldc, variant,
                                  ksplit, M * ldc, kc, ctypes.byref(used), st), "zp_gemm_planes")
    torch.cuda.synchronize()
    stat = ctypes.c_int(0)
    _lib.check(lib.zp_plan_device_status(plan.handle, ctypes.byref(stat)), "status")
    assert stat.value == 0
    assert 1 <= used.value <= max(ksplit, 1)
    got = C[:used.value, :, :N].double().sum(0).cpu()
    Ar = Ap.double().sum(0).cpu()
    Br = Bp.double().sum(0).cpu()
    Ar = Ar[:, :M].t() if a_mn else Ar[:, :K]
    Br = Br[:, :N].t() if b_mn else Br[:, :K]
    ref_planes = Ar[:M, :K] @ Br[:N, :K].t() + (bvec.double() if bias else 0)
    ref_fp32 = A.double() @ B.double().t() + (bvec.double() if bias else 0)
    rel = lambda x, y: ((x - y).norm() / y.norm()).item()  # noqa: E731
    return rel(got, ref_planes), rel(got, ref_fp32)


SHAPES = [(128, 128, 64), (300, 200, 100), (1000, 1152, 1280), (129, 20, 24), (77, 640, 2048)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("variant", [0, 1])
def test_three_planes_k_major(M, N, K, variant):
    _, err = run_gemm(M, N, K, 3, False, False, variant=variant)
    assert err < 4e-6


@pytest.mark.parametrize("M,N,K", SHAPES + [(700, 1152, 1280), (513, 48, 72)])
@pytest.mark.parametrize("variant", [2, 3])          # 2 = single-CTA kernel, 3 = CTA-pair kernel
def test_two_fp16_planes_k_major(M, N, K, variant):
    _, err = run_gemm(M, N, K, 2, False, False, variant=variant)
    assert err < 4e-6


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_one_plane_k_major(M, N, K):
    err, _ = run_gemm(M, N, K, 1, False, False)
    assert err < 4e-6


@pytest.mark.parametrize("planes,variant", [(1, 0), (2, 2), (2, 3), (3, 0), (3, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 192, 200), (1152, 1280, 5000), (24, 40, 333)])
def test_mn_major_operands(M, N, K, planes, variant):
    err_p, err_f = run_gemm(M, N, K, planes, True, True, variant=variant)
    assert (err_p if planes == 1 else err_f) < 4e-6


def test_mixed_majors():
    assert run_gemm(300, 256, 512, 3, True, False, variant=1)[1] < 4e-6
    assert run_gemm(300, 256, 512, 3, False, True, variant=1)[1] < 4e-6


@pytest.mark.parametrize("planes,variant", [(1, 0), (2, 2), (2, 3), (3, 0)])
def test_long_contraction_chunks_and_splits(planes, variant):
    """Contraction over 60 000 'edges' as in the weight gradients: chunked TMEM accumulation plus
    a split over CTAs must hold the tolerance that a single running accumulator cannot."""
    err_p, err_f = run_gemm(640, 512, 60000, planes, True, True, variant=variant, ksplit=4, bias=False)
    assert (err_p if planes == 1 else err_f) < 4e-6
    err_p, err_f = run_gemm(256, 256, 9000, planes, False, False, variant=variant, ksplit=3, kc=512,
                            bias=True)
    assert (err_p if planes == 1 else err_f) < 4e-6


def test_mixed_majors_pair():
    assert run_gemm(300, 256, 512, 2, True, False, variant=3)[1] < 4e-6
    assert run_gemm(300, 128, 512, 2, False, True, variant=3)[1] < 4e-6


@pytest.mark.parametrize("precision", [0, 1, 2])
@pytest.mark.parametrize("M,K,N", [(1000, 128, 3072), (77, 40, 24), (0, 16, 8)])
def test_tensor_core_linear_and_vjp(M, K, N, precision):
    """zp_linear_forward/backward against fp64 torch (bf16 operands: 2e-2, else 4e-6)."""
    from zippel_b200.blocks.eso2 import Plan, TensorCoreLinear
    plan = Plan.get(2, 2, 8, 8, "cuda", precision)
    g = torch.Generator("cpu").manual_seed(M + N)
    x = torch.randn(M, K, generator=g, dtype=torch.float64)
    w = torch.randn(N, K, generator=g, dtype=torch.float64) * 0.1
    b = torch.randn(N, generator=g, dtype=torch.float64)
    up = torch.randn(M, N, generator=g, dtype=torch.float64)
    xr, wr, br = (t.clone().requires_grad_(True) for t in (x, w, b))
    want = torch.nn.functional.linear(xr, wr, br)
    gx, gw, gb = torch.autograd.grad((want * up).sum(), [xr, wr, br])
    xc, wc, bc = (t.float().cuda().requires_grad_(True) for t in (x, w, b))
    got = TensorCoreLinear.apply(plan, xc, wc, bc)
    hx, hw, hb = torch.autograd.grad((got * up.float().cuda()).sum(), [xc, wc, bc])
    tol = 2e-2 if precision == 1 else 4e-6
    rel = lambda a, r: ((a.double().cpu() - r).norm() / r.norm().clamp_min(1e-300)).item()  # noqa: E731
    if M:
        assert rel(got, want.detach()) < tol and rel(hx, gx) < tol and rel(hw, gw) < tol
        assert rel(hb, gb) < tol
    else:
        assert got.shape == (0, N) and hw.abs().max().item() == 0.0
    assert plan.device_status() == 0


def test_bounded_wait_runs_out_and_the_library_keeps_working():
    """A wait that nothing will ever satisfy: the kernel must give up after its time limit, record
    ZP_ERR_DEVICE_TIMEOUT in the plan's status word and return with every warp (no trap, no hang);
    the status reads once and clears, and the next product is correct."""
    import ctypes
    import time
    from zippel_b200 import _lib
    from zippel_b200.blocks.eso2 import Plan
    lib = _lib.load()
    plan = Plan.get(2, 2, 8, 8, "cuda", precision=1)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    scratch = torch.empty(64 << 10, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    _lib.check(lib.zp_selftest_bounded_wait(plan.handle, scratch.data_ptr(), scratch.numel(),
                                            3_000_000, st), "zp_selftest_bounded_wait")   # 3 ms
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0                     # it returned, and soon
    assert plan.device_status() == 5                          # ZP_ERR_DEVICE_TIMEOUT
    assert plan.device_status() == 0                          # read once, then clear
    # a normal product afterwards
    g = torch.Generator("cpu").manual_seed(0)
    a = torch.randn(200, 96, generator=g).cuda()
    b = torch.randn(72, 96, generator=g).cuda()
    ap, bp = torch.empty(200, 96, dtype=torch.bfloat16, device="cuda"), torch.empty(72, 96, dtype=torch.bfloat16, device="cuda")
    for src, dst in ((a, ap), (b, bp)):
        _lib.check(lib.zp_split_planes(src.shape[0], 96, src.data_ptr(), 96, dst.data_ptr(), 96,
                                       src.shape[0] * 96, 1, st), "zp_split_planes")
    c = torch.empty(200, 72, device="cuda")
    _lib.check(lib.zp_gemm_planes(plan.handle, 200, 72, 96, 1, ap.data_ptr(), 96, 200 * 96, 0,
                                  bp.data_ptr(), 96, 72 * 96, 0, None, c.data_ptr(), 72, 0, 1, 0, 0,
                                  None, st), "zp_gemm_planes")
    want = ap.float() @ bp.float().T
    assert (c - want).abs().max().item() < 1e-3 * want.abs().max().item()
    assert plan.device_status() == 0
    assert lib.zp_selftest_bounded_wait(plan.handle, scratch.data_ptr(), 16, 1000, st) == 3   # workspace
