"""ctypes binding of ``libzippel_b200.so`` (the C ABI declared in ``include/zippel_b200.h``).

The library is the only compute path of this package: if it is missing, or the current GPU
is not one it holds code for, every call raises -- there is no fallback.
"""

from __future__ import annotations

import ctypes as C
import pathlib

_LIB_PATH = pathlib.Path(__file__).resolve().parent / "libzippel_b200.so"
_lib = None


class ZpError(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.zp_status_string(status).decode()
        if status == 4:
            msg += ": " + lib.zp_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (status {status})")
        self.status = status


class ZpConfig(C.Structure):
    _fields_ = [("lmax", C.c_int32), ("mmax", C.c_int32), ("sphere_channels", C.c_int32),
                ("hidden_channels", C.c_int32), ("precision", C.c_int32)]


class ZpSizes(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("K", "Km", "nnz", "nnz_pad", "R", "n_gate", "w1_cols")]


class ZpFrontConfig(C.Structure):
    _fields_ = [("lmax", C.c_int32), ("num_basis", C.c_int32), ("edge_channels", C.c_int32),
                ("n_elements", C.c_int32), ("envelope_exponent", C.c_int32),
                ("cutoff", C.c_float), ("gauss_coeff", C.c_float)]


class ZpWeights(C.Structure):
    _fields_ = [("c1_w0", C.c_void_p), ("c1_b0", C.c_void_p), ("c1_wm", C.POINTER(C.c_void_p)),
                ("c2_w0", C.c_void_p), ("c2_b0", C.c_void_p), ("c2_wm", C.POINTER(C.c_void_p))]


# name -> (restype, argtypes); must list every symbol of include/zippel_b200.h
_P, _I64, _SZ = C.c_void_p, C.c_int64, C.c_size_t
SIGNATURES = {
    "zp_status_string": (C.c_char_p, [C.c_int]),
    "zp_last_cuda_error": (C.c_char_p, []),
    "zp_device_supported": (C.c_int, []),
    "zp_plan_create": (C.c_int, [C.POINTER(ZpConfig), C.POINTER(C.c_double), C.POINTER(_P)]),
    "zp_plan_destroy": (C.c_int, [_P]),
    "zp_plan_sizes": (C.c_int, [_P, C.POINTER(ZpSizes)]),
    "zp_plan_tables": (C.c_int, [_P] + [C.POINTER(C.c_int32)] * 4),
    "zp_csr_work_bytes": (_SZ, [_I64, _I64]),
    "zp_csr_build": (C.c_int, [_P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "zp_csr_build_static": (C.c_int, [_P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "zp_csr_status": (C.c_int, [_P, _P, C.POINTER(C.c_int)]),
    "zp_csr_static_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "zp_wigner_forward": (C.c_int, [_P, _I64, _P, _P, _P, _P, _P]),
    "zp_wigner_backward": (C.c_int, [_P, _I64, _P, _P, _P, _P, _P, _P]),
    "zp_workspace_bytes": (_SZ, [_P, _I64, _I64, C.c_int]),
    "zp_eso2_forward": (C.c_int, [_P, _I64, _I64] + [_P] * 9 + [C.POINTER(ZpWeights), _P, _P,
                                                                _SZ, _P]),
    "zp_eso2_forward_inference": (C.c_int, [_P, _I64, _I64] + [_P] * 9 + [C.POINTER(ZpWeights), _P,
                                                                          _P, _SZ, _P]),
    "zp_eso2_backward": (C.c_int, [_P, _I64, _I64] + [_P] * 12 + [C.POINTER(ZpWeights)]
                         + [_P] * 4 + [C.POINTER(ZpWeights), _P, _SZ, _P]),
    "zp_workspace_bytes_radial": (_SZ, [_P, _I64, _I64, C.c_int, C.c_int]),
    "zp_eso2_forward_radial": (C.c_int, [_P, _I64, _I64] + [_P] * 7 + [C.c_int] + [_P] * 4
                               + [C.POINTER(ZpWeights), _P, _P, _SZ, C.c_int, _P]),
    "zp_eso2_backward_radial": (C.c_int, [_P, _I64, _I64] + [_P] * 8 + [C.c_int] + [_P] * 6
                                + [C.POINTER(ZpWeights)] + [_P] * 6
                                + [C.POINTER(ZpWeights), _P, _SZ, _P]),
    "zp_split_planes": (C.c_int, [_I64, _I64, _P, _I64, _P, _I64, _I64, C.c_int, _P]),
    "zp_gemm_planes": (C.c_int, [_P, _I64, _I64, _I64, C.c_int, _P, _I64, _I64, C.c_int, _P, _I64,
                                 _I64, C.c_int, _P, _P, _I64, C.c_int, C.c_int, _I64, C.c_int,
                                 C.POINTER(C.c_int), _P]),
    "zp_linear_work_bytes": (_SZ, [_P, _I64, _I64, _I64]),
    "zp_linear_forward": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _SZ, _P]),
    "zp_linear_backward": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "zp_linear_backward_saved": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _SZ, _P]),
    "zp_layernorm_work_bytes": (_SZ, [C.c_int]),
    "zp_layernorm_silu_forward": (C.c_int, [_I64, C.c_int, _P, _P, _P, C.c_float, _P, _P, _P, _P]),
    "zp_layernorm_silu_backward": (C.c_int, [_I64, C.c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                              _SZ, _P]),
    "zp_readout_work_bytes": (_SZ, [_P, _I64]),
    "zp_readout_forward": (C.c_int, [_P, _I64] + [_P] * 7 + [_SZ, _P]),
    "zp_readout_backward": (C.c_int, [_P, _I64] + [_P] * 12 + [_SZ, _P]),
    "zp_edge_features_work_bytes": (_SZ, [C.POINTER(ZpFrontConfig), _I64, _I64]),
    "zp_edge_features_forward": (C.c_int, [C.POINTER(ZpFrontConfig), _I64, _I64] + [_P] * 16 + [_P]),
    "zp_edge_features_backward": (C.c_int, [C.POINTER(ZpFrontConfig), _I64, _I64] + [_P] * 14
                                  + [_SZ, _P]),
    "zp_neighbors_work_bytes": (_SZ, [_I64, C.c_double, C.c_double]),
    "zp_neighbors_count": (C.c_int, [_P, _I64, C.c_double, C.c_double, C.c_int, _P, _P, _P, _SZ, _P]),
    "zp_neighbors_fill": (C.c_int, [_P, _I64, C.c_double, C.c_double, C.c_int, _P, _I64, _P, _P, _P,
                                    _P, _SZ, _P]),
    "zp_plan_device_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "zp_selftest_bounded_wait": (C.c_int, [_P, _P, _SZ, _I64, _P]),
    "zp_kernel_class_name": (C.c_char_p, [C.c_int]),
    "zp_timing_enable": (C.c_int, [_P, C.c_int]),
    "zp_timing_read": (C.c_int, [_P, C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
}
N_KERNEL_CLASSES = 14


def lib_path() -> pathlib.Path:
    return _LIB_PATH


def load():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m zippel_b200.build` "
                "(there is no non-CUDA path)")
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise ZpError(status, where)
