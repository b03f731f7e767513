"""ctypes binding of the C ABI declared in include/metis_nvfp4.h.

The library is built in-tree (fp4_post_b200/_lib/libmetis_nvfp4.so, see fp4_post_b200.build).
There is no CPU fallback: if the library is missing, `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libmetis_nvfp4.so"

DTYPE_BF16, DTYPE_F32 = 0, 1
SF_ROWMAJOR, SF_MMA = 0, 1
Q_TRANSPOSE, Q_STOCHASTIC, Q_OFFSET_ON_DEVICE, Q_HADAMARD = 1, 2, 4, 8
Q_DEFER_ROWMAJOR, Q_DEFER_TRANSPOSED, Q_SR16 = 16, 32, 64
STATIC_MAX_ELEMENTS = 16 * 1024 * 1024

STATUS_TEXT = {
    0: "ok", -1: "bad argument", -2: "bad shape", -3: "bad alignment", -4: "workspace too small",
    -5: "CUDA error", -6: "unsupported", -7: "too large",
    1: "device timeout waiting for TMA data", 2: "device timeout waiting for the tensor core",
    3: "device timeout waiting for the accumulator hand-off",
}

EXPORTS = (
    "metis_query", "metis_last_error_string", "metis_nvfp4_sf_bytes",
    "metis_nvfp4_quantize_workspace_bytes", "metis_nvfp4_quantize", "metis_rmsnorm_nvfp4_quantize",
    "metis_nvfp4_dequantize", "metis_col_mean_workspace_bytes", "metis_col_mean", "metis_nvfp4_gemv",
    "metis_nvfp4_gemm", "metis_nvfp4_quantize_static", "metis_nvfp4_gemm_workspace_bytes",
    "metis_lowrank_scale",
    "metis_nvfp4_quantize_dual_workspace_bytes", "metis_nvfp4_quantize_dual", "metis_nvfp4_quantize_dual_finish",
    "metis_rmsnorm_mean_workspace_bytes", "metis_rmsnorm_mean",
    "metis_bf16_panel_gemm_workspace_bytes", "metis_bf16_panel_gemm",
    "metis_lowrank_dts_workspace_bytes", "metis_lowrank_dts", "metis_lowrank_du_workspace_bytes", "metis_lowrank_du",
)


class GemmArgs(C.Structure):
    """struct metis_gemm_args"""
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("a_codes", C.c_void_p), ("a_scales", C.c_void_p), ("a_unit", C.c_void_p),
        ("b_codes", C.c_void_p), ("b_scales", C.c_void_p), ("b_unit", C.c_void_p),
        ("alpha", C.c_float), ("rank", C.c_int32),
        ("lr_t", C.c_void_p), ("ldt", C.c_int64),
        ("lr_u", C.c_void_p), ("ldu", C.c_int64),
        ("cvec0", C.c_void_p), ("rvec0", C.c_void_p),
        ("cvec1", C.c_void_p), ("rvec1", C.c_void_p),
        ("c", C.c_void_p), ("ldc", C.c_int64),
        ("d", C.c_void_p), ("ldd", C.c_int64),
        ("d_dtype", C.c_int32), ("reserved", C.c_int32),
        ("status", C.c_void_p), ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("sm_limit", C.c_int32), ("reserved2", C.c_int32),
    ]


_lib = None


class MetisLibraryError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the shared library once and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MetisLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m fp4_post_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    L = C.CDLL(str(LIB_PATH))
    i32, i64, u32, u64, vp, f32 = C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_void_p, C.c_float
    L.metis_query.argtypes = [C.POINTER(i32)] * 3
    L.metis_query.restype = i32
    L.metis_last_error_string.argtypes = []
    L.metis_last_error_string.restype = C.c_char_p
    L.metis_nvfp4_sf_bytes.argtypes = [i64, i64, i32]
    L.metis_nvfp4_sf_bytes.restype = i64
    L.metis_nvfp4_quantize_workspace_bytes.argtypes = [i64, i64]
    L.metis_nvfp4_quantize_workspace_bytes.restype = i64
    L.metis_nvfp4_quantize.argtypes = [vp, i32, i64, i64, i64, vp, u32, u64, u64, i32, vp, vp, vp, vp, i64, vp]
    L.metis_nvfp4_quantize.restype = i32
    L.metis_nvfp4_quantize_dual_workspace_bytes.argtypes = [i64, i64]
    L.metis_nvfp4_quantize_dual_workspace_bytes.restype = i64
    L.metis_nvfp4_quantize_dual.argtypes = [vp, i32, i64, i64, i64, vp, u32, u64, u64, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, vp]
    L.metis_nvfp4_quantize_dual.restype = i32
    L.metis_nvfp4_quantize_dual_finish.argtypes = [i64, i64, u32, i32, vp, vp, vp, vp, vp, vp, vp, i64, vp]
    L.metis_nvfp4_quantize_dual_finish.restype = i32
    L.metis_nvfp4_quantize_static.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp, vp, vp]
    L.metis_nvfp4_quantize_static.restype = i32
    L.metis_rmsnorm_nvfp4_quantize.argtypes = [vp, i32, i64, i64, i64, vp, i32, f32, i32, vp, vp, vp, vp, vp, i64, vp]
    L.metis_rmsnorm_nvfp4_quantize.restype = i32
    L.metis_rmsnorm_mean_workspace_bytes.argtypes = [i64, i64]
    L.metis_rmsnorm_mean_workspace_bytes.restype = i64
    L.metis_rmsnorm_mean.argtypes = [vp, i32, i64, i64, i64, vp, i32, f32, vp, vp, vp, vp, i64, vp]
    L.metis_rmsnorm_mean.restype = i32
    L.metis_nvfp4_dequantize.argtypes = [vp, vp, vp, i32, i64, i64, vp, vp, i32, i64, vp]
    L.metis_nvfp4_dequantize.restype = i32
    L.metis_col_mean_workspace_bytes.argtypes = [i64, i64]
    L.metis_col_mean_workspace_bytes.restype = i64
    L.metis_col_mean.argtypes = [vp, i32, i64, i64, i64, vp, vp, i64, vp]
    L.metis_col_mean.restype = i32
    L.metis_nvfp4_gemv.argtypes = [vp, vp, vp, i32, i64, i64, vp, vp, vp]
    L.metis_nvfp4_gemv.restype = i32
    L.metis_nvfp4_gemm.argtypes = [C.POINTER(GemmArgs)]
    L.metis_nvfp4_gemm.restype = i32
    L.metis_lowrank_scale.argtypes = [vp, i64, i64, i64, vp, i32, vp, vp, vp, vp]
    L.metis_lowrank_scale.restype = i32
    for name in ("metis_bf16_panel_gemm_workspace_bytes", "metis_lowrank_dts_workspace_bytes", "metis_lowrank_du_workspace_bytes"):
        getattr(L, name).argtypes = [i64, i64, i64]
        getattr(L, name).restype = i64
    L.metis_bf16_panel_gemm.argtypes = [vp, i32, i64, vp, i32, i64, i64, i64, i64, vp, i64, vp, i64, vp, vp]
    L.metis_bf16_panel_gemm.restype = i32
    L.metis_lowrank_dts.argtypes = [vp, i64, i64, i64, vp, i64, i64, vp, i64, vp, i32, vp, i64, vp, vp, i64, vp, vp]
    L.metis_lowrank_dts.restype = i32
    L.metis_lowrank_du.argtypes = [vp, i64, i64, i64, vp, i64, i64, vp, i32, i64, vp, i64, vp, vp]
    L.metis_lowrank_du.restype = i32
    L.metis_nvfp4_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    L.metis_nvfp4_gemm_workspace_bytes.restype = i64
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    """Turn a non-zero status into a Python exception, with the library's own message.

    Shape errors become ValueError, as the reference raises for a tensor that blocks of 16 do
    not divide (src/Metis/Metis/quant.py:400-403); everything else is RuntimeError."""
    if rc == 0:
        return
    msg = lib().metis_last_error_string().decode(errors="replace")
    text = f"{what}: {STATUS_TEXT.get(rc, rc)}: {msg}"
    if rc == -2:
        raise ValueError(text)
    raise RuntimeError(text)
