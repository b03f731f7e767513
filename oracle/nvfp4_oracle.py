"""numpy front end of the C oracle (oracle/nvfp4_oracle.c) plus a few pure-numpy helpers.

TEST INFRASTRUCTURE ONLY.  The arithmetic follows the reference's quantizer,
src/Metis/Metis/quant.py:6-36 (round to nearest) and the mean-centred wrapper
src/Metis/Metis/bitlinear.py:311-336; parity is pinned by tests/golden (vectors made by
importing the reference itself, see tests/golden/make_golden.py).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libnvfp4_oracle.so"
_lib = None

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def build(force: bool = False) -> Path:
    """Compile the C oracle with gcc (oracle/Makefile)."""
    src = _HERE / "nvfp4_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        c = ctypes
        _lib.oracle_nvfp4_quantize.argtypes = [c.c_void_p, c.c_int64, c.c_int64, c.c_void_p, c.c_void_p,
                                               c.c_void_p, c.c_void_p, c.c_void_p, c.c_int]
        _lib.oracle_nvfp4_quantize.restype = c.c_int
        _lib.oracle_nvfp4_dequantize.argtypes = [c.c_void_p, c.c_void_p, c.c_float, c.c_int64, c.c_int64,
                                                 c.c_void_p, c.c_void_p]
        _lib.oracle_nvfp4_dequantize.restype = c.c_int
        _lib.oracle_scales_to_mma_layout.argtypes = [c.c_void_p, c.c_int64, c.c_int64, c.c_void_p]
        _lib.oracle_scales_to_mma_layout.restype = None
        _lib.oracle_compare_conversion_rounding.argtypes = [c.c_uint32, c.c_uint32, c.c_void_p, c.c_void_p, c.c_void_p]
        _lib.oracle_compare_conversion_rounding.restype = None
        _lib.oracle_f32_to_e4m3fn.argtypes = [c.c_float]
        _lib.oracle_f32_to_e4m3fn.restype = c.c_uint8
        _lib.oracle_e4m3fn_to_f32.argtypes = [c.c_uint8]
        _lib.oracle_e4m3fn_to_f32.restype = c.c_float
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def quantize(x: np.ndarray, col_mean: np.ndarray | None = None, threads: int = 1):
    """x: float32 [rows, cols] -> (codes u8 [rows, cols/2], scales u8 [rows, cols/16], unit f32,
    block_scale f32 [rows, cols/16]).  Raises ValueError if 16 does not divide cols."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.ndim == 2
    rows, cols = x.shape
    if cols % 16 != 0 or rows == 0:
        raise ValueError(f"NVFP4 block shape (1, 16) does not divide tensor shape {x.shape}")
    if col_mean is not None:
        col_mean = np.ascontiguousarray(col_mean, dtype=np.float32).reshape(cols)
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    bscale = np.empty((rows, cols // 16), np.float32)
    unit = np.zeros(1, np.float32)
    rc = lib().oracle_nvfp4_quantize(_ptr(x), rows, cols, _ptr(col_mean), _ptr(codes), _ptr(scales),
                                     _ptr(unit), _ptr(bscale), int(threads))
    if rc != 0:
        raise ValueError("oracle_nvfp4_quantize rejected the shape")
    return codes, scales, np.float32(unit[0]), bscale


def dequantize(codes: np.ndarray, scales: np.ndarray, unit, col_mean: np.ndarray | None = None) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, half = codes.shape
    cols = half * 2
    if col_mean is not None:
        col_mean = np.ascontiguousarray(col_mean, dtype=np.float32).reshape(cols)
    out = np.empty((rows, cols), np.float32)
    rc = lib().oracle_nvfp4_dequantize(_ptr(codes), _ptr(scales), ctypes.c_float(float(unit)), rows, cols,
                                       _ptr(col_mean), _ptr(out))
    assert rc == 0
    return out


def quantize_dequantize(x: np.ndarray, col_mean: np.ndarray | None = None) -> np.ndarray:
    """The reference's fake-quant output (quant.py:6-36), optionally mean-centred."""
    codes, scales, unit, _ = quantize(x, col_mean)
    return dequantize(codes, scales, unit, col_mean)


def scales_to_mma_layout(scales: np.ndarray, cols: int) -> np.ndarray:
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows = scales.shape[0]
    tiles = ((cols + 255) // 256) * 4
    out = np.empty(((rows + 127) // 128) * tiles * 512, np.uint8)
    lib().oracle_scales_to_mma_layout(_ptr(scales), rows, cols, _ptr(out))
    return out


def unpack_codes(codes: np.ndarray) -> np.ndarray:
    """u8 [rows, cols/2] -> signed e2m1 values float32 [rows, cols]."""
    lo = codes & 0x0F
    hi = codes >> 4
    nib = np.stack([lo, hi], axis=-1).reshape(codes.shape[0], -1)
    val = E2M1_VALUES[nib & 7]
    return np.where(nib & 8, -val, val).astype(np.float32)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    exp = ((b >> 3) & 15).astype(np.int32)
    mant = (b & 7).astype(np.float32)
    v = np.where(exp == 0, mant * np.float32(2.0 ** -9), np.ldexp(1.0 + mant / 8.0, exp - 7)).astype(np.float32)
    v = np.where((exp == 15) & ((b & 7) == 7), np.float32(np.nan), v)
    return np.where(b & 0x80, -v, v).astype(np.float32)


def gemm_reference(a_deq: np.ndarray, b_deq: np.ndarray, t=None, u=None, rvec=None, bias=None) -> np.ndarray:
    """FP32 dequantize-then-matmul oracle: a_deq [M,K] @ b_deq[N,K]^T (+ t @ u^T + rank-1 terms).
    Accumulates in float64 and rounds once, so it is the tightest fp32 statement of the product."""
    out = a_deq.astype(np.float64) @ b_deq.astype(np.float64).T
    if t is not None:
        out += t.astype(np.float64) @ u.astype(np.float64).T
    if rvec is not None:
        out += rvec.astype(np.float64)[None, :]
    if bias is not None:
        out += bias.astype(np.float64)[None, :]
    return out.astype(np.float32)


def compare_conversion_rounding(lo: float, hi: float):
    """For every fp32 v in [lo, hi] (both positive): how often the reference's twice-rounded code differs from a
    round-to-nearest-even conversion of v onto the e2m1 grid, without and with the kernels' (v + t) - t step.
    Returns (count without, count with, the first few v where the plain conversion differs)."""
    lo_bits = int(np.float32(lo).view(np.uint32))
    hi_bits = int(np.float32(hi).view(np.uint32))
    plain, fixed = ctypes.c_uint64(0), ctypes.c_uint64(0)
    first = np.zeros(8, np.uint32)
    lib().oracle_compare_conversion_rounding(lo_bits, hi_bits, ctypes.byref(plain), ctypes.byref(fixed), _ptr(first))
    return plain.value, fixed.value, first[: min(plain.value, 8)].view(np.float32)
