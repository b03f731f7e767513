"""The C-ABI library loads on a machine without a GPU, exports every declared symbol and rejects
bad arguments before it touches the device."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def L(built_library):
    from fp4_post_b200 import cabi
    return cabi.lib()


def declared_symbols():
    text = (ROOT / "include" / "metis_nvfp4.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(metis_\w+)\s*\(", text)))


def test_header_and_binding_list_the_same_entry_points():
    from fp4_post_b200 import cabi
    assert declared_symbols() == sorted(cabi.EXPORTS)


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_is_exported(L, name):
    assert getattr(L, name) is not None


def test_query_reports_abi_and_arch(L):
    abi, sm, n = C.c_int32(), C.c_int32(), C.c_int32(-1)
    assert L.metis_query(C.byref(abi), C.byref(sm), C.byref(n)) == 0
    assert abi.value == 2 and sm.value == 100 and n.value >= 0      # version 2: per-call sm_limit in metis_gemm_args


def test_size_helpers(L):
    # row-major: one byte per 16 elements
    assert L.metis_nvfp4_sf_bytes(100, 64, 0) == 100 * 4
    # tiled: rows padded to 128, scale columns padded to 16 (256 elements), 512 bytes per 128x4 tile
    assert L.metis_nvfp4_sf_bytes(100, 64, 1) == 1 * 4 * 512
    assert L.metis_nvfp4_sf_bytes(129, 272, 1) == 2 * 8 * 512
    assert L.metis_nvfp4_quantize_workspace_bytes(8, 64) == 256 + 8 * 4 * 4
    assert L.metis_col_mean_workspace_bytes(1000, 64) == 8 * 64 * 4


def test_gemm_rejects_a_negative_sm_limit(L):
    from fp4_post_b200 import cabi
    buf = (C.c_uint8 * 1024)()
    p = C.addressof(buf)
    p += (-p) % 256
    a = cabi.GemmArgs()
    a.M, a.N, a.K = 256, 256, 256
    for f in ("a_codes", "a_scales", "a_unit", "b_codes", "b_scales", "b_unit", "d"):
        setattr(a, f, p)
    a.ldd, a.d_dtype, a.alpha, a.sm_limit = 256, cabi.DTYPE_BF16, 1.0, -3
    assert L.metis_nvfp4_gemm(C.byref(a)) == -1 and b"sm_limit" in L.metis_last_error_string()


def test_quantize_rejects_bad_arguments_without_a_device(L):
    from fp4_post_b200 import cabi
    buf = (C.c_uint8 * 4096)()
    p = C.addressof(buf)
    p += (-p) % 256
    # 24 columns: blocks of 16 do not divide it (quant.py:400-403 raises ValueError there)
    rc = L.metis_nvfp4_quantize(p, 1, 4, 24, 24, None, 0, 0, 0, 0, p, p, p, p, 4096, None)
    assert rc == -2
    with pytest.raises(ValueError):
        cabi.check(rc, "quantize")
    assert b"16" in L.metis_last_error_string()
    assert L.metis_nvfp4_quantize(None, 1, 4, 32, 32, None, 0, 0, 0, 0, p, p, p, p, 4096, None) == -1
    assert L.metis_nvfp4_quantize(p, 7, 4, 32, 32, None, 0, 0, 0, 0, p, p, p, p, 4096, None) == -1
    assert L.metis_nvfp4_quantize(p, 1, 4, 32, 32, None, 16, 0, 0, 0, p, p, p, p, 4096, None) == -1   # unknown flag
    assert L.metis_nvfp4_quantize(p, 1, 16, 32, 32, None, 8, 0, 0, 0, p, p, p, p, 4096, None) == -6   # the Hadamard rotation belongs to the transposed output
    assert L.metis_nvfp4_quantize(p, 1, 16, 32, 32, None, 1 | (5 << 16), 0, 0, 0, p, p, p, p, 4096, None) == -1   # sign bits without the rotation
    assert L.metis_nvfp4_quantize(p, 1, 4, 32, 32, None, 0, 0, 0, 0, p, p, p, p, 16, None) == -4     # workspace
    assert L.metis_nvfp4_quantize(p + 4, 1, 4, 32, 32, None, 0, 0, 0, 0, p, p, p, p, 4096, None) == -3
    assert L.metis_nvfp4_quantize(p, 1, 0, 32, 32, None, 0, 0, 0, 0, p, p, p, p, 4096, None) == -2   # empty


def test_dual_quantizer_rejects_bad_arguments_without_a_device(L):
    from fp4_post_b200 import cabi
    buf = (C.c_uint8 * 65536)()
    p = C.addressof(buf)
    p += (-p) % 256
    ws = L.metis_nvfp4_quantize_dual_workspace_bytes(64, 64)
    dual = lambda flags, rows=64, sums=None: L.metis_nvfp4_quantize_dual(p, 0, rows, 64, 64, None, flags, 0, 0, 0, p, p, p, p, p, p, sums, p, ws, None)
    assert dual(cabi.Q_DEFER_ROWMAJOR | cabi.Q_DEFER_TRANSPOSED) == -1           # only one of the two scale passes can be deferred
    assert dual(64) == -1                                                      # unknown flag
    assert dual(cabi.Q_HADAMARD, sums=p) == -1                                 # rotated blocks need weighted sums
    assert dual(0, rows=48, sums=p) == -2                                      # token sums need rows % 64 == 0
    finish = lambda which, rows=64, workspace=p: L.metis_nvfp4_quantize_dual_finish(rows, 64, which, 0, p, p, p, p, p, None, workspace, ws, None)
    assert finish(0) == -1 and finish(cabi.Q_DEFER_ROWMAJOR | cabi.Q_DEFER_TRANSPOSED) == -1
    assert finish(cabi.Q_DEFER_TRANSPOSED, rows=40) == -2
    assert finish(cabi.Q_DEFER_ROWMAJOR, workspace=None) == -4


def test_gemm_rejects_bad_arguments_without_a_device(L):
    from fp4_post_b200 import cabi
    buf = (C.c_uint8 * 1024)()
    p = C.addressof(buf)
    p += (-p) % 256
    a = cabi.GemmArgs()
    a.M, a.N, a.K = 128, 128, 48           # K must be a multiple of 32
    for f in ("a_codes", "a_scales", "a_unit", "b_codes", "b_scales", "b_unit", "d"):
        setattr(a, f, p)
    a.ldd, a.d_dtype, a.alpha = 128, 0, 1.0
    assert L.metis_nvfp4_gemm(C.byref(a)) == -2
    a.K = 64
    a.rank = 12                            # rank must be a multiple of 8
    assert L.metis_nvfp4_gemm(C.byref(a)) == -2
    a.rank = 0
    a.d = None
    assert L.metis_nvfp4_gemm(C.byref(a)) == -1
    assert L.metis_nvfp4_gemm(None) == -1


def test_ops_refuse_cpu_tensors(built_library):
    import torch
    from fp4_post_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.nvfp4_quantize(torch.zeros(4, 32))


def test_gemm_rejects_reserved_bits_other_than_the_two_test_hooks(L):
    # the timing knobs of development builds (issue no MMAs, request no data) do not exist in the shipped library
    from fp4_post_b200 import cabi
    buf = (C.c_uint8 * 1024)()
    p = C.addressof(buf)
    p += (-p) % 256
    for bits in (2, 4, 6, 16, 2 | 8):
        a = cabi.GemmArgs()
        a.M, a.N, a.K = 256, 256, 256
        for f in ("a_codes", "a_scales", "a_unit", "b_codes", "b_scales", "b_unit", "d"):
            setattr(a, f, p)
        a.ldd, a.d_dtype, a.alpha, a.reserved = 256, cabi.DTYPE_BF16, 1.0, bits
        rc = L.metis_nvfp4_gemm(C.byref(a))
        assert rc == -1 and b"reserved" in L.metis_last_error_string(), bits
