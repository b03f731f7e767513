"""The quantizer entry point that owns its scratch (metis_nvfp4_quantize_static).

It exists for callers that cannot allocate device memory around a call -- a serving process with a
fixed memory plan, a foreign-language binding with raw pointers only -- so the test drives it the
way such a caller would: straight through the C ABI, with output buffers that already exist, twice
in a row on the same device.  The second call follows a first one with much larger values, so the
result would be wrong if anything left in the shared scratch leaked from one call into the next.
The reference for both calls is the ordinary entry point, which must agree byte for byte.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def _static_quantize(x, layout):
    """One call through the C ABI into caller-owned outputs; nothing is allocated inside."""
    L = cabi.lib()
    rows, cols = x.shape
    codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty(L.metis_nvfp4_sf_bytes(rows, cols, layout), dtype=torch.uint8, device=x.device)
    unit = torch.empty(1, dtype=torch.float32, device=x.device)
    dtype = cabi.DTYPE_BF16 if x.dtype == torch.bfloat16 else cabi.DTYPE_F32
    rc = L.metis_nvfp4_quantize_static(x.data_ptr(), dtype, rows, cols, x.stride(0), layout, codes.data_ptr(),
                                       scales.data_ptr(), unit.data_ptr(), torch.cuda.current_stream().cuda_stream)
    cabi.check(rc, "metis_nvfp4_quantize_static")
    return codes, scales, unit


@pytest.mark.gpu
def test_two_calls_in_a_row_match_the_workspace_entry_point():
    g = torch.Generator().manual_seed(0)
    first = (torch.randn(2048, 4096, generator=g) * 1000.0).to(torch.bfloat16).cuda()      # large values, 8 Mi elements
    second = (torch.randn(512, 1536, generator=g) * 0.01).cuda()                            # small values, fp32, smaller
    for x, layout in ((first, cabi.SF_MMA), (second, cabi.SF_ROWMAJOR)):
        codes, scales, unit = _static_quantize(x, layout)
        want = ops.nvfp4_quantize(x, sf_layout=layout)
        torch.cuda.synchronize()
        assert torch.equal(unit, want.unit)
        assert torch.equal(codes, want.codes)
        assert torch.equal(scales, want.scales)
    # and against the CPU oracle itself, not only against the sibling entry point
    codes, scales, unit = _static_quantize(second, cabi.SF_ROWMAJOR)
    ocodes, oscales, ounit, _ = O.quantize(second.cpu().numpy())
    assert np.float32(unit.item()) == ounit
    assert np.array_equal(codes.cpu().numpy(), ocodes) and np.array_equal(scales.cpu().numpy(), oscales.reshape(-1))


@pytest.mark.gpu
def test_a_tensor_of_exactly_the_limit_fills_the_whole_scratch():
    # METIS_STATIC_MAX_ELEMENTS elements: the last block maximum lands in the last word of the array
    rows, cols = cabi.STATIC_MAX_ELEMENTS // 4096, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    x[-1, -16:] = 300.0                                       # the largest block is the very last one
    codes, scales, unit = _static_quantize(x, cabi.SF_ROWMAJOR)
    want = ops.nvfp4_quantize(x, sf_layout=cabi.SF_ROWMAJOR)
    torch.cuda.synchronize()
    assert torch.equal(unit, want.unit) and torch.equal(codes, want.codes) and torch.equal(scales, want.scales)
    tail = x[-8:].float().cpu().numpy()
    ocodes, oscales, ounit, _ = O.quantize(tail)              # these rows hold the largest block: same unit as the whole
    assert np.float32(unit.item()) == ounit
    assert np.array_equal(codes[-8:].cpu().numpy(), ocodes)
    assert np.array_equal(scales.view(rows, cols // 16)[-8:].cpu().numpy(), oscales)


def test_a_tensor_beyond_the_limit_is_rejected_before_anything_runs(built_library):
    L = cabi.lib()
    buf = (C.c_uint8 * 512)()
    p = C.addressof(buf)
    p += (-p) % 256
    rows = cabi.STATIC_MAX_ELEMENTS // 4096 + 1
    rc = L.metis_nvfp4_quantize_static(p, cabi.DTYPE_BF16, rows, 4096, 4096, cabi.SF_MMA, p, p, p, None)
    assert rc == -7
    assert b"METIS_STATIC_MAX_ELEMENTS" in L.metis_last_error_string()
    with pytest.raises(RuntimeError, match="too large"):
        cabi.check(rc, "metis_nvfp4_quantize_static")
