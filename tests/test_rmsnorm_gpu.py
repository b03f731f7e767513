"""Fused RMSNorm -> NVFP4 kernel.  Gate (a): the normalised output is within one ulp of the CPU
reference (reduction order and rsqrt may differ in the last bit).  Gate (b): codes, E4M3 bytes
and unit are bit-exact against the oracle quantizer applied to the kernel's own normalised
output.  The raw end-to-end code mismatch against the reference chain is reported."""
import numpy as np
import pytest
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O
from gpu_helpers import assert_packed_equal, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def reference_norm(x, gamma, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * gamma   # llama.py:23-31


def check(x, gamma, eps, layout):
    q, y = ops.rmsnorm_nvfp4_quantize(x.to(DEV), gamma.to(DEV), eps, sf_layout=layout, return_norm=True)
    want = reference_norm(x, gamma, eps)
    assert y.dtype == want.dtype
    yk = y.float().cpu()
    # (a) at most one ulp of the output dtype away
    if want.dtype == torch.bfloat16:
        ulp = torch.maximum(want.float().abs(), torch.tensor(1e-30)) * 2.0 ** -7
    else:
        ulp = torch.maximum(want.float().abs(), torch.tensor(1e-30)) * 2.0 ** -7   # the bf16 rounding of the normalised value dominates
    assert bool(((yk - want.float()).abs() <= ulp).all())
    frac_equal = float((yk == want.float()).float().mean())
    assert frac_equal > 0.995, frac_equal
    # (b) bit-exact quantization of the kernel's own normalised output
    assert_packed_equal(q, yk.numpy(), layout, what="rmsnorm->quant")
    # report: raw code mismatch against the CPU chain
    ocodes, _, _, _ = O.quantize(want.float().numpy())
    mism = float((q.codes.cpu().numpy() != ocodes).mean())
    return frac_equal, mism


def test_golden(rmsnorm_golden):
    for name, g in rmsnorm_golden:
        x = torch.from_numpy(g["x"]).to(torch.bfloat16)
        gamma = torch.from_numpy(g["gamma"])
        gamma = gamma.to(torch.bfloat16) if "gbf16" in name else gamma
        frac_equal, mism = check(x, gamma, 1e-6, cabi.SF_ROWMAJOR)
        print(f"{name}: normalised values identical {frac_equal:.5f}, code bytes differing from the CPU chain {mism:.2e}")
        assert mism < 2e-3


@pytest.mark.parametrize("rows,cols", [(5, 16), (64, 1536), (128, 3584), (256, 4096), (32, 8960), (8, 18944)])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_bf16_rows(rows, cols, gdtype):
    x = synthetic(rows, cols, "student", seed=cols, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(cols + 1)
    gamma = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(gdtype)
    frac_equal, mism = check(x, gamma, 1e-6, cabi.SF_MMA)
    assert mism < 2e-3


# Decode-sized inputs (a handful of rows of up to 8192 elements) take the one-launch cluster kernel:
# one row, rows that fill one pass / all four passes of the 8 CTAs, two blocks per thread, a hidden
# size that is not a power of two, and the first row count past the limit (the streaming kernels).
@pytest.mark.parametrize("rows,cols", [(1, 4096), (8, 4096), (16, 4096), (32, 4096), (33, 4096), (16, 3584),
                                       (9, 8192), (3, 1536), (2, 64)])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_one_launch_path_for_decode_sizes(rows, cols, gdtype, layout):
    x = synthetic(rows, cols, "student", seed=rows * 31 + cols, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(cols + rows)
    gamma = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(gdtype)
    torch.empty(1 << 22, device=DEV, dtype=torch.uint8).fill_(0xA5)       # stale bytes where the outputs will land
    frac_equal, mism = check(x, gamma, 1e-6, layout)
    assert mism < 4e-3
    q1 = ops.rmsnorm_nvfp4_quantize(x.to(DEV), gamma.to(DEV), 1e-6, sf_layout=layout)
    q2, _ = ops.rmsnorm_nvfp4_quantize(x.to(DEV), gamma.to(DEV), 1e-6, sf_layout=layout, return_norm=True)
    assert torch.equal(q1.codes, q2.codes) and torch.equal(q1.scales, q2.scales) and torch.equal(q1.unit, q2.unit)


def test_fp32_rows_and_strided_input():
    x = synthetic(40, 1024, "normal", seed=2, dtype=torch.float32)
    gamma = torch.ones(1024)
    q, y = ops.rmsnorm_nvfp4_quantize(x.to(DEV), gamma.to(DEV), 1e-5, sf_layout=cabi.SF_ROWMAJOR, return_norm=True)
    want = reference_norm(x, gamma, 1e-5)
    assert torch.allclose(y.cpu(), want, rtol=3e-7, atol=1e-30)
    assert_packed_equal(q, y.cpu().numpy(), cabi.SF_ROWMAJOR, what="fp32")
    wide = synthetic(16, 2048, "normal", seed=4, dtype=torch.bfloat16).to(DEV)
    view = wide[:, 512:1536]
    q2, y2 = ops.rmsnorm_nvfp4_quantize(view, gamma.to(DEV).to(torch.bfloat16), 1e-6, sf_layout=cabi.SF_ROWMAJOR, return_norm=True)
    assert_packed_equal(q2, y2.float().cpu().numpy(), cabi.SF_ROWMAJOR, what="strided")


def test_without_the_normalised_output_the_codes_are_the_same():
    x = synthetic(64, 1536, "student", seed=8, dtype=torch.bfloat16).to(DEV)
    gamma = torch.ones(1536, dtype=torch.bfloat16, device=DEV)
    q1 = ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6)
    q2, _ = ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6, return_norm=True)
    assert torch.equal(q1.codes, q2.codes) and torch.equal(q1.scales, q2.scales) and torch.equal(q1.unit, q2.unit)


# ---- the mean-centred / trainable path: normalise + column mean in one pass, then the quantizer -------------------

@pytest.mark.parametrize("rows,cols", [(48, 1536), (256, 3584), (1024, 4096), (40, 8960), (2048, 256)])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_norm_with_column_mean(rows, cols, gdtype):
    x = synthetic(rows, cols, "student", seed=cols + rows, dtype=torch.bfloat16).to(DEV)
    g = torch.Generator().manual_seed(cols + 1)
    gamma = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(gdtype).to(DEV)
    y, mean, rstd = ops.rmsnorm_mean(x, gamma, 1e-6)
    # the same normalised values as the fused quantizer writes, bit for bit (one arithmetic, two kernels)
    _, y_fused = ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6, return_norm=True)
    assert y.dtype == y_fused.dtype and torch.equal(y, y_fused)
    # against the CPU chain: a reciprocal RMS that differs in its last bit moves the normalised value by one
    # bf16 ulp, and the product with gamma by up to two
    want = reference_norm(x.cpu(), gamma.cpu(), 1e-6).float()
    assert bool(((y.float().cpu() - want).abs() <= want.abs().clamp(min=1e-30) * 2.0 ** -6).all())
    assert float((y.float().cpu() == want).float().mean()) > 0.995
    # mean of the kernel's own output, fp32 sums in a fixed order
    assert torch.allclose(mean, y.float().mean(dim=0), rtol=1e-5, atol=1e-6)
    m2 = ops.rmsnorm_mean(x, gamma, 1e-6)[1]
    assert torch.equal(mean, m2)                                   # deterministic
    want_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    assert torch.allclose(rstd, want_rstd, rtol=1e-6, atol=0)
    # second pass: the quantizer on y with that mean, against the oracle
    q = ops.nvfp4_quantize(y, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(q, y.float().cpu().numpy(), cabi.SF_ROWMAJOR, mean=mean.cpu().numpy(), what="norm + mean -> quant")
