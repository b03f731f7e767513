"""The scale pass replaces RN_fp32(s / unit) by s * RN(1 / unit) wherever the E4M3 byte cannot differ
(fp4_post_b200/csrc/quantize.cu, scale_bytes4).  This restates that rule in numpy and checks it against the
division (quant.py:21-23: scales = (s / unit).to(float8_e4m3fn)) on random pairs and on pairs built to sit on
and next to the E4M3 rounding ties."""
import numpy as np
import torch


def _e4m3_byte(q: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(np.minimum(q, np.float32(448.0)).astype(np.float32))       # the kernel's conversion saturates
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def _device_rule(s: np.ndarray, unit: np.ndarray):
    inv = (np.float32(1.0) / unit).astype(np.float32)
    product = (s * inv).astype(np.float32)
    low = product.view(np.uint32) & np.uint32(0xFFFFF)
    exact_needed = ((low - np.uint32(0x7FFF8)) <= np.uint32(16)) | ~(product >= np.float32(0.0157))
    exact = (s / unit).astype(np.float32)
    return np.where(exact_needed, exact, product), exact, product, exact_needed


def _pairs(rng, kind: int, n: int):
    smax = np.exp(rng.uniform(np.log(1e-8), np.log(1e30), size=n // 1000)).astype(np.float32).repeat(1000)
    unit = (smax / np.float32(448.0)).astype(np.float32)
    if kind == 0:        # block scales spread over six decades below the largest
        s = (smax * np.exp(rng.uniform(np.log(1e-6), 0, size=n)).astype(np.float32)).astype(np.float32)
    elif kind == 1:      # quotients on an E4M3 tie (normal and subnormal range), then up to 6 fp32 steps off it
        e, m = rng.integers(-9, 9, size=n), rng.integers(0, 8, size=n)
        tie = (1 + (m + 0.5) / 8) * np.exp2(e)
        s = (tie * unit.astype(np.float64)).astype(np.float32)
        s = (s.view(np.int32) + rng.integers(-6, 7, size=n).astype(np.int32)).view(np.float32)
    else:                # uniform below the largest
        s = (smax * rng.uniform(0, 1, size=n).astype(np.float32)).astype(np.float32)
    return np.minimum(np.maximum(s, np.float32(1e-9)), smax), unit


def test_product_with_the_reciprocal_gives_the_bytes_of_the_division():
    rng = np.random.default_rng(0)
    total = fast = 0
    for it in range(9):
        s, unit = _pairs(rng, it % 3, 2_000_000)
        chosen, exact, product, exact_needed = _device_rule(s, unit)
        # the premise of the rule: the product lies within a few fp32 steps of the correctly rounded quotient
        steps = np.abs(product.view(np.int32).astype(np.int64) - exact.view(np.int32).astype(np.int64))
        assert steps.max() <= 3
        assert np.array_equal(_e4m3_byte(chosen), _e4m3_byte(exact))
        total += s.size
        fast += int((~exact_needed).sum())
    assert fast > total // 3          # and the rule is not vacuous: the product serves most pairs away from ties
