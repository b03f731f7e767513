"""Shared helpers of the GPU parity tests: run a kernel through the C ABI, fetch the packed
result, and state the oracle's answer for the same input."""
import numpy as np
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O


def packed_to_numpy(q):
    return q.codes.cpu().numpy(), q.scales.cpu().numpy(), np.float32(q.unit.item())


def oracle_packed(x_f32: np.ndarray, sf_layout: int, mean=None):
    codes, scales, unit, _ = O.quantize(x_f32, col_mean=mean)
    if sf_layout == cabi.SF_MMA:
        scales = O.scales_to_mma_layout(scales, x_f32.shape[1])
    else:
        scales = scales.reshape(-1)
    return codes, scales, unit


def assert_packed_equal(q, x_f32, sf_layout, mean=None, what=""):
    codes, scales, unit = packed_to_numpy(q)
    ocodes, oscales, ounit = oracle_packed(x_f32, sf_layout, mean)
    assert unit == ounit, f"{what}: unit {unit} vs oracle {ounit}"
    bad = int((codes != ocodes).sum())
    assert bad == 0, f"{what}: {bad}/{codes.size} code bytes differ"
    bad = int((scales != oscales).sum())
    assert bad == 0, f"{what}: {bad}/{scales.size} scale bytes differ"


def synthetic(rows, cols, kind, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    if kind == "normal":
        x = torch.randn(rows, cols, generator=g)
    elif kind == "outliers":          # 1 % of the channels scaled by 20
        x = torch.randn(rows, cols, generator=g)
        x[:, torch.randperm(cols, generator=g)[: max(1, cols // 100)]] *= 20
    elif kind == "student":           # heavy tails plus a per-channel offset
        z = torch.randn(rows, cols, generator=g)
        chi = torch.randn(3, rows, cols, generator=g).pow(2).sum(0)
        x = z / (chi / 3).sqrt() + 2.0 * torch.randn(1, cols, generator=g)
    elif kind == "weights":
        x = torch.randn(rows, cols, generator=g) / cols ** 0.5
    else:
        raise ValueError(kind)
    return x.to(dtype)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
