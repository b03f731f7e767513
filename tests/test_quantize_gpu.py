"""NVFP4 quantizer kernels against the CPU oracle: packed codes, E4M3 bytes and unit bit-exact
for round to nearest; stochastic rounding checked in distribution."""
import numpy as np
import pytest
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O
from gpu_helpers import assert_packed_equal, packed_to_numpy, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


@pytest.mark.parametrize("name", ["randn_64x256", "outliers_32x512", "bf16valued_48x1536", "weights_128x256", "special_8x64"])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_golden_vectors(quant_golden, name, layout):
    g = quant_golden[name]
    x = torch.from_numpy(g["x"]).to(DEV)
    q = ops.nvfp4_quantize(x, sf_layout=layout)
    codes, scales, unit = packed_to_numpy(q)
    assert unit == g["unit"]
    assert np.array_equal(codes, g["codes"])
    want = g["scales"].reshape(-1) if layout == cabi.SF_ROWMAJOR else O.scales_to_mma_layout(g["scales"], x.shape[1])
    assert np.array_equal(scales, want)
    # and the dequantized tensor is the reference's fake-quant output, bit for bit
    assert np.array_equal(q.dequantize(torch.float32).cpu().numpy(), g["qdq"])
    if name == "bf16valued_48x1536":      # the same values arriving as bf16
        qb = ops.nvfp4_quantize(x.to(torch.bfloat16), sf_layout=layout)
        assert np.array_equal(qb.codes.cpu().numpy(), g["codes"])
        assert np.array_equal(qb.scales.cpu().numpy(), want)


def test_golden_mean_centred(quant_golden):
    g = quant_golden["mean_96x256"]
    x = torch.from_numpy(g["x"]).to(DEV)
    mean = torch.from_numpy(g["mean"]).to(DEV)
    q = ops.nvfp4_quantize(x, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    codes, scales, unit = packed_to_numpy(q)
    assert unit == g["unit"] and np.array_equal(codes, g["codes"]) and np.array_equal(scales, g["scales"].reshape(-1))
    assert np.array_equal(q.dequantize(torch.float32).cpu().numpy(), g["qdq"])   # mean added back
    # the kernel's own column mean is the torch mean up to summation order
    got = ops.col_mean(x).cpu().numpy()
    assert np.allclose(got, g["mean"], rtol=2e-6, atol=1e-6)


SHAPES = [(1, 16, "normal"), (3, 48, "normal"), (33, 1536, "student"), (257, 272, "outliers"),
          (2048, 2048, "outliers"), (1024, 3584, "student"), (96, 8960, "normal")]


@pytest.mark.parametrize("rows,cols,kind", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_rows_match_oracle(rows, cols, kind, dtype, layout):
    x = synthetic(rows, cols, kind, seed=rows * 7 + cols, dtype=dtype)
    q = ops.nvfp4_quantize(x.to(DEV), sf_layout=layout)
    assert_packed_equal(q, x.float().numpy(), layout, what=f"{rows}x{cols} {dtype}")


@pytest.mark.parametrize("rows,cols,kind", [(16, 8, "normal"), (48, 24, "normal"), (512, 64, "outliers"),
                                            (1040, 200, "student"), (2048, 2048, "outliers"), (4096, 1536, "student")])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_transposed_matches_oracle_on_the_transpose(rows, cols, kind, dtype):
    x = synthetic(rows, cols, kind, seed=rows + cols, dtype=dtype)
    q = ops.nvfp4_quantize(x.to(DEV), transpose=True, sf_layout=cabi.SF_MMA)
    assert q.shape == (cols, rows)
    assert_packed_equal(q, np.ascontiguousarray(x.float().numpy().T), cabi.SF_MMA, what="transposed")


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_mean_subtraction_matches_oracle(transpose, dtype):
    x = synthetic(640, 384, "student", seed=5, dtype=dtype)
    mean = x.float().mean(0)
    q = ops.nvfp4_quantize(x.to(DEV), transpose=transpose, mean=mean.to(DEV), sf_layout=cabi.SF_ROWMAJOR)
    centred = x.float().numpy() - mean.numpy()[None, :]      # fp32 subtraction, as the kernel does
    if transpose:
        assert_packed_equal(q, np.ascontiguousarray(centred.T), cabi.SF_ROWMAJOR, what="transposed mean")
    else:
        assert_packed_equal(q, x.float().numpy(), cabi.SF_ROWMAJOR, mean=mean.numpy(), what="row mean")


# Decode-sized tensors (at most 16384 blocks, round to nearest) take the one-launch cluster kernel;
# these shapes sit on its limits: one block, one CTA, the largest tensor it takes, the widest decode
# rows, row counts and widths that leave padding in the tiled layout (two row blocks; 17 scale columns:
# a partly filled word), and the first shape past the limit (the streaming path).
@pytest.mark.parametrize("rows,cols", [(1, 16), (1, 4096), (16, 4096), (64, 4096), (16, 8192), (16, 14336), (129, 1536),
                                       (100, 272), (7, 1536), (65, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_one_launch_path_for_small_tensors(rows, cols, dtype, layout):
    x = synthetic(rows, cols, "outliers", seed=rows + 3 * cols, dtype=dtype)
    torch.empty(1 << 22, device=DEV, dtype=torch.uint8).fill_(0xA5)       # stale bytes where the outputs will land
    q = ops.nvfp4_quantize(x.to(DEV), sf_layout=layout)
    assert_packed_equal(q, x.float().numpy(), layout, what=f"small {rows}x{cols}")
    if rows >= 7 and layout == cabi.SF_ROWMAJOR:
        mean = x.float().mean(0)
        wide = torch.zeros(rows, cols + 64, dtype=dtype)
        wide[:, :cols] = x
        view = wide.to(DEV)[:, :cols]                                     # leading dimension cols + 64
        q = ops.nvfp4_quantize(view, mean=mean.to(DEV), sf_layout=layout)
        assert_packed_equal(q, x.float().numpy(), layout, mean=mean.numpy(), what=f"small centred {rows}x{cols}")


def test_bf16_inputs_sitting_exactly_on_rounding_ties():
    # With bf16 data an element is often an exact fraction of the block maximum that lands on a
    # rounding boundary of the reference (x = amax/8 gives |x|/(s/2) = 1.5 up to the rounding of
    # amax/6); the answer then hangs on the reference's exact division.  Every block here holds its
    # maximum plus the boundary ratios and their bf16 neighbours.
    g = torch.Generator().manual_seed(7)
    amax = (torch.rand(20480, 1, generator=g) * 8 + 0.01).to(torch.bfloat16).float() * (2.0 ** torch.randint(-6, 6, (20480, 1), generator=g))
    ratios = torch.tensor([1 / 24, 1 / 8, 5 / 24, 7 / 24, 5 / 12, 7 / 12, 5 / 6])
    near = (amax * ratios).to(torch.bfloat16)                       # [blocks, 7], rounded to bf16
    up = (near.view(torch.int16) + 1).view(torch.bfloat16)
    down = (near.view(torch.int16) - 1).view(torch.bfloat16)
    sign = torch.where(torch.rand(20480, 16, generator=g) < 0.5, -1.0, 1.0)
    x = torch.cat([amax.to(torch.bfloat16), near, up[:, :4], down[:, :4]], dim=1) * sign.to(torch.bfloat16)
    x = x.reshape(-1, 64 * 16)                                       # 64 blocks per row
    for layout in (cabi.SF_ROWMAJOR,):
        q = ops.nvfp4_quantize(x.to(DEV), sf_layout=layout)
        assert_packed_equal(q, x.float().numpy(), layout, what="ties")
    qt = ops.nvfp4_quantize(x.t().contiguous().to(DEV), transpose=True, sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(qt, x.float().numpy(), cabi.SF_ROWMAJOR, what="ties, transposed")


def test_strided_rows():
    wide = synthetic(100, 512, "normal", seed=9, dtype=torch.bfloat16).to(DEV)
    view = wide[:, 128:384]                 # leading dimension 512, 256 columns
    q = ops.nvfp4_quantize(view, sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(q, view.float().cpu().numpy(), cabi.SF_ROWMAJOR, what="strided")
    qt = ops.nvfp4_quantize(view[:96], transpose=True, sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(qt, np.ascontiguousarray(view[:96].float().cpu().numpy().T), cabi.SF_ROWMAJOR, what="strided T")


def test_all_zero_tensor_and_huge_values():
    z = torch.zeros(32, 64, device=DEV)
    q = ops.nvfp4_quantize(z, sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(q, z.cpu().numpy(), cabi.SF_ROWMAJOR, what="zeros")
    big = synthetic(64, 64, "normal", seed=3, dtype=torch.float32) * 1e30
    q = ops.nvfp4_quantize(big.to(DEV), sf_layout=cabi.SF_ROWMAJOR)
    assert_packed_equal(q, big.numpy(), cabi.SF_ROWMAJOR, what="1e30")


def test_shape_errors_raise_value_error():
    with pytest.raises(ValueError, match="does not divide"):
        ops.nvfp4_quantize(torch.zeros(4, 24, device=DEV))
    with pytest.raises(ValueError):
        ops.nvfp4_quantize(torch.zeros(24, 32, device=DEV), transpose=True)     # 24 rows: not blocks of 16


def test_dequantize_roundtrip_bf16_and_tiled_scales():
    x = synthetic(300, 320, "outliers", seed=11, dtype=torch.bfloat16)
    want = O.quantize_dequantize(x.float().numpy())
    for layout in (cabi.SF_ROWMAJOR, cabi.SF_MMA):
        q = ops.nvfp4_quantize(x.to(DEV), sf_layout=layout)
        assert np.array_equal(q.dequantize(torch.float32).cpu().numpy(), want)
        got16 = q.dequantize(torch.bfloat16).float().cpu().numpy()
        assert np.array_equal(got16, torch.from_numpy(want).to(torch.bfloat16).float().numpy())


# the vector product: a warp per row (short and long rows, a row count that is not a multiple of 8); tall and wide
# matrices with the vector staged in shared memory (12290 rows leave a warp with two live rows; 1, 2 and 4 rows per
# warp); few wide rows with a CTA per row
@pytest.mark.parametrize("rows,cols", [(200, 512), (128, 4096), (2050, 1024), (12290, 272), (40, 8208), (600, 8192),
                                       (2372, 8192), (7202, 2048), (14306, 2064)])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_gemv_and_row_sums(rows, cols, layout):
    x = synthetic(rows, cols, "normal", seed=13 + rows, dtype=torch.float32)
    v = torch.randn(cols, generator=torch.Generator().manual_seed(1))
    q = ops.nvfp4_quantize(x.to(DEV), sf_layout=layout)
    deq = O.quantize_dequantize(x.numpy()).astype(np.float64)
    got = ops.nvfp4_gemv(q, v.to(DEV)).cpu().numpy()
    assert np.allclose(got, deq @ v.numpy().astype(np.float64), rtol=1e-5, atol=2e-4)
    assert np.allclose(ops.nvfp4_gemv(q).cpu().numpy(), deq.sum(1), rtol=1e-5, atol=2e-4)


# ---- stochastic rounding ---------------------------------------------------------------------------

GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


@pytest.mark.parametrize("sr_bits", [8, 16])
@pytest.mark.parametrize("transpose", [False, True])
def test_stochastic_rounding_is_unbiased_and_stays_on_neighbours(transpose, sr_bits):
    # every block: one element at 6 (so s = 1 exactly) and 15 copies of a probe value.
    # 16 bits (software): up with probability p in steps of 2^-16.  8 bits (the hardware conversion):
    # up with probability floor(256 p) / 256, i.e. at most 1/256 of the distance to the neighbour short of p.
    probes = [0.1, 0.3, 0.6, 0.85, 1.1, 1.7, 2.3, 3.3, 4.4, 5.5, -0.7, -2.6]
    blocks = 70000                       # 15 * 70000 = 1.05e6 draws per probe
    for p in probes:
        row = torch.full((blocks, 16), p)
        row[:, 0] = 6.0
        x = row.t().contiguous() if transpose else row
        q = ops.nvfp4_quantize(x.to(DEV), transpose=transpose, stochastic=True, seed=1234, offset=int(abs(p) * 100),
                               sf_layout=cabi.SF_ROWMAJOR, sr_bits=sr_bits)
        codes, scales, unit = packed_to_numpy(q)
        vals = O.unpack_codes(codes)[:, 1:]
        lo = GRID[GRID <= abs(p)].max()
        hi = GRID[GRID >= abs(p)].min()
        mags = np.abs(vals)
        assert np.isin(mags, [lo, hi]).all(), f"probe {p}: codes off the two neighbours"
        assert (np.sign(vals[vals != 0]) == np.sign(p)).all()
        frac = (abs(p) - lo) / (hi - lo)
        sigma = (hi - lo) * np.sqrt(frac * (1 - frac) / vals.size)
        if sr_bits == 16:
            assert abs(mags.mean() - abs(p)) < 4 * sigma + 1e-7, f"probe {p}: mean {mags.mean()}"
        else:
            # the reciprocal of the block scale is approximate (2 ulp): p may sit one step of 1/256 lower or higher
            want = lo + (hi - lo) * np.floor(frac * 256) / 256
            assert abs(mags.mean() - want) < 4 * sigma + (hi - lo) / 256 + 1e-7, f"probe {p}: mean {mags.mean()}, want {want}"
            assert abs(mags.mean() - abs(p)) < 4 * sigma + (hi - lo) / 256 + 1e-7
        # scales do not depend on the rounding mode
        qr = ops.nvfp4_quantize(x.to(DEV), transpose=transpose, sf_layout=cabi.SF_ROWMAJOR)
        assert np.array_equal(scales, qr.scales.cpu().numpy()) and unit == np.float32(qr.unit.item())


@pytest.mark.parametrize("sr_bits", [8, 16])
def test_stochastic_rounding_depends_on_seed_and_offset_only(sr_bits):
    x = synthetic(256, 256, "normal", seed=21, dtype=torch.bfloat16).to(DEV)
    a = ops.nvfp4_quantize(x, stochastic=True, seed=7, offset=1, sr_bits=sr_bits).codes
    b = ops.nvfp4_quantize(x, stochastic=True, seed=7, offset=1, sr_bits=sr_bits).codes
    c = ops.nvfp4_quantize(x, stochastic=True, seed=7, offset=2, sr_bits=sr_bits).codes
    assert torch.equal(a, b) and not torch.equal(a, c)
    # dequantized SR output is unbiased against the input within the block scale
    deq = ops.nvfp4_quantize(x, stochastic=True, seed=9, offset=3, sf_layout=cabi.SF_ROWMAJOR, sr_bits=sr_bits).dequantize(torch.float32)
    err = (deq - x.float()).mean().abs().item()
    assert err < 5e-3
    with pytest.raises(ValueError):
        ops.nvfp4_quantize(x, stochastic=True, sr_bits=12)


def test_both_stochastic_roundings_land_on_the_same_two_neighbours():
    # hardware (8 random bits) and software (16) rounding of the same tensor: every element ends on one of its two
    # e2m1 neighbours in both, the scales are the same, and where they differ it is by one grid step
    x = synthetic(512, 1024, "student", seed=4, dtype=torch.bfloat16).to(DEV)
    mean = ops.col_mean(x)
    hw, hwt = ops.nvfp4_quantize_dual(x, mean=mean, stochastic=True, seed=3, offset=1, sf_layout=cabi.SF_ROWMAJOR, sr_bits=8)
    sw, swt = ops.nvfp4_quantize_dual(x, mean=mean, stochastic=True, seed=3, offset=1, sf_layout=cabi.SF_ROWMAJOR, sr_bits=16)
    rn, rnt = ops.nvfp4_quantize_dual(x, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    for a, b, c in ((hw, sw, rn), (hwt, swt, rnt)):
        assert torch.equal(a.scales, b.scales) and torch.equal(a.scales, c.scales) and torch.equal(a.unit, c.unit)
        va, vb, vc = (ops.nvfp4_dequantize(t, torch.float32, add_mean=False) for t in (a, b, c))
        # per block: the scale s = amax / 6 is the value of code magnitude 1.0; neighbouring grid points are at most 2 s apart
        R, C = va.shape
        blocks = lambda v: v.reshape(R, C // 16, 16)
        s_blk = blocks(vc).abs().amax(dim=2, keepdim=True).clamp_min(1e-30) / 4.0      # >= the true s (the block maximum rounds to 4 or 6)
        for v in (va, vb):
            assert bool((blocks(v - vc).abs() <= 2.0001 * s_blk * 1.5).all())          # within one grid step of round-to-nearest
        differ = float((va != vb).float().mean())
        assert 0.02 < differ < 0.6, differ                                             # independent draws differ often, not always


def test_every_bf16_value_below_a_block_maximum():
    # Exact ties are what an approximate division gets wrong, and with bf16 inputs they are common (a
    # quotient of two 8-bit mantissas).  For 4096 block maxima spread over the bf16 range, every bf16
    # value of the seven binades below the maximum (both signs) shares a block with it: 896 magnitudes
    # per maximum, 15 per block beside the maximum.  Codes, scales and unit against the oracle.
    top = torch.arange(0x0F80, 0x7000, 6, dtype=torch.int32)[:4096]              # bf16 bit patterns: normal, far from the ends
    rows = []
    for t in top.tolist():
        mags = torch.arange(t - 896, t, dtype=torch.int32).clamp(min=0)          # the 7 binades below (and up to) t
        signs = (torch.arange(896) % 3 == 0).int() << 15
        vals = (mags | signs).to(torch.int16).view(torch.bfloat16)
        vals = torch.cat([vals, vals[:4]])                                       # 900 = 60 blocks x 15
        block = torch.empty(60, 16, dtype=torch.bfloat16)
        block[:, 0] = torch.tensor([t], dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
        block[:, 1:] = vals.view(60, 15)
        rows.append(block.view(-1))
    x = torch.stack(rows)                                                        # [4096, 960]
    q = ops.nvfp4_quantize(x.to(DEV), sf_layout=cabi.SF_ROWMAJOR)
    codes, scales, unit = packed_to_numpy(q)
    ocodes, oscales, ounit, _ = O.quantize(x.float().numpy(), threads=4)
    assert unit == ounit
    assert np.array_equal(codes, ocodes), f"{int((codes != ocodes).sum())} code bytes differ"
    assert np.array_equal(scales, oscales.reshape(-1))
    # the transposed kernel sees the same blocks as columns
    qt = ops.nvfp4_quantize(x.t().contiguous().to(DEV), transpose=True, sf_layout=cabi.SF_ROWMAJOR)
    assert np.array_equal(qt.codes.cpu().numpy(), ocodes) and np.array_equal(qt.scales.cpu().numpy(), oscales.reshape(-1))


# ---- row-major and transposed quantization from one pass --------------------------------------------------

def _same(a, b):
    return torch.equal(a.codes, b.codes) and torch.equal(a.scales, b.scales) and torch.equal(a.unit, b.unit)


@pytest.mark.parametrize("rows,cols,kind", [(16, 16, "normal"), (48, 80, "outliers"), (128, 64, "normal"), (144, 1536, "student"),
                                            (2048, 2048, "outliers"), (1040, 3584, "student"), (4096, 272, "normal")])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", [cabi.SF_ROWMAJOR, cabi.SF_MMA])
def test_one_pass_gives_both_orientations_bit_for_bit(rows, cols, kind, dtype, layout):
    x = synthetic(rows, cols, kind, seed=rows + 3 * cols, dtype=dtype).to(DEV)
    torch.empty(1 << 22, device=DEV, dtype=torch.uint8).fill_(0xA5)       # stale bytes where the outputs will land
    q, qt = ops.nvfp4_quantize_dual(x, sf_layout=layout)
    assert q.shape == (rows, cols) and qt.shape == (cols, rows)
    assert _same(q, ops.nvfp4_quantize(x, sf_layout=layout))
    assert _same(qt, ops.nvfp4_quantize(x, transpose=True, sf_layout=layout))
    if layout == cabi.SF_ROWMAJOR:                                         # and both against the oracle
        assert_packed_equal(q, x.float().cpu().numpy(), layout, what="dual, row-major")
        assert_packed_equal(qt, x.float().t().contiguous().cpu().numpy(), layout, what="dual, transposed")
    mean = ops.col_mean(x)
    q, qt = ops.nvfp4_quantize_dual(x, mean=mean, sf_layout=layout)
    assert _same(q, ops.nvfp4_quantize(x, mean=mean, sf_layout=layout))
    assert _same(qt, ops.nvfp4_quantize(x, transpose=True, mean=mean, sf_layout=layout))
    assert q.row_vec is mean or torch.equal(q.row_vec, mean)
    assert torch.equal(qt.col_vec, mean)


def test_one_pass_takes_a_strided_view_and_rejects_ragged_token_counts():
    wide = synthetic(256, 1024, "normal", seed=4, dtype=torch.bfloat16).to(DEV)
    view = wide[:, 256:768]
    q, qt = ops.nvfp4_quantize_dual(view, sf_layout=cabi.SF_ROWMAJOR)
    assert _same(q, ops.nvfp4_quantize(view.contiguous(), sf_layout=cabi.SF_ROWMAJOR))
    assert _same(qt, ops.nvfp4_quantize(view.contiguous(), transpose=True, sf_layout=cabi.SF_ROWMAJOR))
    with pytest.raises(ValueError, match="does not divide"):
        ops.nvfp4_quantize_dual(torch.zeros(24, 32, device=DEV))


def test_one_pass_stochastic_keeps_the_scales_and_draws_two_independent_streams():
    x = synthetic(512, 512, "normal", seed=8, dtype=torch.bfloat16).to(DEV)
    q, qt = ops.nvfp4_quantize_dual(x, stochastic=True, seed=3, offset=9, sf_layout=cabi.SF_ROWMAJOR)
    qr, qtr = ops.nvfp4_quantize_dual(x, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(q.scales, qr.scales) and torch.equal(q.unit, qr.unit)
    assert torch.equal(qt.scales, qtr.scales) and torch.equal(qt.unit, qtr.unit)
    # same seed and offset: the same bits again; the two orientations do not share theirs
    q2, qt2 = ops.nvfp4_quantize_dual(x, stochastic=True, seed=3, offset=9, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(q.codes, q2.codes) and torch.equal(qt.codes, qt2.codes)
    sym = synthetic(512, 512, "normal", seed=9, dtype=torch.bfloat16)
    sym = (sym + sym.t()).to(DEV)                                          # x = x^T: both outputs quantize the same matrix
    a, b = ops.nvfp4_quantize_dual(sym, stochastic=True, seed=3, offset=9, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(a.scales, b.scales) and not torch.equal(a.codes, b.codes)
    # both dequantize to x without bias
    for part, ref in ((q, x.float()), (qt, x.float().t())):
        assert (part.dequantize(torch.float32) - ref).mean().abs().item() < 5e-3


# ---- random Hadamard transform folded into the transposed quantizer ------------------------------------------------

def _rotate_blocks_along_rows(x_f32: torch.Tensor, sign_mask: int) -> torch.Tensor:
    """H (s . b) for every block b of 16 consecutive rows of each column, the butterfly in the kernel's order."""
    R, C = x_f32.shape
    v = x_f32.reshape(R // 16, 16, C).clone()
    signs = torch.tensor([-1.0 if (sign_mask >> i) & 1 else 1.0 for i in range(16)], device=x_f32.device)
    v = v * signs[None, :, None]
    h = 1
    while h < 16:
        out = v.clone()
        for i in range(16):
            if (i & h) == 0:
                out[:, i] = v[:, i] + v[:, i + h]
                out[:, i + h] = v[:, i] - v[:, i + h]
        v = out
        h <<= 1
    return v.reshape(R, C)


@pytest.mark.parametrize("rows,cols,dtype", [(16, 16, torch.float32), (256, 64, torch.bfloat16), (2048, 1536, torch.bfloat16), (144, 272, torch.float32)])
def test_rotated_transposed_quantization_is_the_quantization_of_the_rotated_tensor(rows, cols, dtype):
    from fp4_post_b200.Metis.Metis.bitlinear import LinearLowbitFunction as F
    x = synthetic(rows, cols, "outliers", seed=rows + cols, dtype=dtype).to(DEV)
    signs = F._get_hadamard_sign(16, "cpu", torch.float32)
    mask = sum(1 << i for i in range(16) if signs[i] < 0)
    q = ops.nvfp4_quantize(x, transpose=True, hadamard_signs=mask, sf_layout=cabi.SF_ROWMAJOR)
    rotated = _rotate_blocks_along_rows(x.float(), mask)
    # the same matrix the reference's torch path builds: (tile . signs) @ H per tile of 16 along the tokens
    want_ref = F._apply_hadamard_blocks(x.float().t().contiguous(), inverse=False).t()
    assert torch.allclose(rotated, want_ref, rtol=1e-5, atol=1e-5)
    assert_packed_equal(q, rotated.t().contiguous().cpu().numpy(), cabi.SF_ROWMAJOR, what="rotated transposed quantizer")
    # with a mean: subtracted first, then rotated
    mean = ops.col_mean(x)
    q = ops.nvfp4_quantize(x, transpose=True, mean=mean, hadamard_signs=mask, sf_layout=cabi.SF_ROWMAJOR)
    rotated = _rotate_blocks_along_rows(x.float() - mean, mask)
    assert_packed_equal(q, rotated.t().contiguous().cpu().numpy(), cabi.SF_ROWMAJOR, what="rotated, mean-centred")
    # the dual quantizer rotates its transposed output only
    qd, qdt = ops.nvfp4_quantize_dual(x, mean=mean, hadamard_signs=mask, sf_layout=cabi.SF_ROWMAJOR)
    assert _same(qdt, q) and _same(qd, ops.nvfp4_quantize(x, mean=mean, sf_layout=cabi.SF_ROWMAJOR))


def test_two_operands_rotated_alike_give_sixteen_times_the_plain_product():
    # (H s)^T (H s) = 16 I: the weight-gradient product of rotated operands, with alpha = 1/16, is the plain
    # product up to the (different) quantization noise
    M, N, K = 2048, 256, 384
    d = synthetic(M, N, "normal", seed=1, dtype=torch.bfloat16).to(DEV)
    x = synthetic(M, K, "outliers", seed=2, dtype=torch.bfloat16).to(DEV)
    mask = 0b1010011100101101
    plain = ops.nvfp4_gemm(ops.nvfp4_quantize(d, transpose=True), ops.nvfp4_quantize(x, transpose=True), out_dtype=torch.float32)
    rot = ops.nvfp4_gemm(ops.nvfp4_quantize(d, transpose=True, hadamard_signs=mask), ops.nvfp4_quantize(x, transpose=True, hadamard_signs=mask),
                         out_dtype=torch.float32, alpha=1.0 / 16)
    exact = d.double().t() @ x.double()
    e_plain = (plain.double() - exact).norm() / exact.norm()
    e_rot = (rot.double() - exact).norm() / exact.norm()
    assert e_plain < 0.2 and e_rot < 0.2
    assert e_rot < e_plain * 1.1                                  # the rotation spreads the outlier channels: no worse


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(64, 32), (128, 4096), (1024, 528), (16384, 128), (4096, 4096)])
@pytest.mark.parametrize("stochastic", [False, True])
def test_dual_quantizer_forms_the_token_sums_of_the_transposed_output(rows, cols, stochastic):
    """token_sums_t[k] = sum over the tokens of the quantized values of column k: equal to the row sums the
    gemv kernel forms from the same codes and scales (other order of the additions), and the same on every run."""
    torch.manual_seed(rows + cols)
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16) * 3 + 0.5
    mean = ops.col_mean(x)
    for layout in (cabi.SF_ROWMAJOR, cabi.SF_MMA):
        q, qt = ops.nvfp4_quantize_dual(x, mean=mean, stochastic=stochastic, seed=11, offset=4, sf_layout=layout, token_sums=True)
        assert qt.token_sums is not None and qt.token_sums.shape == (cols,)
        want = ops.nvfp4_gemv(qt, None)
        dense = ops.nvfp4_dequantize(qt, torch.float32, add_mean=False).double().sum(dim=1)
        scale = ops.nvfp4_dequantize(qt, torch.float32, add_mean=False).abs().double().sum(dim=1) + 1e-30
        assert ((qt.token_sums.double() - dense).abs() / scale).max().item() < 1e-5
        assert ((want.double() - dense).abs() / scale).max().item() < 1e-5
        q2, qt2 = ops.nvfp4_quantize_dual(x, mean=mean, stochastic=stochastic, seed=11, offset=4, sf_layout=layout, token_sums=True)
        assert torch.equal(qt.token_sums, qt2.token_sums)
        # the outputs themselves are what they were without the by-product
        q3, qt3 = ops.nvfp4_quantize_dual(x, mean=mean, stochastic=stochastic, seed=11, offset=4, sf_layout=layout)
        assert qt3.token_sums is None
        assert torch.equal(qt.codes, qt3.codes) and torch.equal(qt.scales, qt3.scales) and torch.equal(q.scales, q3.scales)


@pytest.mark.gpu
def test_token_sums_are_refused_where_the_scale_pass_cannot_form_them():
    x = torch.randn(48, 64, device=DEV, dtype=torch.bfloat16)
    q, qt = ops.nvfp4_quantize_dual(x, token_sums=True)          # rows not a multiple of 64: the host wrapper leaves them out
    assert qt.token_sums is None
    L = cabi.lib()
    ws = torch.empty(L.metis_nvfp4_quantize_dual_workspace_bytes(48, 64), dtype=torch.uint8, device=DEV)
    sums = torch.empty(64, dtype=torch.float32, device=DEV)
    rc = L.metis_nvfp4_quantize_dual(x.data_ptr(), cabi.DTYPE_BF16, 48, 64, 64, None, 0, 0, 0, cabi.SF_ROWMAJOR,
                                     q.codes.data_ptr(), q.scales.data_ptr(), q.unit.data_ptr(),
                                     qt.codes.data_ptr(), qt.scales.data_ptr(), qt.unit.data_ptr(), sums.data_ptr(),
                                     ws.data_ptr(), ws.numel(), None)
    assert rc == -2          # METIS_ERR_BAD_SHAPE


@pytest.mark.gpu
@pytest.mark.parametrize("defer", ["rowmajor", "transposed"])
@pytest.mark.parametrize("stochastic", [False, True])
def test_deferred_scale_pass_writes_what_the_undeferred_call_writes(defer, stochastic):
    torch.manual_seed(17)
    x = torch.randn(1024, 768, device=DEV, dtype=torch.bfloat16) * 2 - 0.3
    mean = ops.col_mean(x)
    kw = dict(mean=mean, stochastic=stochastic, seed=5, offset=3, token_sums=True)
    want_q, want_t = ops.nvfp4_quantize_dual(x, **kw)
    q, qt, finish = ops.nvfp4_quantize_dual(x, defer=defer, **kw)
    torch.cuda.synchronize()
    # the half that was not deferred is complete, the codes of both are
    done, late = (qt, q) if defer == "rowmajor" else (q, qt)
    want_done, want_late = (want_t, want_q) if defer == "rowmajor" else (want_q, want_t)
    assert torch.equal(done.codes, want_done.codes) and torch.equal(done.scales, want_done.scales) and torch.equal(done.unit, want_done.unit)
    assert torch.equal(late.codes, want_late.codes)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        finish()
    side.synchronize()
    assert torch.equal(late.scales, want_late.scales) and torch.equal(late.unit, want_late.unit)
    assert torch.equal(qt.token_sums, want_t.token_sums)
    with pytest.raises(ValueError):
        ops.nvfp4_quantize_dual(x, defer="both")
