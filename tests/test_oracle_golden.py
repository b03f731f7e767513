"""The CPU oracle against vectors produced by the reference itself (tests/golden)."""
import numpy as np
import pytest

from oracle import nvfp4_oracle as O


def case_names():
    return ["randn_64x256", "outliers_32x512", "bf16valued_48x1536", "weights_128x256", "special_8x64"]


@pytest.mark.parametrize("name", case_names())
def test_quantizer_matches_reference_bit_for_bit(quant_golden, name):
    g = quant_golden[name]
    codes, scales, unit, bscale = O.quantize(g["x"])
    assert np.array_equal(bscale, g["block_scale"])
    assert np.float32(unit) == g["unit"]
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(scales, g["scales"])
    deq = O.dequantize(codes, scales, unit)
    assert np.array_equal(deq, g["qdq"])            # the reference's fake-quant output


def test_threads_do_not_change_the_result(quant_golden):
    g = quant_golden["outliers_32x512"]
    one = O.quantize(g["x"], threads=1)
    many = O.quantize(g["x"], threads=5)
    for a, b in zip(one, many):
        assert np.array_equal(a, b)


def test_mean_centred_quantizer_matches_reference(quant_golden):
    g = quant_golden["mean_96x256"]
    codes, scales, unit, _ = O.quantize(g["x"], col_mean=g["mean"])
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(scales, g["scales"])
    assert np.float32(unit) == g["unit"]
    assert np.array_equal(O.dequantize(codes, scales, unit, col_mean=g["mean"]), g["qdq"])


def test_rounding_ties_go_to_the_even_code(quant_golden):
    g = quant_golden["special_8x64"]
    # row 0, block 0 holds {.25,.75,1.25,1.75,2.5,3.5,5,6} and their negatives with s == 1
    nib = np.stack([g["codes"][0, :8] & 15, g["codes"][0, :8] >> 4], axis=-1).reshape(-1)
    assert list(nib[:8]) == [0, 2, 2, 4, 4, 6, 6, 7]
    assert list(nib[8:16]) == [8, 10, 10, 12, 12, 14, 14, 15]
    # an all-zero block: code 0 everywhere; -0.0 has no sign bit, a tiny negative has one
    assert not g["codes"][2, :8].any()
    assert g["codes"][2, 8] == 0x00 and g["codes"][2, 9] == 0x08


def test_rejects_a_width_that_blocks_of_16_do_not_divide():
    with pytest.raises(ValueError):
        O.quantize(np.zeros((4, 24), np.float32))


def test_rmsnorm_then_quantize_matches_reference(rmsnorm_golden):
    import torch
    for name, g in rmsnorm_golden:
        gamma_bf16 = "gbf16" in name
        x = torch.from_numpy(g["x"]).to(torch.bfloat16)
        gamma = torch.from_numpy(g["gamma"])
        gamma = gamma.to(torch.bfloat16) if gamma_bf16 else gamma
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype) * gamma
        assert np.array_equal(y.float().numpy(), g["y"])
        codes, scales, unit, _ = O.quantize(g["y"])
        assert np.array_equal(codes, g["codes"]) and np.array_equal(scales, g["scales"])
        assert np.float32(unit) == g["unit"]


def test_scale_tile_order():
    rng = np.random.default_rng(0)
    R, C = 200, 320
    sc = rng.integers(0, 127, size=(R, C // 16), dtype=np.uint8)
    tiled = O.scales_to_mma_layout(sc, C)
    tiles = ((C + 255) // 256) * 4
    assert tiled.size == 2 * tiles * 512
    for r, k in [(0, 0), (31, 3), (32, 0), (127, 19), (128, 4), (199, 19)]:
        off = ((r // 128) * tiles + k // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + k % 4
        assert tiled[off] == sc[r, k]
    assert tiled.sum() == sc.sum()     # everything else is zero padding


def test_e4m3_helpers_agree():
    allb = np.arange(256, dtype=np.uint8)
    a = O.e4m3_to_f32(allb)
    b = np.array([O.lib().oracle_e4m3fn_to_f32(int(v)) for v in allb], dtype=np.float32)
    assert np.array_equal(a, b, equal_nan=True)
    finite = allb[~np.isnan(a)]
    back = np.array([O.lib().oracle_f32_to_e4m3fn(float(v)) for v in a[finite]], dtype=np.uint8)
    # every finite byte survives a round trip (-0 keeps its sign)
    assert np.array_equal(back, finite)


def test_conversion_rounding_equals_the_reference_after_the_second_rounding_step():
    # every fp32 quotient from below the first tie (0.25) to past the largest code: 4.7e7 values
    plain, fixed, where = O.compare_conversion_rounding(0.125, 6.5)
    assert fixed == 0
    # a single rounding differs from the reference's two at exactly the fp32 neighbours of three ties
    assert plain == 3
    assert list(where) == [np.nextafter(np.float32(2.5), np.float32(3)), np.nextafter(np.float32(3.5), np.float32(3)),
                           np.nextafter(np.float32(5), np.float32(6))]
