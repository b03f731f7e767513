"""Parity at the shapes of the benchmark configurations that the small-case tests do not reach.

GEMM       M in {4096, 16384} x (N, K) in {(14336, 4096), (4096, 14336)} x rank in {0, 32, 256}:
           the forward product and both backward products (dX = Q(D) Qt(W), dW = Qt(D) Qt(x),
           operands from the transposed quantizer), sampled output rows against a float64 product
           of the dequantized operands each launch was given.  rel-L2 <= 1e-5 (bar: 1e-3).
quantizer  tokens in {8192, 65536} x hidden in {1536, 3584, 4096}, bf16 Student-t (nu = 3) plus a
           per-channel offset: the row kernel, the transposed kernel and the RMSNorm-fused kernel
           against the oracle on sampled rows that contain the block with the largest scale (such a
           sample has the unit of the whole tensor, so codes AND scale bytes must be equal); the
           stochastic modes keep the scales of round-to-nearest and stay on the two neighbours.
The CPU oracle sees a few dozen rows per case, the kernels the whole tensor.
"""
import numpy as np
import pytest
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O
from gpu_helpers import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


# ---- GEMM ------------------------------------------------------------------------------------------

def _randn(rows, cols, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(rows, cols, device=DEV, generator=g) * scale).to(torch.bfloat16)


def _sampled_check(qa, qb, lowrank, out, rows):
    """float64 product of what the kernel was given, on the sampled output rows."""
    idx = torch.tensor(rows, device=DEV)
    a = ops.nvfp4_dequantize(qa, torch.float32, add_mean=False)[idx].double()
    want = a @ ops.nvfp4_dequantize(qb, torch.float32, add_mean=False).double().t()
    if lowrank is not None:
        t, u = lowrank
        scale = float(qa.unit.item()) * float(qb.unit.item())
        want = want + (t[idx].double() * scale) @ u.double().t()
    err = rel_l2(out[idx].double().cpu().numpy(), want.cpu().numpy())
    assert err <= 1e-5, err


def _rows(M, seed, n=48):
    g = torch.Generator().manual_seed(seed)
    return sorted({0, M - 1, *torch.randint(0, M, (n,), generator=g).tolist()})


@pytest.mark.parametrize("rank", [0, 32, 256])
@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [4096, 16384])
def test_rectangular_training_shapes_forward_and_both_backward_products(M, N, K, rank):
    x = _randn(M, K, seed=M + K)
    w = _randn(N, K, seed=N + K + 1, scale=K ** -0.5)
    d = _randn(M, N, seed=M + N + 2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def side(rows, cols, qa, qb, seed):
        if rank == 0:
            return None
        scale = float(qa.unit.item()) * float(qb.unit.item())
        t = (_randn(rows, rank, seed=seed, scale=3.0).float() / scale).to(torch.bfloat16)
        return t, _randn(cols, rank, seed=seed + 1, scale=rank ** -0.5)

    # forward: contraction over K
    qx, qw = ops.nvfp4_quantize(x), ops.nvfp4_quantize(w)
    lr = side(M, N, qx, qw, 7)
    y = ops.nvfp4_gemm(qx, qw, lowrank=lr, out_dtype=torch.float32, status=status)
    _sampled_check(qx, qw, lr, y, _rows(M, 1))
    del y
    # dX: contraction over N, the weight quantized along N by the transposed quantizer
    qd, qw_t = ops.nvfp4_quantize(d), ops.nvfp4_quantize(w, transpose=True)
    assert qw_t.shape == (K, N)
    lr = side(M, K, qd, qw_t, 9)
    dx = ops.nvfp4_gemm(qd, qw_t, lowrank=lr, out_dtype=torch.float32, status=status)
    _sampled_check(qd, qw_t, lr, dx, _rows(M, 2))
    del dx
    # dW: contraction over tokens, both operands from the transposed quantizer
    qd_t, qx_t = ops.nvfp4_quantize(d, transpose=True), ops.nvfp4_quantize(x, transpose=True)
    assert qd_t.shape == (N, M) and qx_t.shape == (K, M)
    lr = side(N, K, qd_t, qx_t, 11)
    dw = ops.nvfp4_gemm(qd_t, qx_t, lowrank=lr, out_dtype=torch.float32, status=status)
    _sampled_check(qd_t, qx_t, lr, dw, _rows(N, 3))
    torch.cuda.synchronize()
    assert status.item() == 0


# ---- quantizers ----------------------------------------------------------------------------------------

def _student(tokens, hidden, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    z = torch.randn(tokens, hidden, device=DEV, generator=g)
    chi = torch.zeros_like(z)
    for _ in range(3):
        chi += torch.randn(tokens, hidden, device=DEV, generator=g).pow(2)
    x = z / (chi / 3).sqrt() + 2.0 * torch.randn(1, hidden, device=DEV, generator=g)
    return x.to(torch.bfloat16)


def _sample_with_top_row(values_f32, n, seed):
    """row indices that include the row holding the block with the largest magnitude"""
    R, C = values_f32.shape
    top = 0
    best = -1.0
    for r0 in range(0, R, 8192):                     # in slabs: no full-size fp32 temporary
        m = values_f32[r0:r0 + 8192].abs().amax(dim=1)
        v, i = m.max(dim=0)
        if float(v) > best:
            best, top = float(v), r0 + int(i)
    g = torch.Generator().manual_seed(seed)
    return sorted({top, 0, R - 1, *torch.randint(0, R, (n,), generator=g).tolist()})


def _assert_rows_equal_oracle(q, source_rows_f32, rows, row_len, what):
    codes, scales, unit, _ = O.quantize(source_rows_f32)
    assert np.float32(q.unit.item()) == unit, what
    assert np.array_equal(q.codes[rows].cpu().numpy(), codes), what
    assert np.array_equal(q.scales.view(-1, row_len // 16)[rows].cpu().numpy(), scales), what


GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _assert_stochastic_on_neighbours(q_sr, q_rn, source, slab=4096):
    """q_sr: stochastic quantization with row-major scales of `source` [R, C] (fp32-convertible);
    same scales and unit as round to nearest, every code one of the two grid neighbours of |x| / s."""
    assert torch.equal(q_sr.scales, q_rn.scales) and torch.equal(q_sr.unit, q_rn.unit)
    grid = GRID.to(DEV)
    R, C = source.shape
    for r0 in range(0, R, slab):
        x = source[r0:r0 + slab].float()
        rows = x.shape[0]
        s = x.abs().view(rows, C // 16, 16).amax(dim=2) / 6 + 1e-9
        v = (x.abs().view(rows, C // 16, 16) / s[:, :, None]).view(rows, C)
        c = q_sr.codes[r0:r0 + slab]
        nib = torch.stack([c & 0xF, c >> 4], dim=2).view(rows, C).long()
        mag = grid[nib & 7]
        # the stochastic path divides with an approximate reciprocal: a value within a few ulp of a grid
        # point may take that point's other neighbour
        lo = grid[torch.bucketize(v * (1 - 4e-6), grid, right=True) - 1]
        hi = grid[torch.bucketize(v * (1 + 4e-6), grid).clamp(max=7)]
        assert bool(((mag >= lo) & (mag <= hi)).all()), f"rows {r0}..: a code left its neighbours"
        neg = (nib >> 3).bool()
        assert bool((neg == (x < 0)).all())


@pytest.mark.parametrize("hidden", [1536, 3584, 4096])
@pytest.mark.parametrize("tokens", [8192, 65536])
def test_row_and_transposed_quantizers_at_sweep_sizes(tokens, hidden):
    x = _student(tokens, hidden, seed=tokens + hidden)
    # row kernel against the oracle
    q = ops.nvfp4_quantize(x, sf_layout=cabi.SF_ROWMAJOR)
    rows = _sample_with_top_row(x, 40, seed=1)
    _assert_rows_equal_oracle(q, x[rows].float().cpu().numpy(), rows, hidden, "row kernel")
    # transposed kernel against the oracle on columns of x, and against the row kernel on the transpose
    xt = x.t().contiguous()
    qt = ops.nvfp4_quantize(x, transpose=True, sf_layout=cabi.SF_ROWMAJOR)
    cols = _sample_with_top_row(xt, 24, seed=2)
    _assert_rows_equal_oracle(qt, xt[cols].float().cpu().numpy(), cols, tokens, "transposed kernel")
    qr = ops.nvfp4_quantize(xt, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(qt.codes, qr.codes) and torch.equal(qt.scales, qr.scales) and torch.equal(qt.unit, qr.unit)
    # the tiled scale order holds the same bytes
    qm = ops.nvfp4_quantize(x, sf_layout=cabi.SF_MMA)
    assert torch.equal(qm.codes, q.codes)
    sample = sorted(set(rows[:8]))
    want = O.scales_to_mma_layout(q.scales.view(tokens, hidden // 16).cpu().numpy(), hidden)
    assert np.array_equal(qm.scales.cpu().numpy(), want), f"tiled scales differ (rows {sample})"
    # mean-centred, both orientations, against the oracle with the kernel's own column mean
    mean = ops.col_mean(x)
    want_mean = x.float().mean(dim=0)
    assert torch.allclose(mean, want_mean, rtol=1e-5, atol=1e-5)
    qc = ops.nvfp4_quantize(x, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    centred = x.float() - mean
    rows_c = _sample_with_top_row(centred, 24, seed=3)
    _assert_rows_equal_oracle(qc, centred[rows_c].cpu().numpy(), rows_c, hidden, "mean-centred row kernel")
    qct = ops.nvfp4_quantize(x, transpose=True, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    centred_t = centred.t().contiguous()
    del centred
    cols_c = _sample_with_top_row(centred_t, 16, seed=4)
    _assert_rows_equal_oracle(qct, centred_t[cols_c].cpu().numpy(), cols_c, tokens, "mean-centred transposed kernel")
    # one pass for both orientations: the same bytes as the two separate kernels
    qd, qdt = ops.nvfp4_quantize_dual(x, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(qd.codes, q.codes) and torch.equal(qd.scales, q.scales) and torch.equal(qd.unit, q.unit)
    assert torch.equal(qdt.codes, qt.codes) and torch.equal(qdt.scales, qt.scales) and torch.equal(qdt.unit, qt.unit)
    qd, qdt = ops.nvfp4_quantize_dual(x, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(qd.codes, qc.codes) and torch.equal(qd.scales, qc.scales) and torch.equal(qd.unit, qc.unit)
    assert torch.equal(qdt.codes, qct.codes) and torch.equal(qdt.scales, qct.scales) and torch.equal(qdt.unit, qct.unit)
    qd, qdt = ops.nvfp4_quantize_dual(x, stochastic=True, seed=5, offset=2, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    _assert_stochastic_on_neighbours(qd, qc, x.float() - mean)
    _assert_stochastic_on_neighbours(qdt, qct, centred_t, slab=256)
    del qd, qdt
    # stochastic rounding, both orientations
    qs = ops.nvfp4_quantize(x, stochastic=True, seed=11, offset=5, sf_layout=cabi.SF_ROWMAJOR)
    _assert_stochastic_on_neighbours(qs, q, x)
    qst = ops.nvfp4_quantize(x, transpose=True, stochastic=True, seed=11, offset=6, sf_layout=cabi.SF_ROWMAJOR)
    _assert_stochastic_on_neighbours(qst, qt, xt, slab=256)
    qsc = ops.nvfp4_quantize(x, transpose=True, stochastic=True, seed=11, offset=7, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    _assert_stochastic_on_neighbours(qsc, qct, centred_t, slab=256)


def _reference_norm(x, gamma, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * gamma


@pytest.mark.parametrize("hidden", [1536, 3584, 4096])
@pytest.mark.parametrize("tokens", [8192, 65536])
def test_rmsnorm_quantizer_at_sweep_sizes(tokens, hidden):
    x = _student(tokens, hidden, seed=3 * tokens + hidden)
    g = torch.Generator(device=DEV).manual_seed(hidden)
    gamma = (1.0 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(torch.bfloat16)
    q, y = ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6, sf_layout=cabi.SF_ROWMAJOR, return_norm=True)
    # (a) the normalised output is within one bf16 ulp of the fp32 chain, identical almost everywhere
    rows = _sample_with_top_row(y, 40, seed=5)
    want = _reference_norm(x[rows], gamma, 1e-6).float()
    got = y[rows].float()
    assert bool(((got - want).abs() <= want.abs().clamp(min=1e-30) * 2.0 ** -7).all())
    assert float((got == want).float().mean()) > 0.995
    # (b) codes, scales and unit bit-exact against the oracle on the kernel's own normalised rows
    _assert_rows_equal_oracle(q, got.cpu().numpy(), rows, hidden, "rmsnorm -> quant")
    # the tiled layout and the call without the normalised output give the same bytes
    q2 = ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6, sf_layout=cabi.SF_MMA)
    assert torch.equal(q2.codes, q.codes) and torch.equal(q2.unit, q.unit)
    want_sf = O.scales_to_mma_layout(q.scales.view(tokens, hidden // 16).cpu().numpy(), hidden)
    assert np.array_equal(q2.scales.cpu().numpy(), want_sf)
    # and the stand-alone row quantizer on that normalised output agrees with the fused kernel
    q3 = ops.nvfp4_quantize(y, sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(q3.codes, q.codes) and torch.equal(q3.scales, q.scales) and torch.equal(q3.unit, q.unit)
