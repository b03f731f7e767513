"""The benchmark's own sizes (16384 tokens, hidden 4096, rank 128), where the CPU oracle cannot
cover the whole tensor in seconds: properties that do not depend on the size, plus the oracle on
rows that pin the tensor-wide quantities.

quantizer  * the transposed kernel on x equals the row kernel on x^T, bit for bit (two kernels,
             two memory paths, one answer);
           * permuting the rows of x permutes the rows of the packed result (unit unchanged);
           * a sample of rows that contains the block with the largest scale has the same unit as
             the whole tensor, so the oracle's codes AND scale bytes for that sample must equal
             the kernel's rows.
GEMM       * rows of the product do not depend on how many other rows there are (CTA pairs on
             the whole matrix against the same kernel on a slice);
           * alpha scales the result exactly; splitting K in two adds up;
           * sampled entries against a float64 product of the dequantized operands.
layer      * the captured graph of the full-size step replays to the eager forward, bit for bit.
"""
import numpy as np
import pytest
import torch

import fp4_post_b200
from fp4_post_b200 import cabi, ops
from fp4_post_b200.graphs import GraphedStep
from oracle import nvfp4_oracle as O

fp4_post_b200.install_reference_aliases()

from Metis.Metis.bitlinear import BitLinear  # noqa: E402
from grpo.grpo import MetisArgs  # noqa: E402
from gpu_helpers import rel_l2  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
M, K, N, R = 16384, 4096, 4096, 128


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


@pytest.fixture(scope="module")
def activations():
    g = torch.Generator().manual_seed(123)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[: K // 100]] *= 20            # 1 % outlier channels, as in the bench
    return x.to(torch.bfloat16).to(DEV)


def _same(a, b):
    return torch.equal(a.codes, b.codes) and torch.equal(a.scales, b.scales) and torch.equal(a.unit, b.unit)


def test_transposed_quantizer_equals_row_quantizer_on_the_transpose(activations):
    x = activations
    qt = ops.nvfp4_quantize(x, transpose=True, sf_layout=cabi.SF_ROWMAJOR)
    qr = ops.nvfp4_quantize(x.t().contiguous(), sf_layout=cabi.SF_ROWMAJOR)
    assert qt.shape == (K, M) and _same(qt, qr)
    mean = ops.col_mean(x)
    qt = ops.nvfp4_quantize(x, transpose=True, mean=mean, sf_layout=cabi.SF_ROWMAJOR)
    centred_t = (x.float() - mean).t().contiguous()                  # fp32 subtraction, as the kernels do
    qr = ops.nvfp4_quantize(centred_t, sf_layout=cabi.SF_ROWMAJOR)
    assert _same(qt, qr)


def test_row_permutation_commutes_with_the_quantizer(activations):
    x = activations
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(5)).to(DEV)
    q = ops.nvfp4_quantize(x, sf_layout=cabi.SF_ROWMAJOR)
    qp = ops.nvfp4_quantize(x[perm].contiguous(), sf_layout=cabi.SF_ROWMAJOR)
    assert torch.equal(qp.unit, q.unit)
    assert torch.equal(qp.codes, q.codes[perm])
    assert torch.equal(qp.scales.view(M, K // 16), q.scales.view(M, K // 16)[perm])


def test_rows_holding_the_largest_block_pin_unit_codes_and_scales_against_the_oracle(activations):
    x = activations
    q = ops.nvfp4_quantize(x, sf_layout=cabi.SF_ROWMAJOR)
    block_max = x.float().abs().view(M, K // 16, 16).amax(dim=2)
    top_row = int(block_max.amax(dim=1).argmax().item())
    rows = sorted({top_row, 0, M - 1, *torch.randint(0, M, (61,), generator=torch.Generator().manual_seed(9)).tolist()})
    sample = x[rows].float().cpu().numpy()
    codes, scales, unit, _ = O.quantize(sample)
    assert np.float32(q.unit.item()) == unit
    assert np.array_equal(q.codes[rows].cpu().numpy(), codes)
    assert np.array_equal(q.scales.view(M, K // 16)[rows].cpu().numpy(), scales)


@pytest.fixture(scope="module")
def operands(activations):
    g = torch.Generator().manual_seed(77)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    t = (torch.randn(M, R, generator=g) * 3).to(torch.bfloat16).to(DEV)
    u = (torch.randn(N, R, generator=g) / R ** 0.5).to(torch.bfloat16).to(DEV)
    return ops.nvfp4_quantize(activations), ops.nvfp4_quantize(w), t, u


def test_rows_of_the_product_do_not_depend_on_the_other_rows(activations, operands):
    qa, qb, t, u = operands
    full = ops.nvfp4_gemm(qa, qb, lowrank=(t, u), out_dtype=torch.float32)
    rows = 512
    # the slice must keep the unit of the whole tensor: quantize the whole, then view its first rows
    part = ops.NVFP4Tensor(qa.codes[:rows], qa.scales[: (rows // 128) * (qa.scales.numel() // (M // 128))], qa.unit,
                           (rows, K), qa.sf_layout)
    sliced = ops.nvfp4_gemm(part, qb, lowrank=(t[:rows].contiguous(), u), out_dtype=torch.float32)
    assert torch.equal(full[:rows], sliced)


def test_alpha_is_exact_and_k_halves_add_up(activations, operands):
    qa, qb, _, _ = operands
    one = ops.nvfp4_gemm(qa, qb, out_dtype=torch.float32)
    two = ops.nvfp4_gemm(qa, qb, out_dtype=torch.float32, alpha=2.0)
    assert torch.equal(two, one * 2)
    # K halves: the first 2048 columns of both operands, re-quantized, are the same blocks with
    # possibly another unit, so compare through the dequantized values
    x_lo, x_hi = activations[:, : K // 2].contiguous(), activations[:, K // 2:].contiguous()
    w = qb.dequantize(torch.float32)
    q_lo, q_hi = ops.nvfp4_quantize(x_lo), ops.nvfp4_quantize(x_hi)
    w_lo, w_hi = ops.nvfp4_quantize(w[:, : K // 2].contiguous()), ops.nvfp4_quantize(w[:, K // 2:].contiguous())
    halves = ops.nvfp4_gemm(q_lo, w_lo, out_dtype=torch.float32) + ops.nvfp4_gemm(q_hi, w_hi, out_dtype=torch.float32)
    whole_from_halves = (torch.cat([q_lo.dequantize(torch.float32), q_hi.dequantize(torch.float32)], dim=1)[:256].double()
                         @ torch.cat([w_lo.dequantize(torch.float32), w_hi.dequantize(torch.float32)], dim=1).double().t())
    assert rel_l2(halves[:256].double().cpu().numpy(), whole_from_halves.cpu().numpy()) <= 1e-5


def test_sampled_entries_against_float64(operands):
    qa, qb, t, u = operands
    out = ops.nvfp4_gemm(qa, qb, lowrank=(t, u), out_dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    rows = torch.randint(0, M, (96,), generator=g).to(DEV)
    a = qa.dequantize(torch.float32)[rows].double()
    b = qb.dequantize(torch.float32).double()
    scale = float(qa.unit.item()) * float(qb.unit.item())
    want = a @ b.t() + (t[rows].double() * scale) @ u.double().t()
    assert rel_l2(out[rows].double().cpu().numpy(), want.cpu().numpy()) <= 1e-5


def test_full_size_step_replays_from_a_graph():
    torch.manual_seed(0)
    args = MetisArgs(forward_svd_rank=R, activation_lowrank_svd=R, backward_lowrank_svd=R, cache_quantized_weight=True)
    args.device = DEV
    layer = BitLinear(K, N, args=args, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "full"
    with torch.no_grad():
        layer.warmup_linear.weight.copy_(torch.randn(N, K, device=DEV) / K ** 0.5)
    layer.split()
    params = list(layer.parameters())
    x = torch.randn(1, M, K, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    gout = torch.randn(1, M, N, device=DEV, dtype=torch.bfloat16)

    def step():
        for p in params:
            p.grad = None
        x.grad = None
        y = layer(x)
        y.backward(gout)
        return y, x.grad

    y_eager = step()[0].detach().clone()     # detached: a live autograd graph from the default stream would break the capture
    graphed = GraphedStep(step, warmup=1)
    y1 = graphed()[0].detach().clone()
    gx1 = graphed.outputs[1].detach().clone()
    y2, gx2 = graphed()
    assert torch.equal(y1, y_eager) and torch.equal(y2, y_eager)
    assert torch.isfinite(gx2).all() and not torch.equal(gx1, gx2)       # stochastic backward: fresh bits per replay
    graphed.release()
