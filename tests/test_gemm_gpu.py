"""tcgen05 NVFP4 GEMM (+ fused bf16 rank-r product, rank-1 epilogue terms, addend) against the FP32
dequantize-then-matmul oracle of the operands it was given.  Tolerance: rel-L2 <= 1e-3 (the
stated bar) for fp32 output; bf16 output is compared with the oracle rounded to bf16."""
import numpy as np
import pytest
import torch

from fp4_post_b200 import cabi, ops
from oracle import nvfp4_oracle as O
from gpu_helpers import rel_l2, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-3


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def operands(M, N, K, seed):
    a = synthetic(M, K, "normal", seed=seed, dtype=torch.bfloat16)
    b = synthetic(N, K, "weights", seed=seed + 1, dtype=torch.bfloat16)
    qa = ops.nvfp4_quantize(a.to(DEV), sf_layout=cabi.SF_MMA)
    qb = ops.nvfp4_quantize(b.to(DEV), sf_layout=cabi.SF_MMA)
    return qa, qb, O.quantize_dequantize(a.float().numpy()), O.quantize_dequantize(b.float().numpy())


def run(qa, qb, **kw):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.nvfp4_gemm(qa, qb, status=status, **kw)
    torch.cuda.synchronize()
    assert status.item() == 0, f"device status {status.item()}"
    return out


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 256, 256), (128, 128, 64), (16, 128, 512), (200, 136, 320),
                                   (384, 512, 1024), (256, 4096, 2048), (1024, 1536, 4096), (130, 264, 96)])
def test_plain_product(M, N, K):
    qa, qb, da, db = operands(M, N, K, seed=M + N + K)
    want = O.gemm_reference(da, db)
    got = run(qa, qb, out_dtype=torch.float32).cpu().numpy()
    assert rel_l2(got, want) <= TOL, rel_l2(got, want)
    assert rel_l2(got, want) <= 1e-5          # fp32 accumulation of exact products: far inside the bar
    got16 = run(qa, qb, out_dtype=torch.bfloat16).float().cpu().numpy()
    want16 = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    assert rel_l2(got16, want16) <= TOL


@pytest.mark.parametrize("rank", [32, 64, 128, 256, 40])
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (200, 136, 320)])
def test_fused_low_rank_product(M, N, K, rank):
    qa, qb, da, db = operands(M, N, K, seed=rank)
    g = torch.Generator().manual_seed(rank)
    t = (torch.randn(M, rank, generator=g) * 3).to(torch.bfloat16)
    u = (torch.randn(N, rank, generator=g) / rank ** 0.5).to(torch.bfloat16)
    scale = float(qa.unit.item()) * float(qb.unit.item())
    # the kernel takes T in accumulator units: T / (unit_a * unit_b)
    t_acc = (t.float() / scale).to(torch.bfloat16)
    want = O.gemm_reference(da, db) + (t_acc.float().numpy().astype(np.float64) * scale @ u.float().numpy().astype(np.float64).T).astype(np.float32)
    got = run(qa, qb, lowrank=(t_acc.to(DEV), u.to(DEV)), out_dtype=torch.float32).cpu().numpy()
    assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)


# the projection shapes of the two decoder configurations (Qwen2-style 1.5B at rank 64, 7B at rank 128)
DECODER_SHAPES = [(1536, 1536, 64), (256, 1536, 64), (8960, 1536, 64), (1536, 8960, 64),
                  (3584, 3584, 128), (512, 3584, 128), (18944, 3584, 128), (3584, 18944, 128)]


@pytest.mark.parametrize("N,K,rank", DECODER_SHAPES)
def test_decoder_projection_shapes(N, K, rank):
    M = 384
    a = synthetic(M, K, "student", seed=N + K, dtype=torch.bfloat16)
    b = synthetic(N, K, "weights", seed=N + K + 1, dtype=torch.bfloat16)
    qa, qb = ops.nvfp4_quantize(a.to(DEV)), ops.nvfp4_quantize(b.to(DEV))
    g = torch.Generator().manual_seed(rank)
    t = (torch.randn(M, rank, generator=g) * 3).to(torch.bfloat16)
    u = (torch.randn(N, rank, generator=g) / rank ** 0.5).to(torch.bfloat16)
    scale = float(qa.unit.item()) * float(qb.unit.item())
    t_acc = (t.float() / scale).to(torch.bfloat16)
    got = run(qa, qb, lowrank=(t_acc.to(DEV), u.to(DEV)), out_dtype=torch.float32)
    # float64 product of what the kernel was given (dequantized on the device: the decoder itself is
    # pinned against the oracle by the quantizer tests)
    want = qa.dequantize(torch.float32).double() @ qb.dequantize(torch.float32).double().t() \
        + (t_acc.to(DEV).double() * scale) @ u.to(DEV).double().t()
    assert rel_l2(got.double().cpu().numpy(), want.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("single_cta", [False, True])
def test_more_tiles_than_sms_ragged_edges_and_rank(single_cta):
    # every persistent CTA (or CTA pair) walks several tiles, so accumulator hand-over, stage ring
    # and scale buffers wrap many times, with rank iterations between the tiles; _debug=8 forces
    # the single-CTA kernel where the dispatcher would take CTA pairs
    M, N, K, rank = 2344, 4872, 512, 64
    qa, qb, da, db = operands(M, N, K, seed=11)
    g = torch.Generator().manual_seed(3)
    t = (torch.randn(M, rank, generator=g) * 3).to(torch.bfloat16)
    u = (torch.randn(N, rank, generator=g) / rank ** 0.5).to(torch.bfloat16)
    scale = float(qa.unit.item()) * float(qb.unit.item())
    t_acc = (t.float() / scale).to(torch.bfloat16)
    want = O.gemm_reference(da, db) + ((t_acc.float().numpy() * scale) @ u.float().numpy().T)
    dbg = 8 if single_cta else 0
    got = run(qa, qb, lowrank=(t_acc.to(DEV), u.to(DEV)), out_dtype=torch.float32, _debug=dbg).cpu().numpy()
    assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)
    got16 = run(qa, qb, lowrank=(t_acc.to(DEV), u.to(DEV)), out_dtype=torch.bfloat16, _debug=dbg).float().cpu().numpy()
    assert rel_l2(got16, torch.from_numpy(want).to(torch.bfloat16).float().numpy()) <= TOL


@pytest.mark.parametrize("M,N,K", [(384, 512, 1024), (130, 264, 96), (1024, 1536, 4096)])
def test_single_cta_kernel_where_pairs_would_run(M, N, K):
    qa, qb, da, db = operands(M, N, K, seed=M + N + K)
    got = run(qa, qb, out_dtype=torch.float32, _debug=8).cpu().numpy()
    assert rel_l2(got, O.gemm_reference(da, db)) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(16, 1024, 4096), (100, 1160, 2304), (128, 4096, 1024)])
def test_decode_sized_products_split_their_k_loop(M, N, K):
    # one row block of A and few column tiles: the K loop is split over idle SMs (fp32 partial sums in
    # a scratch buffer, summed in a fixed order by a second kernel that also applies every epilogue term)
    assert cabi.lib().metis_nvfp4_gemm_workspace_bytes(M, N, K) > 0
    assert cabi.lib().metis_nvfp4_gemm_workspace_bytes(4096, N, K) == 0
    qa, qb, da, db = operands(M, N, K, seed=M + K)
    g = torch.Generator().manual_seed(M)
    rank = 64
    t = (torch.randn(M, rank, generator=g) * 3).to(torch.bfloat16)
    u = (torch.randn(N, rank, generator=g) / rank ** 0.5).to(torch.bfloat16)
    scale = float(qa.unit.item()) * float(qb.unit.item())
    t_acc = (t.float() / scale).to(torch.bfloat16)
    bias, cv, rv = torch.randn(N, generator=g), torch.randn(M, generator=g), torch.randn(N, generator=g)
    c = torch.randn(M, N, generator=g)
    want = (O.gemm_reference(da, db) + (t_acc.float().numpy() * scale) @ u.float().numpy().T) * 0.5 \
        + bias.numpy()[None, :] + np.outer(cv.numpy(), rv.numpy()) + c.numpy()
    kw = dict(lowrank=(t_acc.to(DEV), u.to(DEV)), rank1=[(None, bias.to(DEV)), (cv.to(DEV), rv.to(DEV))], alpha=0.5)
    got = run(qa, qb, c=c.to(DEV), out_dtype=torch.float32, **kw).cpu().numpy()
    assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)
    again = run(qa, qb, c=c.to(DEV), out_dtype=torch.float32, **kw).cpu().numpy()
    assert np.array_equal(got, again)                       # fixed summation order: bit-reproducible
    c16 = c.to(torch.bfloat16)
    got16 = run(qa, qb, c=c16.to(DEV), out_dtype=torch.bfloat16, **kw).float().cpu().numpy()
    want16 = want - c.numpy() + c16.float().numpy()
    assert rel_l2(got16, torch.from_numpy(want16.astype(np.float32)).to(torch.bfloat16).float().numpy()) <= TOL


def test_rank1_terms_bias_and_addend():
    M, N, K = 260, 392, 768
    qa, qb, da, db = operands(M, N, K, seed=77)
    g = torch.Generator().manual_seed(0)
    bias, rv1 = torch.randn(N, generator=g), torch.randn(N, generator=g)
    cv1 = torch.randn(M, generator=g)
    c = torch.randn(M, N, generator=g)
    want = O.gemm_reference(da, db) * 0.5 + bias.numpy()[None, :] + np.outer(cv1.numpy(), rv1.numpy()) + c.numpy()
    got = run(qa, qb, rank1=[(None, bias.to(DEV)), (cv1.to(DEV), rv1.to(DEV))], c=c.to(DEV), alpha=0.5,
              out_dtype=torch.float32).cpu().numpy()
    assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)
    c16 = c.to(torch.bfloat16)
    want16 = O.gemm_reference(da, db) + c16.float().numpy()
    got16 = run(qa, qb, c=c16.to(DEV), out_dtype=torch.bfloat16).float().cpu().numpy()
    assert rel_l2(got16, torch.from_numpy(want16).to(torch.bfloat16).float().numpy()) <= TOL


def test_mean_centred_operand_through_gemv_row_vector():
    # y = (Q(x - mu) + 1 mu^T) Wq^T  ==  Q Wq^T + 1 (mu Wq^T)
    M, N, K = 256, 256, 512
    x = synthetic(M, K, "student", seed=5, dtype=torch.bfloat16)
    w = synthetic(N, K, "weights", seed=6, dtype=torch.bfloat16)
    mu = ops.col_mean(x.to(DEV))
    qx = ops.nvfp4_quantize(x.to(DEV), mean=mu)
    qw = ops.nvfp4_quantize(w.to(DEV))
    got = run(qx, qw, rank1=[(None, ops.nvfp4_gemv(qw, mu))], out_dtype=torch.float32).cpu().numpy()
    xhat = O.quantize_dequantize(x.float().numpy(), col_mean=mu.cpu().numpy())
    want = O.gemm_reference(xhat, O.quantize_dequantize(w.float().numpy()))
    assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)


def test_backward_products_through_the_transposed_quantizer():
    # dX = D W (contract over N) and dW = D^T X (contract over tokens), operands re-quantized
    # along the contraction dimension; compared with the oracle on exactly those operands.
    M, N, K = 512, 384, 256
    x = synthetic(M, K, "normal", seed=1, dtype=torch.bfloat16)
    w = synthetic(N, K, "weights", seed=2, dtype=torch.bfloat16)
    d = synthetic(M, N, "normal", seed=3, dtype=torch.bfloat16)
    qd = ops.nvfp4_quantize(d.to(DEV))
    qwt = ops.nvfp4_quantize(w.to(DEV), transpose=True)            # [K, N]
    dx = run(qd, qwt, out_dtype=torch.float32).cpu().numpy()
    want = O.gemm_reference(O.quantize_dequantize(d.float().numpy()),
                            O.quantize_dequantize(np.ascontiguousarray(w.float().numpy().T)))
    assert rel_l2(dx, want) <= 1e-5
    qdt = ops.nvfp4_quantize(d.to(DEV), transpose=True)            # [N, M]
    qxt = ops.nvfp4_quantize(x.to(DEV), transpose=True)            # [K, M]
    dw = run(qdt, qxt, out_dtype=torch.float32).cpu().numpy()
    want = O.gemm_reference(O.quantize_dequantize(np.ascontiguousarray(d.float().numpy().T)),
                            O.quantize_dequantize(np.ascontiguousarray(x.float().numpy().T)))
    assert rel_l2(dw, want) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (512, 512, 512)])      # single CTA; CTA pairs
def test_a_wait_that_cannot_complete_reports_a_status_and_leaves_the_context_usable(M, N, K):
    # debug knob: the producer arms the first stage for bytes it never requests, so the consumer's
    # bounded wait runs out; the kernel must return with a status instead of spinning.
    qa, qb, da, db = operands(M, N, K, seed=9)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.nvfp4_gemm(qa, qb, status=status, out_dtype=torch.float32, _debug=1)
    torch.cuda.synchronize()
    assert status.item() in (1, 2, 3)
    got = run(qa, qb, out_dtype=torch.float32).cpu().numpy()      # the next launch is fine
    assert rel_l2(got, O.gemm_reference(da, db)) <= 1e-5


@pytest.mark.parametrize("s_dtype", [torch.bfloat16, torch.float32])
def test_lowrank_scale_equals_the_torch_expression_bit_for_bit(s_dtype):
    g = torch.Generator().manual_seed(2)
    yv = (torch.randn(1000, 72, generator=g) * 5).to(torch.bfloat16).to(DEV)
    s = (torch.rand(72, generator=g) + 0.25).to(s_dtype).to(DEV)
    ua = torch.tensor([3.1e-3], device=DEV)
    ub = torch.tensor([7.7e-5], device=DEV)
    want = ((yv * s.to(torch.bfloat16)).float() / (ua * ub)).to(torch.bfloat16)
    got = ops.lowrank_scale(yv, s, ua, ub)
    assert torch.equal(got, want)
    padded = torch.zeros(1000, 80, dtype=torch.bfloat16, device=DEV)      # row pitch larger than r
    padded[:, :72] = yv
    assert torch.equal(ops.lowrank_scale(padded[:, :72], s, ua, ub), want)
    with pytest.raises(TypeError):
        ops.lowrank_scale(yv.float(), s, ua, ub)


def test_argument_errors():
    qa, qb, _, _ = operands(128, 128, 256, seed=4)
    qr = ops.nvfp4_quantize(torch.zeros(128, 256, device=DEV), sf_layout=cabi.SF_ROWMAJOR)
    with pytest.raises(ValueError):
        ops.nvfp4_gemm(qa, qr)                 # row-major scales are not a GEMM operand
    qk = ops.nvfp4_quantize(torch.zeros(128, 128, device=DEV))
    with pytest.raises(ValueError):
        ops.nvfp4_gemm(qa, qk)                 # inner dimensions differ
