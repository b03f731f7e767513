"""The bf16 tensor-core products of the low-rank branch's backward against float64 on the same bf16
inputs: the generic panel product in all four operand storage orders (an operand stored with the
contraction in its rows is read as it lies, never transposed in memory), then the two entry points that
autograd's backward of `ulinear(torch.mul(s, y))` (bitlinear.py:752-757) maps onto.
Tolerance: fp32 accumulation of exact bf16 products, rel-L2 <= 1e-5 before the stated bf16 roundings."""
import pytest
import torch

from fp4_post_b200 import ops
from gpu_helpers import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def _randn(rows, cols, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(rows, cols, device=DEV, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("Mg,Ng,Kg", [(128, 64, 64), (128, 128, 256), (256, 128, 1024), (200, 32, 136), (384, 256, 4096),
                                      (1000, 96, 520), (4096, 128, 2048)])
def test_panel_product_in_every_storage_order(Mg, Ng, Kg, a_mn, b_mn):
    a = _randn(Mg, Kg, seed=Mg + Kg)
    b = _randn(Ng, Kg, seed=Ng + Kg + 1, scale=Kg ** -0.5)
    want = a.double() @ b.double().t()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops.bf16_panel_gemm(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b,
                              a_mn_major=a_mn, b_mn_major=b_mn, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert got.shape == (Mg, Ng)
    assert rel_l2(got.double().cpu().numpy(), want.cpu().numpy()) <= 1e-5


def test_panel_product_reads_strided_operands_as_they_lie():
    wide = _randn(512, 1024, seed=3)
    a = wide[:, 128:640]                       # [512, 512] view with row pitch 1024
    b = _randn(64, 512, seed=4)
    got = ops.bf16_panel_gemm(a, b)
    assert rel_l2(got.double().cpu().numpy(), (a.double() @ b.double().t()).cpu().numpy()) <= 1e-5
    got = ops.bf16_panel_gemm(a, b, a_mn_major=True)      # the same memory read as [Kg = 512, Mg = 512]
    assert rel_l2(got.double().cpu().numpy(), (a.double().t() @ b.double().t()).cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("M,N,r", [(256, 384, 32), (512, 1536, 64), (2048, 4096, 128), (1000, 520, 256), (16384, 4096, 128)])
@pytest.mark.parametrize("s_dtype", [torch.bfloat16, torch.float32])
def test_gradient_through_ulinear_and_the_scaling(M, N, r, s_dtype):
    g = _randn(M, N, seed=M + N)
    u = _randn(N, r, seed=N + r, scale=N ** -0.5)
    yv = _randn(M, r, seed=M + r + 7)
    s = (torch.rand(r, device=DEV, generator=torch.Generator(device=DEV).manual_seed(r)) + 0.5).to(s_dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    d_yv, ds = ops.lowrank_dts(g, u, yv, s, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    # the products in float64, then the roundings autograd's bf16 ops apply
    d_ts64 = g.double() @ u.double()
    d_ts = d_ts64.to(torch.bfloat16)
    want_dyv = (d_ts.float() * s.to(torch.bfloat16).float()).to(torch.bfloat16)
    # a sum that lands within fp32 summation error of a bf16 rounding boundary rounds the other way (a few
    # elements in 1e5): d_ts then differs by one ulp, d_yv by up to two
    diff = (d_yv.float() - want_dyv.float()).abs()
    assert bool((diff <= want_dyv.float().abs() * 2.0 ** -6 + 2e-5).all())       # sums that cancel to ~1e-4 keep the absolute error of their 4096 terms
    assert float((diff == 0).float().mean()) > 0.99
    want_ds = (d_ts.float() * yv.float()).to(torch.bfloat16).double().sum(dim=0)
    assert rel_l2(ds.double().cpu().numpy(), want_ds.cpu().numpy()) <= 2e-3
    # the weight gradient of ulinear: contraction over the tokens
    ts = (yv.float() * s.to(torch.bfloat16).float()).to(torch.bfloat16)
    for out_dtype in (torch.bfloat16, torch.float32):
        du = ops.lowrank_du(g, ts, out_dtype=out_dtype, status=status)
        want = g.double().t() @ ts.double()
        tol = 1e-5 if out_dtype == torch.float32 else 4e-3
        assert du.dtype == out_dtype and du.shape == (N, r)
        assert rel_l2(du.double().cpu().numpy(), want.cpu().numpy()) <= tol
    torch.cuda.synchronize()
    assert status.item() == 0


def test_bad_shapes_are_rejected_on_the_host():
    g, u, yv = _randn(64, 64, 1), _randn(64, 12, 2), _randn(64, 12, 3)
    with pytest.raises(ValueError):
        ops.lowrank_dts(g, u, yv, torch.ones(12, device=DEV))          # rank 12: not a multiple of 8
    with pytest.raises(ValueError):
        ops.bf16_panel_gemm(_randn(64, 64, 4), _randn(300, 64, 5))     # more than 256 columns
