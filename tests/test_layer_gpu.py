"""The Metis layer on the GPU through its public modules.

dense mode   native quantizer kernels + torch.matmul: the reference's wiring, checked against the
             vectors recorded from the reference's own BitLinear (forward and every gradient).
packed mode  real FP4 operands on the tcgen05 GEMM with the rank-r product fused; the forward is
             checked against dense mode, and every gradient against the same formulas evaluated in
             float64 on the dequantized operands the kernels actually consumed.
"""
import numpy as np
import pytest
import torch

import fp4_post_b200
from fp4_post_b200 import cabi, ops

fp4_post_b200.install_reference_aliases()

from Metis.Metis.bitlinear import BitLinear, LinearLowbit, LinearLowbitFunction, PackedOperand  # noqa: E402
from Metis.Metis.quant import (Cast2NVFp4e2m1Block, Cast2NVFp4e2m1BlockNOSR,  # noqa: E402
                               nvfp4_nosr_qdq_compile_status)
from grpo.grpo import MetisArgs, replace_linear_with_metis  # noqa: E402
from gpu_helpers import rel_l2  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
F = LinearLowbitFunction


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


CONFIG_KEYS = ("compute_dtype", "q_forward_input", "q_forward_weight", "q_backward_input", "q_backward_weight",
               "q_backward_outputgrad", "enable_activation_svd", "enable_backward_svd", "enable_nv_recipe",
               "activation_lowrank_svd", "backward_lowrank_svd", "metis_mode", "tp_simulate", "tp_parts", "gemm_mode",
               "activation_broadcast_dim", "backward_broadcast_dim", "activation_lowrank_niter", "backward_lowrank_niter")


@pytest.fixture(autouse=True)
def restore_configuration():
    saved = {k: getattr(F, k) for k in CONFIG_KEYS}
    yield
    for k, v in saved.items():
        setattr(F, k, v)
    BitLinear.rollout_merge_active = False


def metis_args(rank, backward_q="nvfp4e2m1bnosr", cache=False, gemm_mode="packed", **kw):
    a = MetisArgs(forward_svd_rank=rank, activation_lowrank_svd=rank, backward_lowrank_svd=rank,
                  cache_quantized_weight=cache, **kw)
    a.device = DEV
    a.q_backward_input = a.q_backward_weight = a.q_backward_outputgrad = backward_q
    a.gemm_mode = gemm_mode
    return a


def build_layer(g, args, dtype):
    """BitLinear with the golden factors (so both sides use the same U, s, V, R)."""
    N, K = g["W"].shape
    layer = BitLinear(K, N, args=args, bias=True, dtype=dtype, compute_dtype=dtype)
    with torch.no_grad():
        layer.warmup_linear.weight.copy_(torch.from_numpy(g["W"]))
        layer.warmup_linear.bias.copy_(torch.from_numpy(g["bias"]))
    layer.layer_name = "golden.layer"
    layer.split()
    with torch.no_grad():     # the exact factors of the record (SVD signs may differ between LAPACK builds)
        layer.vlinear.weight.copy_(torch.from_numpy(g["V"]))
        layer.ulinear.weight.copy_(torch.from_numpy(g["U"]))
        layer.s.copy_(torch.from_numpy(g["S"]))
        layer.warmup_linear.weight.copy_(torch.from_numpy(g["R"]))
    return layer.to(DEV)


def grads_of(layer, x):
    return dict(dx=x.grad, dR=layer.warmup_linear.weight.grad, dV=layer.vlinear.weight.grad,
                dU=layer.ulinear.weight.grad, ds=layer.s.grad, dbias=layer.warmup_linear.bias.grad)


def test_dense_mode_reproduces_the_reference_layer(layer_golden):
    g = layer_golden
    layer = build_layer(g, metis_args(int(g["rank"]), gemm_mode="dense"), torch.float32)
    x = torch.from_numpy(g["x"]).to(DEV).requires_grad_(True)
    y = layer(x)
    y.backward(torch.from_numpy(g["grad_out"]).to(DEV))
    assert rel_l2(y.detach().cpu().numpy(), g["y"]) <= 1e-3
    for name, got in grads_of(layer, x).items():
        err = rel_l2(got.cpu().numpy(), g[name])
        assert err <= 1e-3, f"{name}: rel-L2 {err}"     # the stated bar; a code flips only if a mean differs in its last bit


def test_packed_forward_matches_dense_forward(layer_golden):
    g = layer_golden
    x = torch.from_numpy(g["x"]).to(DEV)
    outs = {}
    for mode in ("dense", "packed"):
        layer = build_layer(g, metis_args(int(g["rank"]), gemm_mode=mode), torch.float32)
        with torch.no_grad():
            outs[mode] = layer(x).cpu().numpy()
    assert rel_l2(outs["packed"], outs["dense"]) <= 1e-4
    assert rel_l2(outs["packed"], g["y"]) <= 1e-3          # and so the reference's forward


def _f64(t):
    return t.detach().double().cpu()


def _value(q, add_mean=True):
    """float64 matrix an NVFP4Tensor stands for (dequantized by the library, bit-exact elsewhere)."""
    v = _f64(ops.nvfp4_dequantize(q, torch.float32, add_mean=False))
    if add_mean and q.row_vec is not None:
        v = v + _f64(q.row_vec)[None, :]
    if add_mean and q.col_vec is not None:
        v = v + _f64(q.col_vec)[:, None]
    return v


@pytest.mark.parametrize("backward_q", ["nvfp4e2m1bnosr", "nvfp4e2m1b"])
def test_packed_backward_equals_the_chain_rule_on_the_operands_it_consumed(backward_q):
    torch.manual_seed(0)
    B, T, K, N, r = 2, 128, 256, 192, 32
    args = metis_args(r, backward_q=backward_q)
    layer = BitLinear(K, N, args=args, bias=True, dtype=torch.float32, compute_dtype=torch.float32)
    with torch.no_grad():
        layer.warmup_linear.weight.mul_(3.0)
    layer.layer_name = "t"
    layer.split()
    layer = layer.to(DEV)
    x = (torch.randn(B, T, K) + torch.randn(1, 1, K)).to(DEV).requires_grad_(True)
    gout = torch.randn(B, T, N, device=DEV)

    recorded = []
    real = F._pack_centred

    def spy(tensor, quantizer, centred, mean_cache=None, cache_key="default", **kw):
        op = real(tensor, quantizer, centred, mean_cache, cache_key, **kw)
        recorded.append(op)
        return op

    F._pack_centred = staticmethod(spy)
    try:
        y = layer(x)
        assert isinstance(y.grad_fn, torch.autograd.function.BackwardCFunction) and "MetisFused" in type(y.grad_fn).__name__
        y.backward(gout)
    finally:
        F._pack_centred = staticmethod(real)
    assert len(recorded) == 3
    # activation, then (in either order) grad of vlinear's output [M, r] and grad of the residual's output [M, N]
    xa = recorded[0]
    dv, dg = sorted(recorded[1:], key=lambda op: op.q.shape[1])
    assert dv.q.shape[1] == r and dg.q.shape[1] == N

    M = B * T
    U, s = _f64(layer.ulinear.weight), _f64(layer.s)
    g2 = _f64(gout).reshape(M, N)
    xh = _value(xa.q)
    # forward as the kernels saw it; weights: re-quantize (round to nearest is deterministic)
    Vq = _value(ops.nvfp4_quantize(layer.vlinear.weight.detach()))
    Rq = _value(ops.nvfp4_quantize(layer.warmup_linear.weight.detach()))
    yv = xh @ Vq.T
    y_want = (yv * s) @ U.T + xh @ Rq.T + _f64(layer.warmup_linear.bias)
    assert rel_l2(_f64(y).reshape(M, N).numpy(), y_want.numpy()) <= 1e-4

    # backward: transposed quantizations actually used (cached on the operands)
    Vt = _value(ops.nvfp4_quantize(layer.vlinear.weight.detach(), transpose=True))        # [K, r]
    Rt = _value(ops.nvfp4_quantize(layer.warmup_linear.weight.detach(), transpose=True))  # [K, N]
    x_t = _value(xa.transposed())                                                         # [K, M] = x^^T
    want = {}
    want["dbias"] = g2.sum(0)
    want["dU"] = g2.T @ (yv * s)
    d_ts = g2 @ U
    want["ds"] = (d_ts * yv).sum(0)
    want["dR"] = _value(dg.transposed()) @ x_t.T
    want["dV"] = _value(dv.transposed()) @ x_t.T
    want["dx"] = (_value(dg.q) @ Rt.T + _value(dv.q) @ Vt.T).reshape(B, T, K)
    got = grads_of(layer, x)
    for name in ("dbias", "dU", "ds", "dR", "dV", "dx"):
        err = rel_l2(_f64(got[name]).numpy(), want[name].numpy())
        assert err <= 1e-3, f"{name}: rel-L2 {err}"
    # the quantized gradient operands really are the centred gradients
    d_yv = d_ts * s
    assert rel_l2(_value(dv.q).numpy(), d_yv.numpy()) < 0.2
    assert rel_l2(_value(dg.q).numpy(), g2.numpy()) < 0.2


def test_packed_gradients_agree_with_dense_gradients_up_to_quantization_noise(layer_golden):
    g = layer_golden
    res = {}
    for mode in ("dense", "packed"):
        layer = build_layer(g, metis_args(int(g["rank"]), gemm_mode=mode), torch.float32)
        x = torch.from_numpy(g["x"]).to(DEV).requires_grad_(True)
        layer(x).backward(torch.from_numpy(g["grad_out"]).to(DEV))
        res[mode] = {k: v.cpu().numpy() for k, v in grads_of(layer, x).items()}
    for name in ("dU", "ds", "dbias"):          # not quantized in either mode
        assert rel_l2(res["packed"][name], res["dense"][name]) <= 1e-3, name
    for name in ("dx", "dR", "dV"):             # same expectation, different quantization blocks
        assert rel_l2(res["packed"][name], res["dense"][name]) <= 0.25, name


def test_bf16_input_gradient_fused_into_one_launch_matches_two_launches():
    from Metis.Metis.bitlinear import MetisFusedFunction
    torch.manual_seed(5)
    args = metis_args(64, cache=True)                     # round to nearest everywhere: deterministic
    layer = BitLinear(512, 384, args=args, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "f"
    layer.split()
    layer = layer.to(DEV)
    x = torch.randn(2, 256, 512, device=DEV, dtype=torch.bfloat16)
    gout = torch.randn(2, 256, 384, device=DEV, dtype=torch.bfloat16)
    grads = {}
    for fused in (True, False):
        MetisFusedFunction.fuse_dx_side_product = fused
        try:
            xin = x.clone().requires_grad_(True)
            layer(xin).backward(gout)
            grads[fused] = xin.grad.float().cpu().numpy()
        finally:
            MetisFusedFunction.fuse_dx_side_product = True
    # both round the low-rank branch's contribution to bf16 once, at different points
    assert rel_l2(grads[True], grads[False]) <= 1e-2


def test_native_backward_of_the_unquantized_branch_matches_torch_matmul():
    # dU, ds and d_yv from the tensor-core panel products against the same step with torch.matmul for
    # the U branch; round to nearest everywhere, so that everything downstream of d_yv is deterministic
    from Metis.Metis.bitlinear import MetisFusedFunction
    torch.manual_seed(7)
    args = metis_args(64, cache=True)
    layer = BitLinear(1024, 768, args=args, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "ubranch"
    layer.split()
    layer = layer.to(DEV)
    x = torch.randn(2, 512, 1024, device=DEV, dtype=torch.bfloat16)
    gout = torch.randn(2, 512, 768, device=DEV, dtype=torch.bfloat16)
    res = {}
    for native in (True, False):
        MetisFusedFunction.native_lowrank_backward = native
        try:
            xin = x.clone().requires_grad_(True)
            for p in layer.parameters():
                p.grad = None
            layer(xin).backward(gout)
            res[native] = {k: v.float().cpu().numpy() for k, v in dict(
                dx=xin.grad, dR=layer.warmup_linear.weight.grad, dV=layer.vlinear.weight.grad,
                dU=layer.ulinear.weight.grad, ds=layer.s.grad).items()}
        finally:
            MetisFusedFunction.native_lowrank_backward = True
    # same bf16 inputs, fp32 accumulation on both sides: only summation order and a rare last-bit flip differ
    assert rel_l2(res[True]["dU"], res[False]["dU"]) <= 4e-3
    assert rel_l2(res[True]["ds"], res[False]["ds"]) <= 1e-2
    for name in ("dx", "dR"):
        assert rel_l2(res[True][name], res[False][name]) <= 1e-2, name
    assert rel_l2(res[True]["dV"], res[False]["dV"]) <= 5e-2       # d_yv is re-quantized: a flipped bf16 bit may move a code


def test_second_stream_gives_the_gradients_of_the_single_stream_order_bit_for_bit():
    # round to nearest everywhere, cached weights (so that the forward overlaps too): a missing
    # dependency between the two streams would show as a difference
    from Metis.Metis.bitlinear import MetisFusedFunction
    torch.manual_seed(11)
    args = metis_args(64, cache=True)
    layer = BitLinear(1024, 768, args=args, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "streams"
    layer.split()
    layer = layer.to(DEV)
    x = torch.randn(4, 512, 1024, device=DEV, dtype=torch.bfloat16)
    gout = torch.randn(4, 512, 768, device=DEV, dtype=torch.bfloat16)
    results = {}
    for concurrent in (True, False, True):
        MetisFusedFunction.concurrent_branches = concurrent
        try:
            for rep in range(3):                                  # repeat: a race need not show the first time
                xin = x.clone().requires_grad_(True)
                for p in layer.parameters():
                    p.grad = None
                y = layer(xin)
                y.backward(gout)
                got = [y.detach().clone(), xin.grad.clone()] + [p.grad.clone() for p in layer.parameters()]
                key = results.setdefault("ref", got)
                for a, b in zip(got, key):
                    assert torch.equal(a, b), f"concurrent={concurrent}, repetition {rep}"
        finally:
            MetisFusedFunction.concurrent_branches = True


def test_grpo_defaults_bf16_stochastic_backward_and_shared_activation():
    torch.manual_seed(1)
    block = torch.nn.Module()
    block.q_proj = torch.nn.Linear(512, 512, bias=True)
    block.k_proj = torch.nn.Linear(512, 128, bias=True)
    block.o_proj = torch.nn.Linear(512, 512, bias=False)
    model = torch.nn.Sequential(block).to(DEV).to(torch.bfloat16)
    args = MetisArgs(forward_svd_rank=64, cache_quantized_weight=True)
    args.device = DEV
    replace_linear_with_metis(model, dtype=torch.bfloat16, metis_args=args, compute_dtype=torch.bfloat16)
    blk = model[0]
    assert F.q_backward_outputgrad is Cast2NVFp4e2m1Block and F.q_forward_input is Cast2NVFp4e2m1BlockNOSR

    calls = {"n": 0}
    real = Cast2NVFp4e2m1BlockNOSR.quantize_packed.__func__
    real_dual = Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual.__func__

    def counting(cls, x, **kw):
        calls["n"] += 1
        return real(cls, x, **kw)

    def counting_dual(cls, x, **kw):             # autograd is recording: row-major and transposed from one pass
        calls["n"] += 1
        return real_dual(cls, x, **kw)

    Cast2NVFp4e2m1BlockNOSR.quantize_packed = classmethod(counting)
    Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual = classmethod(counting_dual)
    try:
        x = torch.randn(4, 64, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        q, k = blk.q_proj(x), blk.k_proj(x)
        # one activation quantization for the group + V and R of each projection
        assert calls["n"] == 1 + 4
        o = blk.o_proj(q)
        assert q.dtype == torch.bfloat16 and q.shape == (4, 64, 512) and k.shape == (4, 64, 128)
        (o.float().pow(2).mean() + k.float().mean()).backward()
        before = calls["n"]
        blk.q_proj(x); blk.k_proj(x)              # same x object and unchanged weights: everything cached
        assert calls["n"] == before
        with torch.no_grad():
            blk.q_proj.warmup_linear.weight.add_(0.01)
        blk.q_proj(x)
        assert calls["n"] == before + 1           # only the changed weight
    finally:
        Cast2NVFp4e2m1BlockNOSR.quantize_packed = classmethod(real)
        Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual = classmethod(real_dual)
    for name, p in model.named_parameters():
        assert p.grad is not None and p.grad.dtype == torch.bfloat16 and torch.isfinite(p.grad).all(), name
    assert x.grad is not None and torch.isfinite(x.grad).all()
    # against plain bf16 linears with the same merged weights the loss gradient points the same way
    w = blk.q_proj
    merged = (w.ulinear.weight.float() * w.s.float()) @ w.vlinear.weight.float() + w.warmup_linear.weight.float()
    y_ref = torch.nn.functional.linear(x.detach().float(), merged, w.warmup_linear.bias.float())
    with torch.no_grad():
        y = w(x.detach()).float()
    assert rel_l2(y.cpu().numpy(), y_ref.detach().cpu().numpy()) < 0.2


def test_decode_keeps_a_running_mean_and_rollout_uses_the_fp4_weights():
    torch.manual_seed(2)
    args = metis_args(32, cache=True)
    layer = BitLinear(256, 256, args=args, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "dec"
    layer.split()
    layer = layer.to(DEV)
    prefill = torch.randn(4, 16, 256, device=DEV, dtype=torch.bfloat16)
    step = torch.randn(4, 1, 256, device=DEV, dtype=torch.bfloat16)
    BitLinear.rollout_merge_active = True
    with torch.no_grad():
        layer(prefill)
        me0, n0 = layer.mean_cache["dec.shared"]
        assert n0 == 64
        y = layer(step)
        me1, n1 = layer.mean_cache["dec.shared"]
    assert n1 == 68 and y.shape == (4, 1, 256)
    want = (me0.float() * 64 + step.float().reshape(-1, 256).mean(0) * 4) / 68
    assert me1.dtype == torch.float32       # the cache entry is the kernel's fp32 mean, not a bf16 copy
    assert torch.allclose(me1.reshape(-1), want.reshape(-1), rtol=1e-6, atol=1e-6)
    # same answer as the dense merged-weight path of the reference, up to bf16 rounding
    F.gemm_mode = "dense"
    layer.mean_cache.clear()
    with torch.no_grad():
        layer(prefill)
        y_dense = layer(step)
    assert rel_l2(y.float().cpu().numpy(), y_dense.float().cpu().numpy()) < 2e-2


def test_three_call_protocol_equals_the_fused_kernel():
    x = torch.randn(4, 32, device=DEV)
    Q = Cast2NVFp4e2m1BlockNOSR
    s = Q.get_scalar(x)
    expected = Q.rquant(Q.quant(x, s), s)
    torch.testing.assert_close(Q.quantize_dequantize(x), expected, rtol=0, atol=0)


def test_compile_flag_validates_the_native_kernel_against_the_eager_graph():
    x = torch.randn(8, 16, 128, device=DEV, dtype=torch.bfloat16)
    Q = Cast2NVFp4e2m1BlockNOSR
    Q.compile_quantize_dequantize = False
    expected = Q.quantize_dequantize(x)
    Q.compile_quantize_dequantize = True
    try:
        actual = Q.quantize_dequantize(x)
    finally:
        Q.compile_quantize_dequantize = False
    torch.testing.assert_close(actual, expected, rtol=0, atol=0)
    assert nvfp4_nosr_qdq_compile_status() == "validated"


def test_rmsnorm_module_feeds_a_projection_group_without_requantizing():
    from Metis.models.llama import RMSNorm
    torch.manual_seed(3)
    args = metis_args(32, cache=True, enable_activation_svd=False)
    group = {"name": "blk.qkv", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    proj = BitLinear(512, 256, args=args, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    proj.layer_name, proj.activation_group = "blk.q_proj", group
    proj.split()
    proj = proj.to(DEV)
    norm = RMSNorm(512).to(DEV).to(torch.bfloat16)
    x = torch.randn(2, 64, 512, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        want_norm = norm(x)
        packed, y = norm.forward_quantized(x, return_norm=True, activation_group=group)
        assert isinstance(packed, PackedOperand) and group["input_ref"]() is y
        assert (y.float() - want_norm.float()).abs().max() <= want_norm.float().abs().max() * 2 ** -7
        fused = proj(y)                      # picks the registered operand up by identity
        plain = proj(y.clone())              # quantizes the same values itself
    assert torch.equal(fused, plain)


def test_rmsnorm_module_in_mean_mode_is_trainable_and_matches_the_unfused_chain():
    # GRPO defaults: mean-centred activations, stochastic backward replaced by round to nearest here so that the
    # two chains can be compared; the fused entry must give what norm -> BitLinear gives, with gradients
    from Metis.models.llama import RMSNorm
    torch.manual_seed(4)
    args = metis_args(32, cache=True)                      # enable_activation_svd=True, metis_mode="mean"
    group = {"name": "blk.qkv", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    proj = BitLinear(512, 256, args=args, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    proj.layer_name, proj.activation_group = "blk.q_proj", group
    proj.split()
    proj = proj.to(DEV)
    norm = RMSNorm(512).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.1 * torch.randn(512, device=DEV))
    x = (torch.randn(2, 64, 512, device=DEV) + torch.randn(1, 1, 512, device=DEV)).to(torch.bfloat16)
    gout = torch.randn(2, 64, 256, device=DEV, dtype=torch.bfloat16)
    res = {}
    for fused in (True, False):
        xin = x.clone().requires_grad_(True)
        for p in list(proj.parameters()) + [norm.weight]:
            p.grad = None
        if fused:
            packed, y = norm.forward_quantized(xin, return_norm=True, activation_group=group)
            assert isinstance(packed, PackedOperand) and packed.mean is not None and packed._qt is not None
            assert group["input_ref"]() is y and "blk.qkv.shared" in group["mean_cache"]
        else:
            group["input_ref"] = group["quantized_input"] = None
            y = norm(xin)
        out = proj(y)
        out.backward(gout)
        res[fused] = dict(y=out.detach().float().cpu().numpy(), dx=xin.grad.float().cpu().numpy(),
                          dgamma=norm.weight.grad.float().cpu().numpy(), dR=proj.warmup_linear.weight.grad.float().cpu().numpy())
    # same normalised values up to a last bf16 bit, same quantizer: outputs and gradients agree closely
    assert rel_l2(res[True]["y"], res[False]["y"]) <= 2e-2
    assert rel_l2(res[True]["dR"], res[False]["dR"]) <= 5e-2
    assert rel_l2(res[True]["dx"], res[False]["dx"]) <= 5e-2
    assert rel_l2(res[True]["dgamma"], res[False]["dgamma"]) <= 5e-2


def test_rmsnorm_module_keeps_the_rolling_decode_mean_of_its_group():
    from Metis.models.llama import RMSNorm
    torch.manual_seed(6)
    metis_args(32, cache=True)                             # configures the class attributes (mean mode)
    F.enable_activation_svd, F.metis_mode, F.compute_dtype = True, "mean", torch.bfloat16
    F.q_forward_input = Cast2NVFp4e2m1BlockNOSR
    group = {"name": "g", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    norm = RMSNorm(256).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        p0, y0 = norm.forward_quantized(torch.randn(4, 16, 256, device=DEV, dtype=torch.bfloat16), return_norm=True, activation_group=group)
        me0, n0 = group["mean_cache"]["g.shared"]
        p1, y1 = norm.forward_quantized(torch.randn(4, 1, 256, device=DEV, dtype=torch.bfloat16), return_norm=True, activation_group=group)
        me1, n1 = group["mean_cache"]["g.shared"]
    assert n0 == 64 and n1 == 68
    want = (me0.float() * 64 + y1.float().reshape(-1, 256).mean(0) * 4) / 68
    assert torch.allclose(me1.reshape(-1), want.reshape(-1), rtol=1e-5, atol=1e-6)
    assert torch.allclose(p1.mean.reshape(-1), me1.reshape(-1))


def test_packed_gradients_average_towards_the_dense_gradients_over_stochastic_draws(layer_golden):
    # The packed backward quantizes W, D and x once more along the contraction dimension; D with stochastic
    # rounding.  Its gradients are noisy versions of the dense (reference-wiring) ones: they point the same
    # way, and the noise of the stochastic part averages out over draws.
    g = layer_golden
    x0 = torch.from_numpy(g["x"]).to(DEV)
    gout = torch.from_numpy(g["grad_out"]).to(DEV)

    def grads(mode, backward_q):
        layer = build_layer(g, metis_args(int(g["rank"]), backward_q=backward_q, gemm_mode=mode), torch.float32)
        x = x0.clone().requires_grad_(True)
        layer(x).backward(gout)
        return {k: v.double().cpu() for k, v in grads_of(layer, x).items()}

    dense = grads("dense", "nvfp4e2m1bnosr")                         # deterministic reference wiring
    draws = [grads("packed", "nvfp4e2m1b") for _ in range(24)]       # the device-side Philox counter moves on every call
    for name in ("dx", "dR", "dV"):
        single = draws[0][name]
        mean = torch.stack([d[name] for d in draws]).mean(0)
        cos = torch.nn.functional.cosine_similarity(single.flatten(), dense[name].flatten(), dim=0).item()
        e1 = (single - dense[name]).norm().item() / dense[name].norm().item()
        em = (mean - dense[name]).norm().item() / dense[name].norm().item()
        print(f"{name}: cosine {cos:.4f}, rel-L2 of one draw {e1:.3f}, of the mean of 24 draws {em:.3f}")
        # measured on B200: cosine 0.97-0.98; rel-L2 0.19-0.25 for one draw, 0.14-0.20 for the mean of 24 (what is
        # left is the deterministic re-quantization of x and W along the other dimension)
        assert cos > 0.95, name
        assert em < 0.92 * e1, name                                  # the stochastic part of the error shrinks
        assert not torch.equal(draws[0][name], draws[1][name])       # fresh bits every call


def test_wgrad_rotation_keeps_the_weight_gradients_and_leaves_everything_else_alone():
    # packed_wgrad_rht rotates both operands of dR and dV along the tokens (the NVIDIA baseline's Wgrad recipe):
    # same gradients up to quantization noise, identical forward, dx, dU, ds
    torch.manual_seed(9)
    args = metis_args(32, cache=True)
    layer = BitLinear(512, 384, args=args, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "rht"
    layer.split()
    layer = layer.to(DEV)
    x = (torch.randn(2, 256, 512, device=DEV) + 0.5 * torch.randn(1, 1, 512, device=DEV)).to(torch.bfloat16)
    x[..., 7] *= 30                                            # an outlier channel: what the rotation is for
    gout = torch.randn(2, 256, 384, device=DEV, dtype=torch.bfloat16)
    res = {}
    for rht in (False, True):
        F.packed_wgrad_rht = rht
        try:
            xin = x.clone().requires_grad_(True)
            for p in layer.parameters():
                p.grad = None
            y = layer(xin)
            y.backward(gout)
            res[rht] = dict(y=y.detach().clone(), **{k: v.clone() for k, v in grads_of(layer, xin).items()})
        finally:
            F.packed_wgrad_rht = False
    for name in ("y", "dx", "dU", "ds", "dbias"):
        assert torch.equal(res[True][name], res[False][name]), name
    # float64 weight gradients of the unquantized chain as the yardstick
    g2, x2 = gout.double().reshape(-1, 384), x.double().reshape(-1, 512)
    exact_dR = g2.t() @ x2
    for name in ("dR", "dV"):
        a, b = res[True][name].double(), res[False][name].double()
        assert not torch.equal(a, b)
        assert (a - b).norm() / b.norm() < 0.3, name
    e_plain = (res[False]["dR"].double() - exact_dR).norm() / exact_dR.norm()
    e_rot = (res[True]["dR"].double() - exact_dR).norm() / exact_dR.norm()
    assert e_rot < e_plain * 1.1


def test_deferred_scale_passes_leave_every_result_bit_for_bit():
    """The scale pass of the orientation an operand's first consumer does not need runs on a third stream:
    forward output and all gradients equal those of the undeferred order exactly (round to nearest everywhere)."""
    torch.manual_seed(11)
    dev = torch.device(DEV)
    results = {}
    for defer in (True, False):
        torch.manual_seed(11)
        margs = MetisArgs(forward_svd_rank=32, activation_lowrank_svd=32, backward_lowrank_svd=32)
        margs.device = dev
        margs.q_backward_input = margs.q_backward_weight = margs.q_backward_outputgrad = "nvfp4e2m1bnosr"
        layer = BitLinear(512, 384, args=margs, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
        layer.layer_name = "defer"
        layer.split()
        LinearLowbitFunction.defer_scale_pass = defer
        try:
            x = (torch.randn(2, 256, 512, device=dev) + 0.25).to(torch.bfloat16).requires_grad_(True)
            g = torch.randn(2, 256, 384, device=dev).to(torch.bfloat16)
            y = layer(x)
            y.backward(g)
            torch.cuda.synchronize()
        finally:
            LinearLowbitFunction.defer_scale_pass = True
        results[defer] = [y.detach().clone(), x.grad.clone()] + [p.grad.clone() for p in layer.parameters() if p.grad is not None]
    assert len(results[True]) == len(results[False]) >= 6
    for a, b in zip(results[True], results[False]):
        assert torch.equal(a, b)


def test_svd_activation_mode_runs_on_the_native_quantizers():
    """metis_mode "svd" (bitlinear.py:243-309): x^ = Q(U) diag(s) Q(V) + Q(x - that), with the randomized SVD
    from torch and every quantization on this library's kernels; the products stay dense (the reference's
    wiring).  The factors come from random projections, so the check is what the mode is for: on an input
    with a strong low-rank part the reconstruction beats plain quantization, and a layer trains in it."""
    torch.manual_seed(5)
    M, K, r = 512, 256, 16
    low = torch.randn(M, r, device=DEV) @ torch.randn(r, K, device=DEV) * 4.0
    x = (low + torch.randn(M, K, device=DEV) * 0.5).reshape(2, M // 2, K)
    plain = Cast2NVFp4e2m1BlockNOSR.quantize_dequantize(x)
    mixed = F.svd_quant(x, quant_func=Cast2NVFp4e2m1BlockNOSR, rank=r, niter=2, metis_mode="svd")
    assert mixed.shape == x.shape and mixed.is_cuda
    err_plain, err_mixed = rel_l2(plain.cpu().numpy(), x.cpu().numpy()), rel_l2(mixed.cpu().numpy(), x.cpu().numpy())
    assert err_mixed < 0.6 * err_plain, (err_mixed, err_plain)

    args = metis_args(16, metis_mode="svd")
    layer = BitLinear(K, 192, args=args, bias=True, dtype=torch.float32, compute_dtype=torch.float32).to(DEV)
    layer.layer_name = "svd.layer"
    layer.split()
    xin = x.clone().requires_grad_(True)
    y = layer(xin)
    y.backward(torch.randn_like(y))
    want = xin.detach().reshape(-1, K) @ (layer.ulinear.weight @ torch.diag(layer.s) @ layer.vlinear.weight + layer.warmup_linear.weight).T \
        + layer.warmup_linear.bias
    assert rel_l2(y.detach().reshape(-1, 192).cpu().numpy(), want.detach().cpu().numpy()) < 0.15
    assert xin.grad is not None and torch.isfinite(xin.grad).all()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())
