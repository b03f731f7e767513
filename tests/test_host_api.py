"""Host-side contracts of the Metis modules, the ones the reference pins in its own
tests/test_metis_quant_cache.py: caches, activation sharing, RHT algebra, replacement without
split.  They run on the CPU with stub quantizer classes, exactly as the reference's do; the
NVFP4 classes themselves need a GPU and are covered by the gpu-marked tests."""
from types import SimpleNamespace

import pytest
import torch

import fp4_post_b200

fp4_post_b200.install_reference_aliases()

from Metis.Metis.bitlinear import BitLinear, LinearLowbit, LinearLowbitFunction  # noqa: E402
from Metis.Metis.quant import Cast2Fp32, Cast2NVFp4e2m1BlockNOSR, quant_func, nvfp4_nosr_qdq_compile_status  # noqa: E402
from grpo.grpo import MetisArgs, replace_linear_with_metis  # noqa: E402

F = LinearLowbitFunction


def counting_quantizer(returns_copy=False, forbid_get_scalar=False):
    class Counting(Cast2Fp32):
        calls = 0

        @classmethod
        def quantize_dequantize(cls, value):
            cls.calls += 1
            return value.detach().clone() if returns_copy else value

    if forbid_get_scalar:
        def boom(cls, value):
            raise AssertionError("mean activation path must use fused QDQ")
        Counting.get_scalar = classmethod(boom)
    return Counting


@pytest.fixture(autouse=True)
def plain_configuration():
    """Identity quantizers, fp32, no decomposition; each test changes what it needs."""
    saved = {k: getattr(F, k) for k in ("compute_dtype", "q_forward_input", "q_forward_weight", "q_backward_input",
                                        "q_backward_weight", "q_backward_outputgrad", "enable_activation_svd",
                                        "enable_backward_svd", "enable_nv_recipe", "activation_lowrank_svd",
                                        "backward_lowrank_svd", "metis_mode", "tp_simulate", "tp_parts",
                                        "hadamard_workspace_mb", "hadamard_backend", "hadamard_tile_size",
                                        "activation_broadcast_dim", "activation_lowrank_niter", "gemm_mode")}
    F.compute_dtype = torch.float32
    for k in ("q_forward_input", "q_forward_weight", "q_backward_input", "q_backward_weight", "q_backward_outputgrad"):
        setattr(F, k, Cast2Fp32)
    F.enable_activation_svd = F.enable_backward_svd = F.enable_nv_recipe = False
    F.tp_simulate, F.tp_parts, F.metis_mode = False, 1, "mean"
    yield
    for k, v in saved.items():
        setattr(F, k, v)
    BitLinear.rollout_merge_active = False


def svd_layer(name="test.layer", group=None, bias=False, cache=False, k=16, n=8, r=4):
    """A split BitLinear put together by hand, as the reference's tests do (no SVD needed)."""
    args = SimpleNamespace(device="cpu", cache_quantized_weight=cache, forward_svd_rank=r)
    layer = BitLinear.__new__(BitLinear)
    torch.nn.Module.__init__(layer)
    layer.args = args
    layer.is_svd_quant = True
    layer.mean_cache = {}
    layer.activation_group = group
    layer._merged_rollout_weight_cache = None
    layer.layer_name = name
    layer.vlinear = LinearLowbit(k, r, bias=False, args=args)
    layer.ulinear = torch.nn.Linear(r, n, bias=False)
    layer.warmup_linear = LinearLowbit(k, n, bias=bias, args=args)
    layer.s = torch.nn.Parameter(torch.ones(r))
    return layer


def mean_mode(rank=4):
    F.enable_activation_svd = True
    F.activation_lowrank_svd = rank
    F.activation_lowrank_niter = 0
    F.activation_broadcast_dim = -1
    F.metis_mode = "mean"


def test_registry_has_the_reference_keys_and_protocol():
    assert sorted(quant_func) == sorted(["fp4e2m1", "nvfp4e2m1b", "mxfp4e2m1b", "mxfp4e2m1bnosr", "nvfp4e2m1bnosr",
                                         "fp6e3m2", "fp6e3m2b", "fp8e4m3", "fp8e4m3b", "fp32", "1p58bit"])
    for cls in quant_func.values():
        for method in ("get_scalar", "quant", "rquant", "quantize_dequantize"):
            assert callable(getattr(cls, method))
    assert nvfp4_nosr_qdq_compile_status() in ("validated", "not validated") or nvfp4_nosr_qdq_compile_status().startswith("disabled")


def test_nvfp4_classes_refuse_cpu_tensors_and_bad_shapes():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        Cast2NVFp4e2m1BlockNOSR.quantize_dequantize(torch.randn(4, 32))
    with pytest.raises(ValueError, match="does not divide"):
        Cast2NVFp4e2m1BlockNOSR.quantize_dequantize(torch.randn(4, 24))


@pytest.mark.parametrize("key", ["fp4e2m1", "mxfp4e2m1bnosr", "fp6e3m2", "fp6e3m2b", "fp8e4m3", "fp8e4m3b", "fp32"])
def test_pure_torch_formats_round_trip_on_cpu(key):
    torch.manual_seed(0)
    x = torch.randn(8, 64)
    y = quant_func[key].quantize_dequantize(x.clone())
    assert y.shape == x.shape and torch.isfinite(y).all()
    # a quantizer may lose precision but not the signal
    assert torch.nn.functional.cosine_similarity(x.flatten(), y.flatten(), dim=0) > 0.9


def test_weight_cache_is_reused_until_the_parameter_changes():
    Q = counting_quantizer(returns_copy=True)
    F.q_forward_weight = Q
    layer = LinearLowbit(16, 8, bias=False, args=SimpleNamespace(device="cpu", cache_quantized_weight=True))
    x = torch.randn(2, 3, 16, requires_grad=True)
    layer(x).sum().backward()
    assert layer.weight.grad is not None
    layer(x.detach())
    assert Q.calls == 1                       # forward, backward, forward: quantized once
    with torch.no_grad():
        layer.weight.add_(0.1)                # bumps Parameter._version
    layer(x.detach())
    assert Q.calls == 2
    layer.to(torch.float32)                   # any _apply drops the entry
    assert layer._quantized_weight_cache is None


def test_without_the_flag_the_weight_is_quantized_every_call():
    Q = counting_quantizer(returns_copy=True)
    F.q_forward_weight = Q
    layer = LinearLowbit(16, 8, bias=True, args=SimpleNamespace(device="cpu"))
    layer(torch.randn(1, 2, 16)); layer(torch.randn(1, 2, 16))
    assert Q.calls == 2


def test_mean_mode_calls_the_fused_qdq_once_and_keeps_the_mean():
    Q = counting_quantizer(forbid_get_scalar=True)
    x = torch.randn(2, 3, 16)
    cache = {}
    out = F.svd_quant(x, quant_func=Q, metis_mode="mean", mean_cache=cache, cache_key="k")
    assert out.shape == x.shape and Q.calls == 1
    me, count = cache["k"]
    assert count == 6 and torch.allclose(me, x.reshape(-1, 16).mean(0, keepdim=True))
    torch.testing.assert_close(out, x)        # identity quantizer: mean + (x - mean)


def test_decode_updates_a_count_weighted_running_mean():
    Q = counting_quantizer()
    cache = {}
    prefill = torch.randn(2, 5, 16)
    F.svd_quant(prefill, quant_func=Q, metis_mode="mean", mean_cache=cache, cache_key="k")
    step = torch.randn(2, 1, 16)              # one token per sequence
    F.svd_quant(step, quant_func=Q, metis_mode="mean", mean_cache=cache, cache_key="k")
    me, count = cache["k"]
    want = (prefill.reshape(-1, 16).sum(0) + step.reshape(-1, 16).sum(0)) / 12
    assert count == 12 and torch.allclose(me.reshape(-1), want, atol=1e-6)
    F.svd_quant(prefill, quant_func=Q, metis_mode="mean", mean_cache=cache, cache_key="k")
    assert cache["k"][1] == 10                # a new prefill starts over


def test_unknown_mode_raises():
    with pytest.raises(ValueError, match="Unsupported metis_mode"):
        F.svd_quant(torch.randn(2, 3, 16), quant_func=Cast2Fp32, metis_mode="nope")


@pytest.mark.parametrize("shape,budget", [((2, 3, 1536), 128), ((64, 1536), 1)])
def test_block_hadamard_round_trip(shape, budget):
    x = torch.randn(*shape)
    F.hadamard_workspace_mb = budget          # 1 MiB forces several chunks
    y = F._apply_hadamard_blocks(x, inverse=False)
    assert not torch.allclose(y, x)
    torch.testing.assert_close(F._apply_hadamard_blocks(y, inverse=True), x, rtol=1e-5, atol=1e-5)


def test_hadamard_configuration_errors():
    F.hadamard_tile_size = 12
    with pytest.raises(ValueError, match="power of two"):
        F._apply_hadamard_blocks(torch.randn(2, 24))
    F.hadamard_tile_size = 16
    with pytest.raises(ValueError, match="must divide"):
        F._apply_hadamard_blocks(torch.randn(2, 24))
    F.hadamard_backend = "nope"
    with pytest.raises(ValueError, match="Unsupported Hadamard backend"):
        F._apply_hadamard_blocks(torch.randn(2, 32))


def test_rht_is_not_applied_to_forward_activations():
    F.enable_nv_recipe = True
    x = torch.randn(2, 3, 1536)
    torch.testing.assert_close(F.quantize_input(x), x, rtol=1e-5, atol=1e-5)


def test_rht_rotates_only_the_weight_gradient_operands():
    F.enable_nv_recipe = True
    F.hadamard_backend, F.hadamard_tile_size = "torch_gemm", 16
    layer = LinearLowbit(16, 16, bias=False, args=SimpleNamespace(device="cpu", cache_quantized_weight=False))
    x = torch.randn(2, 3, 16, requires_grad=True)
    layer(x).sum().backward()
    want = torch.ones(16, 1) @ x.detach().reshape(-1, 16).sum(0, keepdim=True)     # identity QDQ: dW = 1 . sum x
    torch.testing.assert_close(layer.weight.grad, want, rtol=1e-5, atol=1e-5)


def test_replacement_without_forward_svd_does_not_split():
    model = torch.nn.Sequential(torch.nn.Linear(16, 8, bias=False))
    args = MetisArgs(enable_forward_svd=False)
    args.device = "cpu"
    layer = replace_linear_with_metis(model, dtype=torch.float32, metis_args=args, target_modules=["0"],
                                      compute_dtype=torch.float32)[0]
    assert isinstance(layer.warmup_linear, LinearLowbit)
    assert layer.vlinear is None and layer.ulinear is None and layer.s is None and not layer.is_svd_quant


def test_replacement_with_forward_svd_splits_on_cpu_and_keeps_the_product():
    torch.manual_seed(0)
    block = torch.nn.Module()
    block.q_proj, block.k_proj, block.o_proj = (torch.nn.Linear(32, 32, bias=b) for b in (True, False, False))
    model = torch.nn.Sequential(block)
    w, b = block.q_proj.weight.detach().clone(), block.q_proj.bias.detach().clone()
    args = MetisArgs(forward_svd_rank=8)
    args.device = "cpu"
    args.q_forward_input = args.q_forward_weight = "fp32"
    args.q_backward_input = args.q_backward_weight = args.q_backward_outputgrad = "fp32"
    replace_linear_with_metis(model, dtype=torch.float32, metis_args=args, compute_dtype=torch.float32)
    q = model[0].q_proj
    assert q.is_svd_quant and q.s.shape == (8,) and q.vlinear.weight.shape == (8, 32) and q.ulinear.weight.shape == (32, 8)
    assert sorted(n for n, _ in q.named_parameters()) == ["s", "ulinear.weight", "vlinear.weight", "warmup_linear.bias",
                                                          "warmup_linear.weight"]
    rebuilt = q.ulinear.weight @ torch.diag(q.s) @ q.vlinear.weight + q.warmup_linear.weight
    torch.testing.assert_close(rebuilt, w, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(q.warmup_linear.bias, b)
    # q/k share one activation group, o_proj has none
    assert model[0].q_proj.activation_group is model[0].k_proj.activation_group
    assert model[0].q_proj.activation_group["name"] == "0.qkv" and model[0].o_proj.activation_group is None
    x = torch.randn(2, 4, 32)
    torch.testing.assert_close(q(x), torch.nn.functional.linear(x, w, b), rtol=1e-4, atol=1e-4)


def test_low_rank_and_residual_branches_share_one_quantized_activation():
    Q = counting_quantizer()
    F.q_forward_input = Q
    mean_mode()
    layer = svd_layer()
    x = torch.randn(2, 3, 16, requires_grad=True)
    layer(x).sum().backward()
    assert Q.calls == 1
    assert x.grad is not None and layer.vlinear.weight.grad is not None and layer.warmup_linear.weight.grad is not None
    assert layer.s.grad is not None and layer.ulinear.weight.grad is not None
    assert "test.layer.shared" in layer.mean_cache


def test_projections_of_one_group_quantize_their_input_once():
    Q = counting_quantizer()
    F.q_forward_input = Q
    mean_mode()
    group = {"name": "blk.attention.qkv", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    q_proj, k_proj = svd_layer("blk.q_proj", group), svd_layer("blk.k_proj", group)
    x = torch.randn(2, 3, 16, requires_grad=True)
    (q_proj(x).sum() + k_proj(x).sum()).backward()
    assert Q.calls == 1
    assert q_proj.vlinear.weight.grad is not None and k_proj.vlinear.weight.grad is not None
    assert "blk.attention.qkv.shared" in group["mean_cache"]
    # a different tensor object, even with equal values, is quantized again (identity, not equality)
    q_proj(x.detach().clone())
    assert Q.calls == 2
    del x
    import gc
    gc.collect()


def test_forward_group_off_the_gpu_is_the_calls_one_after_the_other():
    from Metis.Metis.bitlinear import forward_group
    Q = counting_quantizer()
    F.q_forward_input = Q
    mean_mode()
    group = {"name": "blk.attention.qkv", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    q_proj, k_proj = svd_layer("blk.q_proj", group), svd_layer("blk.k_proj", group)
    x = torch.randn(2, 3, 16)
    with torch.no_grad():
        got = forward_group((q_proj, k_proj), x)
        want = [q_proj(x), k_proj(x)]
    assert Q.calls == 1                                  # one shared quantization for all four calls
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    plain = torch.nn.Linear(16, 8)
    assert torch.equal(forward_group((plain,), x)[0], plain(x))        # anything callable, e.g. before the layers are installed


def test_group_entry_is_dropped_when_the_input_dies():
    mean_mode()
    group = {"name": "g", "mean_cache": {}, "input_ref": None, "quantized_input": None}
    layer = svd_layer("l", group)
    x = torch.randn(1, 2, 16)
    with torch.no_grad():
        layer(x)
    assert group["input_ref"]() is x
    del x
    import gc
    gc.collect()
    assert group["input_ref"] is None and group["quantized_input"] is None


def test_merged_rollout_weight_matches_and_is_cached_until_a_factor_changes():
    mean_mode()
    layer = svd_layer(bias=True, cache=True)
    x = torch.randn(2, 3, 16)
    with torch.no_grad():
        expected = layer(x)
        BitLinear.rollout_merge_active = True
        actual = layer(x)
        first = layer._get_merged_rollout_weight(torch.float32)
        again = layer._get_merged_rollout_weight(torch.float32)
        layer.s.add_(0.1)
        updated = layer._get_merged_rollout_weight(torch.float32)
    torch.testing.assert_close(actual, expected)
    assert first is again and updated is not first
    # with gradients enabled the merged path is not taken
    y = layer(x.requires_grad_(True))
    assert y.grad_fn is not None


def test_backward_returns_fp32_weight_gradients_and_needs_3d_input():
    layer = LinearLowbit(16, 8, bias=True, args=SimpleNamespace(device="cpu"))
    x = torch.randn(2, 3, 16, requires_grad=True)
    y = layer(x)
    y.sum().backward()
    assert layer.weight.grad.dtype == torch.float32 and layer.bias.grad.shape == (8,)
    torch.testing.assert_close(layer.bias.grad, torch.full((8,), 6.0))
    with pytest.raises(IndexError):
        layer(torch.randn(3, 16, requires_grad=True)).sum().backward()     # 2-D is unsupported, as in the reference


def test_constructor_writes_the_process_global_configuration():
    args = MetisArgs(enable_forward_svd=False, metis_mode="mean")
    args.device = "cpu"
    args.q_forward_input = args.q_forward_weight = "fp8e4m3"
    args.q_backward_outputgrad = "fp4e2m1"
    BitLinear(16, 8, args=args, bias=False, dtype=torch.float32, compute_dtype=torch.bfloat16)
    assert F.q_forward_input is quant_func["fp8e4m3"] and F.q_backward_outputgrad is quant_func["fp4e2m1"]
    assert F.compute_dtype is torch.bfloat16 and F.metis_mode == "mean"
    assert F.tp_simulation is False and F.tp_simulate is False      # written under one name, read under the other
    with pytest.raises(ValueError, match="Unsupported compute_dtype"):
        BitLinear(16, 8, args=args, dtype=torch.float64)


def test_graph_capture_and_packed_export_need_a_cuda_device():
    # no CPU fallback anywhere on the NVFP4 path: the helpers say so instead of computing something else
    from fp4_post_b200 import checkpoint, graphs, ops
    if torch.cuda.is_available():
        pytest.skip("checks the message given on a machine without a GPU")
    with pytest.raises(RuntimeError, match="CUDA"):
        graphs.GraphedStep(lambda: None)
    with pytest.raises((RuntimeError, TypeError, ValueError)):
        ops.lowrank_scale(torch.zeros(8, 8, dtype=torch.bfloat16), torch.ones(8), torch.ones(1), torch.ones(1))
    with pytest.raises((RuntimeError, AssertionError)):
        checkpoint.export_packed({"m.warmup_linear.weight": torch.zeros(16, 32)}, device="cuda")


def test_random_lane_is_scoped_and_restored():
    from fp4_post_b200.Metis.Metis.quant import Cast2NVFp4e2m1Block, random_lane
    base = Cast2NVFp4e2m1Block._lane
    with random_lane(3):
        assert Cast2NVFp4e2m1Block._lane == 3
        with random_lane(1):
            assert Cast2NVFp4e2m1Block._lane == 1
        assert Cast2NVFp4e2m1Block._lane == 3
    assert Cast2NVFp4e2m1Block._lane == base


def test_a_saved_operand_notices_an_in_place_change_before_it_quantizes_again():
    from types import SimpleNamespace
    from Metis.Metis.bitlinear import PackedOperand

    class Recorder:
        calls = 0

        @classmethod
        def quantize_packed(cls, x, **kw):
            cls.calls += 1
            return SimpleNamespace(row_vec=None, kw=kw)

    x = torch.randn(32, 32)
    op = PackedOperand(SimpleNamespace(row_vec=None), x, Recorder, x.shape)
    x.add_(1.0)                                    # what autograd reports for a saved tensor
    with pytest.raises(RuntimeError, match="modified in place"):
        op.transposed()
    assert Recorder.calls == 0
    fresh = PackedOperand(SimpleNamespace(row_vec=None), x, Recorder, x.shape, rotate=5)
    qt = fresh.transposed()
    assert Recorder.calls == 1 and qt.kw["transpose"] and qt.kw["hadamard_signs"] == 5 and fresh.transposed() is qt
