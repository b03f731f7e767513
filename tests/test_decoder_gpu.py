"""The decoder harness with real NVFP4 Metis layers on the GPU: the fused norm -> quantizer entry feeds
the q/k/v and gate/up groups, the whole training step captures into one CUDA graph, and the fused-norm
model agrees with the same model running plain RMSNorm modules."""
import copy

import pytest
import torch

import fp4_post_b200

fp4_post_b200.install_reference_aliases()

from fp4_post_b200.decoder import Decoder, DecoderConfig  # noqa: E402
from fp4_post_b200.graphs import GraphedStep  # noqa: E402
from grpo.grpo import MetisArgs, replace_linear_with_metis  # noqa: E402
from Metis.Metis import bitlinear  # noqa: E402
from Metis.Metis.bitlinear import BitLinear, LinearLowbitFunction as F, forward_group  # noqa: E402
from Metis.Metis.quant import Cast2NVFp4e2m1BlockNOSR  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
SMALL = DecoderConfig(hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000)


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def _metis_decoder(fuse_norms, backward_q="nvfp4e2m1bnosr"):
    torch.manual_seed(0)
    model = Decoder(SMALL, fuse_norms=fuse_norms).to(DEV).to(torch.bfloat16)
    args = MetisArgs(forward_svd_rank=32, activation_lowrank_svd=32, backward_lowrank_svd=32)
    args.device = DEV
    args.q_backward_input = args.q_backward_weight = args.q_backward_outputgrad = backward_q
    replace_linear_with_metis(model, dtype=torch.bfloat16, metis_args=args, compute_dtype=torch.bfloat16)
    return model


def test_fused_norms_feed_the_projection_groups_and_match_plain_norms():
    ids = torch.randint(0, SMALL.vocab, (2, 64), device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    calls = {"n": 0}
    real = Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual.__func__

    def counting(cls, x, **kw):
        calls["n"] += 1
        return real(cls, x, **kw)

    losses, grads = {}, {}
    for fused in (True, False):
        model = _metis_decoder(fused)
        Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual = classmethod(counting)
        try:
            calls["n"] = 0
            loss = model.loss(ids)
            per_forward = calls["n"]
            loss.backward()
        finally:
            Cast2NVFp4e2m1BlockNOSR.quantize_packed_dual = classmethod(real)
        # per block: 4 activations (qkv group, o_proj, gate/up group, down_proj) + 7 x (V, R) weights
        assert per_forward == SMALL.layers * (4 + 14), (fused, per_forward)
        losses[fused] = float(loss)
        grads[fused] = {n: p.grad.float().clone() for n, p in model.named_parameters()}
        assert all(torch.isfinite(g).all() for g in grads[fused].values())
        assert isinstance(model.layers[0].self_attn.q_proj, BitLinear)
    assert abs(losses[True] - losses[False]) < 2e-2 * abs(losses[False])
    name = "layers.1.mlp.down_proj.warmup_linear.weight"
    a, b = grads[True][name], grads[False][name]
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.9


def test_a_whole_decoder_step_replays_from_one_graph():
    model = _metis_decoder(True, backward_q="nvfp4e2m1b")
    params = list(model.parameters())
    ids = torch.randint(0, SMALL.vocab, (2, 64), device=DEV, generator=torch.Generator(device=DEV).manual_seed(2))

    def step():
        for p in params:
            p.grad = None
        loss = model.loss(ids)
        loss.backward()
        return loss

    eager = float(step())
    graphed = GraphedStep(step, warmup=1)
    l1 = float(graphed())
    g1 = model.layers[0].mlp.down_proj.warmup_linear.weight.grad.clone()
    l2 = float(graphed())
    g2 = model.layers[0].mlp.down_proj.warmup_linear.weight.grad.clone()
    graphed.release()
    assert abs(l1 - eager) < 1e-3 * abs(eager) and l1 == l2            # the forward rounds to nearest: deterministic
    assert torch.isfinite(g2).all() and not torch.equal(g1, g2)         # the backward draws fresh bits per replay


@pytest.mark.parametrize("tokens", [16, 128])
def test_a_projection_group_on_parallel_streams_equals_the_calls_one_after_the_other(tokens):
    """Rollout (no_grad): q/k/v and gate/up run as branches of their own behind the shared quantization; the
    logits are bit for bit those of the sequential forward, eagerly and replayed from a CUDA graph."""
    model = _metis_decoder(True)
    for m in model.modules():
        if hasattr(m, "cache_quantized_weight"):
            m.cache_quantized_weight = True
    ids = torch.randint(0, SMALL.vocab, (1, tokens), device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    attn = model.layers[0].self_attn
    h = torch.randn(1, tokens, SMALL.hidden, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        bitlinear.GROUP_BRANCHES = False
        try:
            want_logits = model(ids)
            want = forward_group((attn.q_proj, attn.k_proj, attn.v_proj), h)
        finally:
            bitlinear.GROUP_BRANCHES = True
        got = forward_group((attn.q_proj, attn.k_proj, attn.v_proj), h)
        logits = model(ids)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        assert torch.equal(logits, want_logits)

        def rollout():
            return model(ids)
        graphed = GraphedStep(rollout, warmup=2)
        replayed = graphed()
        torch.cuda.synchronize()
        assert torch.equal(replayed, want_logits)
        graphed.release()
