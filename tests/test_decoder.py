"""The Qwen2-style decoder harness on the CPU: shapes, the loss, and that `replace_linear_with_metis`
(the reference's installer, src/grpo/grpo.py:119-196) finds its seven projections per block by name and
groups q/k/v and gate/up.  With identity quantizers W = U diag(s) V + R is exact, so the Metis model
must reproduce the plain model."""
import copy

import torch

import fp4_post_b200

fp4_post_b200.install_reference_aliases()

from fp4_post_b200.decoder import QWEN2_1P5B, QWEN2_7B, Decoder, DecoderConfig  # noqa: E402
from grpo.grpo import MetisArgs, replace_linear_with_metis  # noqa: E402
from Metis.Metis.bitlinear import BitLinear  # noqa: E402

TINY = DecoderConfig(hidden=64, layers=2, heads=4, kv_heads=2, head_dim=16, ffn=128, vocab=97)


def test_configurations_carry_the_benchmark_shapes():
    assert (QWEN2_1P5B.hidden, QWEN2_1P5B.layers, QWEN2_1P5B.heads, QWEN2_1P5B.kv_heads, QWEN2_1P5B.ffn, QWEN2_1P5B.vocab) == (1536, 28, 12, 2, 8960, 151936)
    assert (QWEN2_7B.hidden, QWEN2_7B.layers, QWEN2_7B.heads, QWEN2_7B.kv_heads, QWEN2_7B.ffn, QWEN2_7B.vocab) == (3584, 28, 28, 4, 18944, 152064)
    # per token and layer: q, o 1536x1536, k, v 1536x256, gate, up 1536x8960, down 8960x1536, plus the rank-64 terms
    per_layer = sum(2 * n * k + 2 * 64 * (k + n) for k, n in ((1536, 1536), (1536, 256), (1536, 256), (1536, 1536), (1536, 8960), (1536, 8960), (8960, 1536)))
    assert QWEN2_1P5B.linear_flops_per_token(64) == 28 * per_layer


def test_metis_layers_install_by_name_and_reproduce_the_plain_model_with_identity_quantizers():
    torch.manual_seed(0)
    plain = Decoder(TINY)
    ids = torch.randint(0, TINY.vocab, (2, 12))
    want = plain(ids)
    assert want.shape == (2, 12, TINY.vocab)
    args = MetisArgs(forward_svd_rank=8, activation_lowrank_svd=8, backward_lowrank_svd=8, enable_activation_svd=False, enable_backward_svd=False)
    args.device = "cpu"
    for k in ("q_forward_input", "q_forward_weight", "q_backward_input", "q_backward_weight", "q_backward_outputgrad"):
        setattr(args, k, "fp32")
    metis = replace_linear_with_metis(copy.deepcopy(plain), dtype=torch.float32, metis_args=args, compute_dtype=torch.float32)
    blk = metis.layers[0]
    names = [n for n, m in metis.named_modules() if isinstance(m, BitLinear)]
    assert len(names) == 7 * TINY.layers and not isinstance(metis.lm_head, BitLinear)
    assert blk.self_attn.q_proj.activation_group is blk.self_attn.k_proj.activation_group is blk.self_attn.v_proj.activation_group
    assert blk.mlp.gate_proj.activation_group is blk.mlp.up_proj.activation_group
    assert blk.self_attn.o_proj.activation_group is None and blk.mlp.down_proj.activation_group is None
    got = metis(ids)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    loss = metis.loss(ids)
    loss.backward()
    assert torch.isfinite(loss)
    for n, p in metis.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n
