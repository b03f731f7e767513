"""A Qwen2-style decoder in plain torch, the caller the Metis layers sit in during post-training.

The reference installs its layers into Hugging Face Qwen2 models (src/grpo/grpo.py:119-196:
`replace_linear_with_metis` swaps q/k/v/o/gate/up/down projections for BitLinear and lets q/k/v and
gate/up share one quantized activation).  This module is that model family restated with the same
sub-module names, so the same function installs the same layers, and nothing else: token embedding,
pre-norm blocks (RMSNorm -> GQA attention with rotary embeddings -> residual, RMSNorm -> SwiGLU ->
residual), final norm, untied bf16 lm_head.  Attention is torch's scaled_dot_product_attention.
It exists to measure the layer inside a whole training step (random weights, synthetic token ids); it
is not a model zoo.

With `fuse_norms=True` the two RMSNorms of a block hand their output to the projection group that
follows already quantized (RMSNorm.forward_quantized): one pass over the hidden state computes the
normalised tensor and its column mean, the next quantizes it for all projections of the group.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as Fn
from torch import nn

from fp4_post_b200.Metis.Metis.bitlinear import forward_group
from fp4_post_b200.Metis.models.llama import RMSNorm


@dataclass
class DecoderConfig:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 1e6
    eps: float = 1e-6
    qkv_bias: bool = True            # Qwen2: biases on q/k/v only

    def linear_flops_per_token(self, rank: int) -> int:
        """Algorithmic forward flops of the Metis projections per token: 2 N K + 2 r (K + N) each."""
        shapes = [(self.hidden, self.heads * self.head_dim), (self.hidden, self.kv_heads * self.head_dim),
                  (self.hidden, self.kv_heads * self.head_dim), (self.heads * self.head_dim, self.hidden),
                  (self.hidden, self.ffn), (self.hidden, self.ffn), (self.ffn, self.hidden)]
        return self.layers * sum(2 * n * k + 2 * rank * (k + n) for k, n in shapes)


QWEN2_1P5B = DecoderConfig(hidden=1536, layers=28, heads=12, kv_heads=2, head_dim=128, ffn=8960, vocab=151936)
QWEN2_7B = DecoderConfig(hidden=3584, layers=28, heads=28, kv_heads=4, head_dim=128, ffn=18944, vocab=152064)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, T, D]; rotate-half convention."""
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return x * cos + torch.cat((-x2, x1), dim=-1) * sin


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.q_proj = nn.Linear(cfg.hidden, cfg.heads * cfg.head_dim, bias=cfg.qkv_bias)
        self.k_proj = nn.Linear(cfg.hidden, cfg.kv_heads * cfg.head_dim, bias=cfg.qkv_bias)
        self.v_proj = nn.Linear(cfg.hidden, cfg.kv_heads * cfg.head_dim, bias=cfg.qkv_bias)
        self.o_proj = nn.Linear(cfg.heads * cfg.head_dim, cfg.hidden, bias=False)

    def forward(self, h, cos, sin):
        B, T, _ = h.shape
        c = self.cfg
        q, k, v = forward_group((self.q_proj, self.k_proj, self.v_proj), h)     # one shared activation, three branches
        q = q.view(B, T, c.heads, c.head_dim).transpose(1, 2)
        k = k.view(B, T, c.kv_heads, c.head_dim).transpose(1, 2)
        v = v.view(B, T, c.kv_heads, c.head_dim).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = Fn.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(a.transpose(1, 2).reshape(B, T, c.heads * c.head_dim))


class MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden, cfg.ffn, bias=False)
        self.up_proj = nn.Linear(cfg.hidden, cfg.ffn, bias=False)
        self.down_proj = nn.Linear(cfg.ffn, cfg.hidden, bias=False)

    def forward(self, h):
        gate, up = forward_group((self.gate_proj, self.up_proj), h)
        return self.down_proj(Fn.silu(gate) * up)


class Block(nn.Module):
    def __init__(self, cfg: DecoderConfig, fuse_norms: bool):
        super().__init__()
        self.fuse_norms = fuse_norms
        self.input_layernorm = RMSNorm(cfg.hidden, cfg.eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden, cfg.eps)
        self.mlp = MLP(cfg)

    def _normed(self, norm, x, first_of_group):
        group = getattr(first_of_group, "activation_group", None)
        if self.fuse_norms and group is not None and x.is_cuda:
            return norm.forward_quantized(x, return_norm=True, activation_group=group)[1]
        return norm(x)

    def forward(self, x, cos, sin):
        x = x + self.self_attn(self._normed(self.input_layernorm, x, self.self_attn.q_proj), cos, sin)
        return x + self.mlp(self._normed(self.post_attention_layernorm, x, self.mlp.gate_proj))


class Decoder(nn.Module):
    def __init__(self, cfg: DecoderConfig, fuse_norms: bool = True):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab, cfg.hidden)
        self.layers = nn.ModuleList(Block(cfg, fuse_norms) for _ in range(cfg.layers))
        self.norm = RMSNorm(cfg.hidden, cfg.eps)
        self.lm_head = nn.Linear(cfg.hidden, cfg.vocab, bias=False)      # stays bf16: not in the reference's target list

    def rotary(self, T: int, device, dtype):
        d = self.cfg.head_dim
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        ang = torch.outer(torch.arange(T, device=device, dtype=torch.float32), inv)
        ang = torch.cat((ang, ang), dim=-1)
        return ang.cos().to(dtype)[None, None], ang.sin().to(dtype)[None, None]

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.embed_tokens(ids)
        cos, sin = self.rotary(ids.shape[1], ids.device, x.dtype)
        for blk in self.layers:
            x = blk(x, cos, sin)
        return self.lm_head(self.norm(x))

    def loss(self, ids: torch.Tensor) -> torch.Tensor:
        """Next-token cross entropy on the given ids."""
        logits = self.forward(ids)
        return Fn.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
