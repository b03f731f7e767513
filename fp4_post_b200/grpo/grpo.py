"""Dependency-light mirror of the two symbols of the reference's src/grpo/grpo.py that configure
and install the Metis layers: `MetisArgs` (grpo.py:62-117) and `replace_linear_with_metis` /
`replace_model_with_metis` (grpo.py:119-215).  The TRL trainer glue around them is not mirrored."""
from __future__ import annotations

import torch

from fp4_post_b200.Metis.Metis import BitLinear


class MetisArgs:
    """Plain attribute bag read by BitLinear / LinearLowbit; defaults are the GRPO defaults."""

    def __init__(self, metis_mode: str = "mean", enable_forward_svd: bool = True, enable_activation_svd: bool = True,
                 enable_backward_svd: bool = True, forward_svd_rank: int = 64, activation_lowrank_svd: int = 64,
                 backward_lowrank_svd: int = 64, cache_quantized_weight: bool = False, compile_qdq: bool = False,
                 enable_nv_recipe: bool = False, hadamard_workspace_mb: int = 128, hadamard_tile_size: int = 16,
                 hadamard_backend: str = "auto"):
        self.device = "cuda"
        self.enable_forward_svd = enable_forward_svd
        self.enable_lowbit = True
        self.enable_te = False
        # forward: round to nearest; backward: stochastic rounding
        self.q_forward_input = "nvfp4e2m1bnosr"
        self.q_forward_weight = "nvfp4e2m1bnosr"
        self.q_backward_input = "nvfp4e2m1b"
        self.q_backward_weight = "nvfp4e2m1b"
        self.q_backward_outputgrad = "nvfp4e2m1b"
        self.enable_backward_svd = enable_backward_svd
        self.backward_lowrank_svd = backward_lowrank_svd
        self.backward_lowrank_niter = 2
        self.enable_activation_svd = enable_activation_svd
        self.activation_lowrank_svd = activation_lowrank_svd
        self.activation_lowrank_niter = 0
        self.activation_broadcast_dim = 0
        self.backward_broadcast_dim = -1
        self.enable_nv_recipe = enable_nv_recipe
        self.hadamard_workspace_mb = hadamard_workspace_mb
        self.hadamard_tile_size = hadamard_tile_size
        self.hadamard_backend = hadamard_backend
        self.gradacc_broadcast = False
        self.gradacc_broadcast_steps = 1
        self.forward_svd_warmup_steps = 50    # layers are split explicitly after replacement
        self.forward_svd_rank = forward_svd_rank
        self.tp_simulation = False
        self.tp_parts = 4
        self.metis_mode = metis_mode
        self.cache_quantized_weight = cache_quantized_weight
        self.compile_qdq = compile_qdq


_QKV = {"q_proj", "k_proj", "v_proj"}
_GATE_UP = {"gate_proj", "up_proj"}
DEFAULT_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def replace_linear_with_metis(model, dtype, metis_args, target_modules=None, compute_dtype=None):
    """Swap every nn.Linear whose last name component is in `target_modules` for a BitLinear that
    carries the same weights; q/k/v and gate/up of one block share an activation group so that
    their common input is quantized once."""
    targets = DEFAULT_TARGETS if target_modules is None else target_modules
    compute_dtype = torch.float32 if compute_dtype is None else compute_dtype
    groups = {}
    for name, module in list(model.named_modules()):
        parent_name, _, leaf = name.rpartition(".")
        if leaf not in targets or not isinstance(module, torch.nn.Linear):
            continue
        parent = model.get_submodule(parent_name) if parent_name else model
        has_bias = module.bias is not None
        layer = BitLinear(in_features=module.in_features, out_features=module.out_features, args=metis_args,
                          bias=has_bias, dtype=dtype, compute_dtype=compute_dtype)
        if module.weight.numel() == 0:
            # ZeRO-3 leaves empty shards behind: gather before copying (grpo.py:160-167)
            import deepspeed
            with deepspeed.zero.GatheredParameters([module.weight], modifier_rank=0), torch.no_grad():
                layer.warmup_linear.weight.copy_(module.weight)
                if has_bias:
                    with deepspeed.zero.GatheredParameters([module.bias], modifier_rank=0):
                        layer.warmup_linear.bias.copy_(module.bias)
        else:
            with torch.no_grad():
                layer.warmup_linear.weight.copy_(module.weight)
                if has_bias:
                    layer.warmup_linear.bias.copy_(module.bias)
        layer.layer_name = name
        group_name = None
        if leaf in _QKV:
            group_name = f"{parent_name}.qkv"
        elif leaf in _GATE_UP:
            group_name = f"{parent_name}.gate_up"
        if group_name is not None:
            layer.activation_group = groups.setdefault(
                group_name, {"name": group_name, "mean_cache": {}, "input_ref": None, "quantized_input": None})
        if metis_args.enable_forward_svd:
            layer.split()
        setattr(parent, leaf, layer)
    return model


def replace_model_with_metis(model, metis_args=None):
    """bf16 storage and compute, default targets (grpo.py:199-215)."""
    metis_args = MetisArgs() if metis_args is None else metis_args
    return replace_linear_with_metis(model=model, dtype=torch.bfloat16, metis_args=metis_args,
                                     target_modules=list(DEFAULT_TARGETS), compute_dtype=torch.bfloat16)
