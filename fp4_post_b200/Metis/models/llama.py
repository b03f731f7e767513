"""RMSNorm of the reference's demo LLaMA (src/Metis/models/llama.py:16-31), plus the fused
RMSNorm -> NVFP4 entry the B200 build adds.  The rest of that file (toy attention, RoPE,
pipeline wrapper) is outside the accelerated path and is not mirrored."""
from __future__ import annotations

import torch
from torch import nn

from fp4_post_b200 import cabi, ops
from fp4_post_b200.Metis.Metis.bitlinear import PackedOperand
from fp4_post_b200.Metis.Metis.quant import Cast2NVFp4e2m1BlockNOSR


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, device: str = "cuda"):
        super().__init__()
        self.device = device
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def _norm(self, x):
        return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps)

    def forward(self, x):
        # fp32 normalisation, rounded back to x's dtype, then scaled (llama.py:26-31)
        return self._norm(x.float()).type_as(x) * self.weight

    @torch.no_grad()
    def forward_quantized(self, x: torch.Tensor, *, return_norm: bool = False, activation_group: dict | None = None):
        """One kernel: normalise, scale and quantize to NVFP4, reading x from HBM once.

        Returns a PackedOperand that `LinearLowbit.forward(..., quantized_input=...)` and
        `BitLinear` consume directly.  If `activation_group` (the dict the projection layers of
        one group share) is given together with return_norm=True, the result is registered there
        under the identity of the returned normalised tensor, so q/k/v (or gate/up) find it
        without quantizing again.  Inference only (no autograd)."""
        if not x.is_cuda:
            raise RuntimeError("RMSNorm.forward_quantized runs on sm_100a kernels only (no CPU fallback)")
        res = ops.rmsnorm_nvfp4_quantize(x, self.weight, self.eps, sf_layout=cabi.SF_MMA, return_norm=True)
        q, y = res
        packed = PackedOperand(q, y.reshape(-1, y.shape[-1]), Cast2NVFp4e2m1BlockNOSR, y.shape)
        if activation_group is not None:
            import weakref

            def forget(dead, group=activation_group):
                if group.get("input_ref") is dead:
                    group["input_ref"] = None
                    group["quantized_input"] = None

            activation_group["input_ref"] = weakref.ref(y, forget)
            activation_group["quantized_input"] = packed
        return (packed, y) if return_norm else packed
