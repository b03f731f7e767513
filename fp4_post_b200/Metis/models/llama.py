"""RMSNorm of the reference's demo LLaMA (src/Metis/models/llama.py:16-31), plus the fused
RMSNorm -> NVFP4 entry the B200 build adds.  The rest of that file (toy attention, RoPE,
pipeline wrapper) is outside the accelerated path and is not mirrored."""
from __future__ import annotations

import weakref

import torch
from torch import nn

from fp4_post_b200 import cabi, ops
from fp4_post_b200.Metis.Metis.bitlinear import LinearLowbitFunction, PackedOperand
from fp4_post_b200.Metis.Metis.quant import Cast2NVFp4e2m1BlockNOSR, is_native


class _NormWithMean(torch.autograd.Function):
    """y = RMSNorm(x) * weight and the column mean of y from one kernel (one read of x); the backward is
    the ordinary RMSNorm backward, with the rounding of the normalised value to x's dtype (llama.py:28)
    passed straight through."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        y, mean, rstd = ops.rmsnorm_mean(x, weight, eps)
        ctx.save_for_backward(x, weight, rstd)
        ctx.mark_non_differentiable(mean)
        return y, mean

    @staticmethod
    def backward(ctx, dy, _dmean):
        x, weight, rstd = ctx.saved_tensors
        cols = x.shape[-1]
        xf = x.reshape(-1, cols).float()
        n = xf * rstd[:, None]
        dyf = dy.reshape(-1, cols).float()
        dweight = (dyf * n.to(x.dtype).float()).sum(dim=0).to(weight.dtype)
        dn = dyf * weight.float()
        dx = rstd[:, None] * (dn - n * (dn * n).mean(dim=-1, keepdim=True))
        return dx.to(x.dtype).reshape(x.shape), dweight, None


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

    def forward_quantized(self, x: torch.Tensor, *, return_norm: bool = False, activation_group: dict | None = None):
        """Normalise, scale and quantize to NVFP4 for the projections that follow, in the activation mode
        the layers are configured with (the class attributes of LinearLowbitFunction):

          direct (enable_activation_svd off), no autograd   ONE kernel: x is read once, codes and scales come out
          mean mode (the GRPO default), or autograd on      two passes: normalise + column mean of the output,
                                                            then the quantizer on the normalised tensor (both
                                                            orientations at once when autograd is recording);
                                                            differentiable, the rolling decode mean is kept
          anything else (svd mode, other quantizers)        the unfused path: forward(), then quantize_input

        Returns a PackedOperand that `LinearLowbit.forward(..., quantized_input=...)` and `BitLinear`
        consume directly (with return_norm=True also the normalised tensor).  If `activation_group` (the
        dict the projection layers of one group share) is given together with return_norm=True, the
        result is registered there under the identity of the returned normalised tensor, so q/k/v (or
        gate/up) find it without quantizing again."""
        if not x.is_cuda:
            raise RuntimeError("RMSNorm.forward_quantized runs on sm_100a kernels only (no CPU fallback)")
        F = LinearLowbitFunction
        centred = bool(F.enable_activation_svd)
        recording = torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)
        mean_cache = activation_group["mean_cache"] if activation_group is not None else None
        cache_key = f"{activation_group['name']}.shared" if activation_group is not None else "default"
        native = is_native(F.q_forward_input) and F.gemm_mode == "packed" and not F.tp_simulate and x.shape[-1] % 16 == 0
        if not native or (centred and F.metis_mode != "mean"):
            y = self.forward(x)
            packed = F.quantize_input(y, mean_cache=mean_cache, cache_key=cache_key)
        elif centred or recording:
            y, mean = _NormWithMean.apply(x, self.weight, self.eps)
            packed = F._pack_centred(y.to(F.compute_dtype), F.q_forward_input, centred, mean_cache, cache_key,
                                     both=torch.is_grad_enabled(), fresh_mean=mean if centred else None)
        else:
            with torch.no_grad():
                q, y = ops.rmsnorm_nvfp4_quantize(x, self.weight, self.eps, sf_layout=cabi.SF_MMA, return_norm=True)
            packed = PackedOperand(q, y.reshape(-1, y.shape[-1]), Cast2NVFp4e2m1BlockNOSR, y.shape)
        if activation_group is not None:

            def forget(dead, group=activation_group):
                if group.get("input_ref") is dead:
                    group["input_ref"] = None
                    group["quantized_input"] = None

            activation_group["input_ref"] = weakref.ref(y, forget)
            activation_group["quantized_input"] = packed
        return (packed, y) if return_norm else packed
