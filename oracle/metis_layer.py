"""CPU restatement of the reference's Metis linear layer in its default ("mean") mode with
round-to-nearest NVFP4 everywhere: forward and backward of

    y = U (s . (x^ Vq^T)) + x^ Rq^T + b,     x^ = mean + QDQ(x - mean)

TEST INFRASTRUCTURE ONLY (also the timed CPU baseline of the benchmark).  Follows
decisivemoments/fp4-post src/Metis/Metis/bitlinear.py: activation quantization 311-336 and
371-393, forward 407-441 and 736-769, backward 443-513 (gradient of the quantized linears) with
autograd's rules for the unquantized `torch.mul(self.s, y)` and `ulinear` in between.  The
quantizer is the C oracle (oracle/nvfp4_oracle.c); products are fp32 torch.matmul.
Parity is pinned by tests/golden/layer_cases.npz, recorded from the reference's own BitLinear.
"""
from __future__ import annotations

import numpy as np
import torch

from . import nvfp4_oracle as O


def qdq(t: torch.Tensor, threads: int = 1) -> torch.Tensor:
    """Fake quantization of a 2-D fp32 tensor along its last dimension (quant.py:6-36)."""
    codes, scales, unit, _ = O.quantize(t.numpy(), threads=threads)
    return torch.from_numpy(O.dequantize(codes, scales, unit))


def mean_qdq(t: torch.Tensor, threads: int = 1) -> torch.Tensor:
    """mean + QDQ(t - mean) over the rows of a 2-D tensor (bitlinear.py:326-332)."""
    me = t.mean(dim=0, keepdim=True)
    return me + qdq(t - me, threads)


def forward(x, U, s, V, R, bias=None, threads: int = 1):
    """x [B,T,K]; U [N,r], s [r], V [r,K], R [N,K].  Returns y and what backward needs."""
    B, T, K = x.shape
    xh = mean_qdq(x.reshape(-1, K), threads)          # one shared activation for both branches
    Vq, Rq = qdq(V, threads), qdq(R, threads)
    yv = xh @ Vq.T                                    # vlinear
    ts = s * yv                                       # torch.mul(self.s, y)
    y = ts @ U.T + xh @ Rq.T                          # ulinear (plain) + warmup_linear
    if bias is not None:
        y = y + bias
    return y.reshape(B, T, -1), dict(xh=xh, Vq=Vq, Rq=Rq, yv=yv, ts=ts)


def backward(grad_out, saved, U, s, has_bias: bool, threads: int = 1):
    """Gradients of forward(); the output gradients of the two quantized linears are
    mean-centred and fake-quantized (bitlinear.py:462-474), grad_bias comes from the
    unquantized gradient (bitlinear.py:455)."""
    B, T, N = grad_out.shape
    g = grad_out.reshape(-1, N)
    xh, Vq, Rq, yv, ts = (saved[k] for k in ("xh", "Vq", "Rq", "yv", "ts"))
    dbias = g.sum(dim=0) if has_bias else None
    # residual branch
    gq = mean_qdq(g, threads)
    dR = gq.T @ xh
    dx = gq @ Rq
    # ulinear and the scaling by s
    dU = g.T @ ts
    d_ts = g @ U
    ds = (d_ts * yv).sum(dim=0)
    d_yv = d_ts * s
    # vlinear
    dq = mean_qdq(d_yv, threads)
    dV = dq.T @ xh
    dx = dx + dq @ Vq
    return dict(dx=dx.reshape(B, T, -1), dR=dR, dV=dV, dU=dU, ds=ds, dbias=dbias)


def split_weight(W: torch.Tensor, rank: int):
    """W = U diag(s) V + R by exact fp32 SVD (bitlinear.py:797-827)."""
    U, S, Vh = torch.linalg.svd(W.float(), full_matrices=False)
    U, S, Vh = U[:, :rank].contiguous(), S[:rank].contiguous(), Vh[:rank].contiguous()
    return U, S, Vh, W - U @ torch.diag(S) @ Vh


def flops(M: int, N: int, K: int, r: int, backward_too: bool = True) -> int:
    """Algorithmic flops of the layer: 2MNK + 2Mr(K+N) forward, three times that with backward."""
    f = 2 * M * N * K + 2 * M * r * (K + N)
    return 3 * f if backward_too else f
