"""The Metis linear layer, API-compatible with the reference's src/Metis/Metis/bitlinear.py:
`LinearLowbitFunction` (autograd), `LinearLowbit`, `BitLinear`, with the same constructor
arguments, attributes, parameter names (warmup_linear / vlinear / ulinear / s), class-level
configuration and caches (weight cache keyed on Parameter._version, shared activation per
projection group by weakref identity, merged rollout weight, rolling decode mean).

Two execution modes, chosen per call:

  packed   operands are real NVFP4 (packed codes + E4M3 scales + unit, `PackedOperand`) produced
           by the native quantizers, and every product runs on the tcgen05 block-scaled GEMM with
           the bf16 rank-r term  U (s . x V^T)  fused into the same accumulator.  Taken when the
           configured quantizer classes are the native NVFP4 ones, tensors live on a CUDA device
           and `LinearLowbitFunction.gemm_mode == "packed"` (the default).
  dense    operands are dequantized tensors and the products are torch.matmul, exactly the
           reference's wiring (bitlinear.py:407-513).  Taken for stub / non-NVFP4 quantizer classes
           on any device (this is what the reference's own tests exercise), or when
           `gemm_mode == "dense"` (used to check the autograd wiring against the reference).

In packed mode the backward products contract over N (dX) and over tokens (dW), so W, D and x are
quantized a second time along those dimensions by the transposed quantizer; the reference
instead reuses values quantized along the last dimension (bitlinear.py:502-508).
"""
from __future__ import annotations

import math
import weakref

import torch
import torch.nn as nn
import torch.nn.init as init

from fp4_post_b200 import ops
from .quant import *  # noqa: F401,F403  (the reference re-exports its quantizers the same way)
from .quant import is_native, quant_func, random_lane


class PackedOperand:
    """One GEMM operand in NVFP4 with everything the backward products need.

    `q`      NVFP4Tensor of the matrix viewed as [rows, cols], blocks along cols; q.row_vec is the
             column mean that was subtracted (mean mode) or None.
    `source` the tensor it was quantized from (kept so that the transposed quantization needed by
             dX / dW can be produced on demand) and `quantizer` the class that did it.
    """

    def __init__(self, q, source, quantizer, shape, rotate=None):
        self.q = q
        self.source = source
        self.quantizer = quantizer
        self.shape = tuple(shape)      # shape of the tensor this stands for, e.g. [B, T, K]
        self.rotate = rotate           # sign mask of the Hadamard rotation of the transposed quantization, or None
        self._version = source._version    # what autograd's saved-tensor check would compare
        self._qt = None
        self._dense = {}
        self.mean_event = None         # recorded when the column mean exists (before the quantization that uses it)
        self.fresh = True              # produced by kernels of the current call (cleared by a weight-cache hit)
        self.ready_event = None        # quantized on the second stream: what the current stream waits for before its first use
        # Scale pass of one of the two outputs left to another stream (ops.nvfp4_quantize_dual(defer=...)): the
        # event after which that output is complete.  Every consumer's stream waits for it.
        self._q_event = None
        self._qt_event = None

    @property
    def dtype(self):
        return self.source.dtype

    @property
    def mean(self):
        return self.q.row_vec

    def transposed(self):
        """Quantization of the transpose (blocks along the rows of the source), cached."""
        if self._qt is None:
            if self.source._version != self._version:
                # the same complaint autograd makes about a saved tensor: the backward would otherwise
                # quantize values the forward never saw
                raise RuntimeError("a tensor needed for the backward of a Metis layer was modified in place after "
                                   f"the forward (version {self.source._version}, expected {self._version})")
            self._qt = self.quantizer.quantize_packed(self.source, transpose=True, mean=self.q.row_vec,
                                                      hadamard_signs=self.rotate)
        if self._qt_event is not None:
            torch.cuda.current_stream(self._qt.codes.device).wait_event(self._qt_event)
        return self._qt

    def rowmajor(self):
        """`q`, once its scale pass has run (see _q_event)."""
        if self._q_event is not None:
            torch.cuda.current_stream(self.q.codes.device).wait_event(self._q_event)
        return self.q

    def join_deferred(self):
        """Order the current stream after every scale pass of this operand that was left to another stream.
        Called where a forward or backward function ends, after its last launch: by then the pass is long
        finished, and a stream capture that ends there sees the other stream joined."""
        for ev in (self._q_event, self._qt_event):
            if ev is not None:
                torch.cuda.current_stream(self.q.codes.device).wait_event(ev)

    def dense(self, dtype):
        """The dequantized tensor the reference would have produced (mean added back)."""
        if dtype not in self._dense:
            native = dtype if dtype in (torch.bfloat16, torch.float32) else torch.float32
            self._dense[dtype] = self.q.dequantize(native).to(dtype).reshape(self.shape)
        return self._dense[dtype]


def _packed_matmul(a, b, rank1=(), lowrank=None, c=None, out_dtype=torch.bfloat16, sm_limit=0):
    return ops.nvfp4_gemm(a, b, rank1=rank1, lowrank=lowrank, c=c, out_dtype=out_dtype, sm_limit=sm_limit)


def _backward_can_pack(shared) -> bool:
    """Whether the configured backward can run on packed operands for this activation."""
    return LinearLowbitFunction._packed_backward_ok(shared.source)


def _bf16_factors(t32: torch.Tensor, u: torch.Tensor, act: torch.dtype):
    """The rank-r factors as bf16 operands of the side product.  With bf16 activations they are
    simply rounded (the reference computes them in bf16 too).  With fp32 activations each factor
    is split into a bf16 head and tail and the product is issued as [Th Tl Th] [Uh Uh Ul]^T, which
    keeps about 16 significant bits at three times the (small) rank."""
    r = t32.shape[1]
    if act != torch.float32 or 3 * r > 256:
        return t32.to(torch.bfloat16), u.to(torch.bfloat16)
    u32 = u.float()
    t_hi, u_hi = t32.to(torch.bfloat16), u32.to(torch.bfloat16)
    t_lo, u_lo = (t32 - t_hi.float()).to(torch.bfloat16), (u32 - u_hi.float()).to(torch.bfloat16)
    return torch.cat([t_hi, t_lo, t_hi], dim=1), torch.cat([u_hi, u_hi, u_lo], dim=1)


def _dual_ok(flat: torch.Tensor) -> bool:
    """Shapes the one-pass row + transposed quantizer takes."""
    return flat.shape[0] % 16 == 0 and flat.shape[1] % 16 == 0


def _gemm_ok(M, N, K):
    """Shapes the packed GEMM takes (rows of packed codes must be multiples of 16 bytes)."""
    return K % 32 == 0 and M > 0 and N > 0


# -----------------------------------------------------------------------------
# autograd.Function: quantized linear, forward and backward
# -----------------------------------------------------------------------------
class LinearLowbitFunction(torch.autograd.Function):
    """y = Q(x) @ Q(W)^T + b with a quantized backward (reference: bitlinear.py:18-513).
    Class attributes are process-global configuration written by BitLinear.__init__."""

    q_forward_input = Cast2Fp4e2m1
    q_forward_weight = Cast2Fp4e2m1
    q_backward_input = Cast2Fp4e2m1
    q_backward_weight = Cast2Fp4e2m1
    q_backward_outputgrad = Cast2Fp4e2m1

    enable_nv_recipe = False
    _hadamard_cache = {}
    hadamard_workspace_mb = 128
    hadamard_tile_size = 16
    hadamard_backend = "auto"
    _dao_hadamard_transform = None
    _dao_hadamard_checked = False
    _hadamard_sign_cache = {}

    activation_lowrank_niter = 0
    backward_lowrank_niter = 0
    enable_activation_svd = False
    activation_lowrank_svd = -1
    enable_backward_svd = False
    backward_lowrank_svd = -1
    activation_broadcast_dim = -1
    backward_broadcast_dim = -1

    tp_simulate = False
    tp_parts = 4

    compute_dtype = torch.float32
    metis_mode = "mean"
    mean_cache = None
    mean_cache_key = "default"

    # "packed": real FP4 operands on the tensor-core GEMM; "dense": dequantize + torch.matmul
    gemm_mode = "packed"
    # Packed mode only: rotate both operands of the weight-gradient product by the signed 16 x 16 Hadamard
    # matrix along the tokens before they are quantized (the NVIDIA baseline's treatment of the Wgrad
    # operands, bitlinear.py:395-405, folded into the transposed quantizer; the rotations cancel in the
    # product).  The forward-weight rotation of `enable_nv_recipe` (bitlinear.py:578-585) has no packed form
    # (the activation is quantized unrotated) and stays on the dense torch path.
    packed_wgrad_rht = False
    # Packed mode, CUDA: an operand that is quantized in both orientations hands the scale pass of the
    # orientation its first consumer does not need to a third stream (the transposed one of a forward
    # activation, the row-major one of an output gradient).  Results do not change.
    defer_scale_pass = True

    @staticmethod
    def _wgrad_rotation():
        """Sign mask of the Wgrad rotation (bit i set: position i of a block of 16 is negated), or None."""
        F = LinearLowbitFunction
        if not F.packed_wgrad_rht:
            return None
        signs = F._get_hadamard_sign(16, "cpu", torch.float32)
        return sum(1 << i for i in range(16) if signs[i] < 0)

    # ---- random Hadamard transform of the NV baseline (kept in torch; bitlinear.py:75-211) ----------
    @staticmethod
    def _get_hadamard(size: int, device, dtype) -> torch.Tensor:
        key = (int(size), device, dtype)
        hit = LinearLowbitFunction._hadamard_cache.get(key)
        if hit is not None:
            return hit
        if size <= 0 or size & (size - 1):
            raise ValueError(f"Hadamard block size must be a power of two, got {size}")
        h = torch.ones((1, 1), device=device, dtype=dtype)
        while h.shape[0] < size:   # Sylvester doubling
            h = torch.cat((torch.cat((h, h), dim=1), torch.cat((h, -h), dim=1)), dim=0)
        LinearLowbitFunction._hadamard_cache[key] = h
        return h

    @staticmethod
    def _get_hadamard_sign(size: int, device, dtype) -> torch.Tensor:
        key = (int(size), device, dtype)
        hit = LinearLowbitFunction._hadamard_sign_cache.get(key)
        if hit is not None:
            return hit
        gen = torch.Generator(device="cpu")
        gen.manual_seed(1729 + size)     # the reference's fixed seed, so both sides rotate alike
        bits = torch.randint(0, 2, (size,), generator=gen, dtype=torch.int8)
        signs = (bits * 2 - 1).to(device=device, dtype=dtype)
        LinearLowbitFunction._hadamard_sign_cache[key] = signs
        return signs

    @staticmethod
    def _get_dao_hadamard_transform():
        F = LinearLowbitFunction
        if not F._dao_hadamard_checked:
            try:
                from fast_hadamard_transform import hadamard_transform
                F._dao_hadamard_transform = hadamard_transform
            except ImportError:
                F._dao_hadamard_transform = None
            F._dao_hadamard_checked = True
        return F._dao_hadamard_transform

    @staticmethod
    def _apply_hadamard_blocks(value: torch.Tensor, inverse: bool = False) -> torch.Tensor:
        """x -> (x . signs) H per tile of the last dimension; inverse: (y H / d) . signs."""
        F = LinearLowbitFunction
        dim = value.shape[-1]
        if dim <= 1 or value.numel() == 0:
            return value
        tile = int(F.hadamard_tile_size)
        if tile <= 0 or tile & (tile - 1):
            raise ValueError(f"Hadamard tile size must be a positive power of two, got {tile}")
        if dim % tile:
            raise ValueError(f"RHT tile size {tile} must divide hidden dimension {dim}; "
                             "set --metis_hadamard_tile_size to a compatible power of two")
        if F.hadamard_backend not in {"auto", "dao_cuda", "torch_gemm"}:
            raise ValueError(f"Unsupported Hadamard backend: {F.hadamard_backend}")
        dao = F._get_dao_hadamard_transform() if (F.hadamard_backend in {"auto", "dao_cuda"} and value.is_cuda) else None
        if F.hadamard_backend == "dao_cuda" and dao is None:
            raise RuntimeError("Hadamard backend dao_cuda was requested but fast_hadamard_transform is unavailable. "
                               "Install it with: pip install -v git+https://github.com/Dao-AILab/fast-hadamard-transform.git")
        if dao is not None:
            flat = value.reshape(-1, tile)
            signs = F._get_hadamard_sign(tile, value.device, value.dtype)
            out = dao(flat, scale=1.0 / tile) * signs if inverse else dao(flat * signs, scale=1.0)
            return out.reshape_as(value)

        work_dtype = torch.float32 if value.dtype in (torch.float16, torch.bfloat16) else value.dtype
        h = F._get_hadamard(tile, value.device, work_dtype)
        signs = F._get_hadamard_sign(tile, value.device, work_dtype)
        tiles = value.reshape(-1, tile)
        out = torch.empty_like(tiles)
        # two work-dtype copies of a chunk are alive at once; stay inside the budget
        budget = max(1, int(F.hadamard_workspace_mb)) * 1024 * 1024
        step = max(1, budget // (2 * tile * torch.empty((), dtype=work_dtype).element_size()))
        for start in range(0, tiles.shape[0], step):
            chunk = tiles[start:start + step].to(work_dtype)
            if inverse:
                res = torch.mm(chunk, h).mul_(1.0 / tile).mul_(signs)
            else:
                res = torch.mm(chunk * signs, h)
            out[start:start + step].copy_(res)
        return out.reshape_as(value)

    # ---- low-rank / mean-centred fake quantization (dense mode; bitlinear.py:213-368) ---------------
    @staticmethod
    def _rolling_mean(flat: torch.Tensor, seq_len: int, mean_cache, cache_key):
        """Column mean of `flat`; at decode (one token per sequence) the count-weighted running
        mean over everything seen since the last prefill (bitlinear.py:314-328)."""
        rows = flat.shape[0]
        fresh = flat.mean(dim=0, keepdim=True)
        if seq_len == 1 and mean_cache is not None and cache_key in mean_cache:
            old, count = mean_cache[cache_key]
            total = count + rows
            me = (old * count + fresh * rows) / total
            mean_cache[cache_key] = (me.detach(), total)
            return me
        if mean_cache is not None:
            mean_cache[cache_key] = (fresh.detach(), rows)
        return fresh

    @staticmethod
    def svd_quant(input_: torch.Tensor, quant_func, rank: int = 60, niter: int = 0, broadcast_dim: int = -1,
                  tp_simulate: bool = False, tp_parts: int = 4, metis_mode="mean",
                  mean_cache: dict = None, cache_key: str = "default"):
        """Split the input into a high-precision part and a quantized remainder, then recombine.
        "mean": column mean + QDQ(x - mean).  "svd": rank-`rank` randomized SVD with quantized
        factors + QDQ(residual)."""

        def svd_piece(piece):
            picked = piece.select(broadcast_dim, 0) if broadcast_dim >= 0 else piece
            shape = picked.shape
            three_d = len(shape) == 3
            picked2 = picked.reshape(-1, shape[-1]) if three_d else picked
            full2 = piece.reshape(-1, shape[-1]) if three_d else piece
            dt = picked2.dtype
            as32 = picked2.to(torch.float32)
            if torch.isnan(as32).any() or torch.isinf(as32).any():
                print("⚠️ Warning: NaN or Inf detected in input before SVD")
            with torch.amp.autocast(as32.device.type, enabled=False):
                u, s, v = torch.svd_lowrank(as32, q=rank, niter=niter)
            u, s, vt = u.to(dt), s.to(dt), v.to(dt).T

            def three_call(t):
                sc = quant_func.get_scalar(t)
                return quant_func.rquant(quant_func.quant(t, sc), sc)

            kernel = three_call(u) @ torch.diag(s) @ three_call(vt)
            if broadcast_dim >= 0:
                kernel = kernel.unsqueeze(broadcast_dim)
            out = kernel + quant_func.quantize_dequantize(full2 - kernel)
            return out.view(shape[0], shape[1], -1) if three_d else out

        def mean_piece(piece):
            shape = piece.shape
            flat = piece.reshape(-1, shape[-1])
            seq_len = shape[1] if len(shape) == 3 else shape[0]
            me = LinearLowbitFunction._rolling_mean(flat, seq_len, mean_cache, cache_key)
            out = me + quant_func.quantize_dequantize(flat - me)
            return out.view(shape[0], shape[1], -1) if len(shape) == 3 else out

        if tp_simulate:
            width = input_.shape[-1]
            parts = max(1, int(tp_parts))
            cuts = [(width * p) // parts for p in range(parts + 1)]
            return torch.cat([svd_piece(input_[..., a:b]) for a, b in zip(cuts, cuts[1:]) if b > a], dim=-1)
        if metis_mode == "svd":
            return svd_piece(input_)
        if metis_mode == "mean":
            return mean_piece(input_)
        raise ValueError(f"Unsupported metis_mode: {metis_mode}")

    # ---- packed-mode quantization of activations / gradients ---------------------------------------------
    @staticmethod
    def _use_packed(tensor: torch.Tensor, quantizer) -> bool:
        F = LinearLowbitFunction
        return (F.gemm_mode == "packed" and tensor.is_cuda and is_native(quantizer)
                and not F.tp_simulate and tensor.shape[-1] % 16 == 0)

    @staticmethod
    def _pack_centred(tensor, quantizer, centred: bool, mean_cache=None, cache_key="default", both=False,
                      fresh_mean=None, defer=None):
        """NVFP4 of `tensor` ([..., C] viewed as rows), optionally after subtracting the column
        mean (rolling at decode).  The native counterpart of svd_quant(metis_mode="mean").
        `both`: the transposed quantization (needed by the backward products) comes out of the same
        pass over the tensor, where both dimensions are multiples of 16.  `fresh_mean`: the column
        mean of `tensor` when its producer computed it already (the fused RMSNorm does).  `defer`: see below."""
        flat = tensor.reshape(-1, tensor.shape[-1])
        mean = None
        if centred:
            seq_len = tensor.shape[1] if tensor.dim() == 3 else tensor.shape[0]
            fresh = ops.col_mean(flat) if fresh_mean is None else fresh_mean
            rows = flat.shape[0]
            if seq_len == 1 and mean_cache is not None and cache_key in mean_cache:
                old, count = mean_cache[cache_key]
                total = count + rows
                mean = (old.reshape(-1).float() * count + fresh * rows) / total
                mean_cache[cache_key] = (mean.detach().reshape(1, -1), total)
            else:
                mean = fresh
                if mean_cache is not None:
                    mean_cache[cache_key] = (fresh.detach().reshape(1, -1), rows)
        mean_event = None
        if mean is not None and flat.is_cuda:
            mean_event = torch.cuda.Event()
            mean_event.record()             # work that needs only the mean may overlap the quantization
        rotate = LinearLowbitFunction._wgrad_rotation()
        if both and _dual_ok(flat):
            # a centred operand's weight-gradient product needs the token sums of the transposed quantization
            # `defer`: the consumer that comes first needs one of the two outputs only; the scale pass of the other
            # ("rowmajor" or "transposed") runs on the third stream, off this stream's critical path
            defer = defer if flat.is_cuda else None
            res = quantizer.quantize_packed_dual(flat, mean=mean, hadamard_signs=rotate, token_sums=mean is not None, defer=defer)
            done = None
            if defer is not None:
                q, qt, finish = res
                done = _finish_beside(finish, flat.device)
            else:
                q, qt = res
            if getattr(qt, "token_sums", None) is not None:
                qt._row_sums = qt.token_sums
                if defer == "transposed":
                    qt._row_sums_event = done
        else:
            q, qt, defer, done = quantizer.quantize_packed(flat, mean=mean), None, None, None
        packed = PackedOperand(q, flat, quantizer, tensor.shape, rotate=rotate)
        packed._qt = qt
        packed.mean_event = mean_event
        if defer == "transposed":
            packed._qt_event = done
        elif defer == "rowmajor":
            packed._q_event = done
        return packed

    @staticmethod
    def _backward_centred() -> bool:
        """True when the output gradient is mean-centred before quantization (bitlinear.py:462-474)."""
        F = LinearLowbitFunction
        return bool(F.enable_backward_svd and F.backward_lowrank_svd > 0 and F.metis_mode == "mean")

    @staticmethod
    def _packed_backward_ok(grad_output: torch.Tensor) -> bool:
        """The packed backward covers direct quantization of the gradient and the mean mode."""
        F = LinearLowbitFunction
        mode_ok = (not F.enable_backward_svd) or F._backward_centred()
        return bool(mode_ok and not F.enable_nv_recipe and F._use_packed(grad_output, F.q_backward_outputgrad))

    @staticmethod
    def quantize_input(input_: torch.Tensor, mean_cache: dict = None, cache_key: str = "default"):
        """Quantized activation: a PackedOperand in packed mode, else the dequantized tensor
        (bitlinear.py:371-393)."""
        F = LinearLowbitFunction
        input_ = input_.to(F.compute_dtype)
        centred = F.enable_activation_svd
        if F._use_packed(input_, F.q_forward_input) and (not centred or F.metis_mode == "mean"):
            # with autograd recording, the weight-gradient product will want x quantized along the tokens
            return F._pack_centred(input_, F.q_forward_input, centred, mean_cache, cache_key,
                                   both=torch.is_grad_enabled(), defer="transposed" if F.defer_scale_pass else None)
        if centred:
            return F.svd_quant(input_, quant_func=F.q_forward_input, rank=F.activation_lowrank_svd,
                               niter=F.activation_lowrank_niter, broadcast_dim=F.activation_broadcast_dim,
                               tp_simulate=F.tp_simulate, tp_parts=F.tp_parts, metis_mode=F.metis_mode,
                               mean_cache=mean_cache, cache_key=cache_key)
        return F.q_forward_input.quantize_dequantize(input_)

    @staticmethod
    def _quantize_wgrad_operand(value: torch.Tensor, quantizer) -> torch.Tensor:
        """Dense QDQ of one weight-gradient operand; rotated only for the NV baseline
        (bitlinear.py:395-405).  The three-call sequence is kept because stubs override it."""
        F = LinearLowbitFunction
        if F.enable_nv_recipe:
            value = F._apply_hadamard_blocks(value, inverse=False)
        scalar = quantizer.get_scalar(value)
        value = quantizer.rquant(quantizer.quant(value, scalar), scalar)
        if F.enable_nv_recipe:
            value = F._apply_hadamard_blocks(value, inverse=True)
        return value

    # ---- forward / backward ----------------------------------------------------------------------------------------
    @staticmethod
    def forward(ctx, input_: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, quantized_weight,
                quantized_input):
        F = LinearLowbitFunction
        if quantized_input is None:
            quantized_input = F.quantize_input(input_, mean_cache=F.mean_cache, cache_key=F.mean_cache_key)
        xa, wq = quantized_input, quantized_weight
        packed = isinstance(xa, PackedOperand) and isinstance(wq, PackedOperand) \
            and _gemm_ok(xa.q.shape[0], wq.q.shape[0], xa.q.shape[1])
        ctx.packed = packed
        ctx.has_bias = bias is not None
        if packed:
            ctx.xa, ctx.wq = xa, wq
            ctx.save_for_backward(bias)
            rank1 = []
            if xa.mean is not None:
                rank1.append((None, ops.nvfp4_gemv(wq.q, xa.mean)))     # 1 (x) (mean @ Wq^T)
            if bias is not None:
                rank1.append((None, bias.float()))
            out_dtype = xa.dtype if xa.dtype in (torch.bfloat16, torch.float32) else torch.float32
            y = _packed_matmul(xa.rowmajor(), wq.q, rank1=rank1, out_dtype=out_dtype)
            xa.join_deferred()
            wq.join_deferred()
            return y.reshape(*xa.shape[:-1], wq.q.shape[0]).to(xa.dtype)
        # dense mode: the reference's wiring
        if isinstance(xa, PackedOperand):
            xa = xa.dense(F.compute_dtype)
        if isinstance(wq, PackedOperand):
            wq = wq.dense(weight.dtype)
        ctx.save_for_backward(xa, wq, bias)
        output = torch.matmul(xa, wq.T)
        if bias is not None:
            output += bias
        return output

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        F = LinearLowbitFunction
        grad_output = grad_output.to(F.compute_dtype)
        grad_bias = grad_output.sum(dim=(0, 1)) if ctx.has_bias else None
        d0, d1, d2 = grad_output.shape[0], grad_output.shape[1], grad_output.shape[2]   # 3-D, as the reference
        if ctx.packed:
            xa, wq = ctx.xa, ctx.wq
            M, N, K = d0 * d1, d2, xa.q.shape[1]
            if F._packed_backward_ok(grad_output) and _gemm_ok(M, K, N) and _gemm_ok(N, K, M):
                da = F._pack_centred(grad_output, F.q_backward_outputgrad, F._backward_centred(), both=True)
                grad_input, grad_weight = _packed_backward(da, xa, wq, M, N, K)
                grad_input = grad_input.reshape(d0, d1, K)
                grad_bias = grad_bias.to(torch.float32) if grad_bias is not None else None
                return grad_input, grad_weight, grad_bias, None, None
            # shapes or quantizers the packed backward does not take: continue densely
            input_, weight = xa.dense(F.compute_dtype), wq.dense(F.compute_dtype)
        else:
            input_, weight, _ = ctx.saved_tensors

        if F.enable_backward_svd:
            if F.backward_lowrank_svd > 0:
                grad_output = F.svd_quant(grad_output, quant_func=F.q_backward_outputgrad,
                                          rank=F.backward_lowrank_svd, niter=F.backward_lowrank_niter,
                                          broadcast_dim=F.backward_broadcast_dim, tp_simulate=F.tp_simulate,
                                          tp_parts=F.tp_parts, metis_mode=F.metis_mode)
                grad_t = grad_output.reshape(-1, d2).T
            else:
                ug, sg, vg = torch.linalg.svd(grad_output, full_matrices=False)
                us, vs = ug.abs().mean(), vg.abs().mean()
                q = F.q_backward_outputgrad
                grad_t = q(ug / us) @ torch.diag(sg) @ q(vg / vs)
                grad_t *= us * vs
        else:
            grad_t = F._quantize_wgrad_operand(grad_output, F.q_backward_outputgrad).reshape(-1, d2).T

        wgrad_input = input_
        if F.enable_nv_recipe:
            wgrad_input = F._quantize_wgrad_operand(input_, F.q_backward_input)
        grad_weight = torch.matmul(grad_t, wgrad_input.reshape(-1, wgrad_input.shape[-1]))
        grad_input = torch.matmul(grad_t.T.reshape(d0, d1, d2), weight)
        grad_weight = grad_weight.to(torch.float32)
        grad_bias = grad_bias.to(torch.float32) if grad_bias is not None else None
        return grad_input, grad_weight, grad_bias, None, None


_ONES = {}
_AUX_STREAMS = {}


def _finish_beside(finish, device, index=2):
    """Run the deferred scale pass of a dual quantization (ops.nvfp4_quantize_dual(defer=...)) on a stream kept
    for such passes (index 2: activations and gradients, 4: weights, which are quantized on the second stream and
    would otherwise hold up the activation's pass queued behind theirs), after everything issued so far on the
    current stream.  Returns the event that marks it done."""
    here, beside = torch.cuda.current_stream(device), _aux_stream(device, index)
    issued = torch.cuda.Event()
    issued.record(here)
    beside.wait_event(issued)
    with torch.cuda.stream(beside):
        finish()
        done = torch.cuda.Event()
        done.record(beside)
    return done


GROUP_BRANCHES = True     # forward_group: members of a projection group on streams of their own (rollout)
_BRANCH = 0          # which member of a projection group is being issued (forward_group): each has its own side streams


def _aux_stream(device: torch.device, index: int = 0) -> "torch.cuda.Stream":
    """A side stream of `device` for work that may overlap the current stream's.  Index 0: the low-rank branch and
    the mean's row vectors; 1: the mean row of the input gradient; 2, 4: deferred scale passes (activations and
    gradients, weights); 3: members of a projection group (forward_group); 5: the weights' quantization."""
    # the streams of deferred scale passes (2, 4) yield to everything else: their results are wanted last.  Not in a
    # data-parallel step: the collectives' kernel (default priority) would queue behind every side stream for the
    # SMs the capped GEMM leaves it
    priority = 0 if (index in (2, 4) or GRADIENT_REDUCER is not None) else -1
    key = (device, index, _BRANCH, priority)
    st = _AUX_STREAMS.get(key)
    if st is None:
        st = _AUX_STREAMS[key] = torch.cuda.Stream(device=device, priority=priority)
    return st


def critical_path_priority() -> int:
    """Priority for the stream a step is issued or captured on (see _aux_stream)."""
    return 0 if GRADIENT_REDUCER is not None else -1


def forward_group(layers, x: torch.Tensor):
    """[layer(x) for layer in layers] for projections that read the same activation (q/k/v, gate/up: the groups
    of bitlinear.py:676-702, which quantize that activation once).  At rollout sizes a member's forward is a chain
    of half a dozen kernels of a few microseconds each, far too small to fill the GPU, so without autograd the
    members are issued on streams of their own behind the shared quantization and run side by side (inside a
    captured graph: parallel branches).  Results are bit for bit those of the calls one after the other."""
    global _BRANCH
    layers = list(layers)
    parallel = (GROUP_BRANCHES and len(layers) > 1 and x.is_cuda and not torch.is_grad_enabled()
                and MetisFusedFunction.concurrent_branches and _BRANCH == 0 and all(isinstance(l, BitLinear) and l.is_svd_quant for l in layers))
    if not parallel:
        return [layer(x) for layer in layers]
    dev = x.device
    main = torch.cuda.current_stream(dev)
    if getattr(layers[0], "activation_group", None) is not None:
        LinearLowbitFunction.mean_cache = layers[0].mean_cache
        layers[0]._get_shared_quantized_input(x)      # a grouped activation is quantized here, once, in front of the fork
    fork = torch.cuda.Event()
    fork.record(main)
    outs = [None] * len(layers)
    try:
        for i in range(1, len(layers)):
            _BRANCH = i
            st = _aux_stream(dev, 3)
            st.wait_event(fork)
            with torch.cuda.stream(st):
                outs[i] = layers[i](x)
                done = torch.cuda.Event()
                done.record(st)
            outs[i].record_stream(main)
            outs[i] = (outs[i], done)
    finally:
        _BRANCH = 0
    outs[0] = layers[0](x)
    for i in range(1, len(layers)):
        y, done = outs[i]
        main.wait_event(done)
        outs[i] = y
    return outs


class _beside:
    """`with _beside(event, device) as join: ...` issues the body on the device's second stream once
    `event` has happened; `join(*tensors)` afterwards makes the current stream wait for it and hands
    the tensors over.  With event None the body simply runs on the current stream."""

    def __init__(self, event, device):
        self.event, self.device, self.ctx = event, device, None

    def __enter__(self):
        if self.event is None:
            return lambda *tensors: None
        self.main, self.aux = torch.cuda.current_stream(self.device), _aux_stream(self.device)
        self.aux.wait_event(self.event)
        self.ctx = torch.cuda.stream(self.aux)
        self.ctx.__enter__()

        def join(*tensors):
            self.main.wait_stream(self.aux)
            for t in tensors:
                if t is not None:
                    t.record_stream(self.main)
        return join

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


# fp4_post_b200.dp.GradientReducer installs itself here: the fused backward hands it every weight
# gradient the moment it is final (data-parallel training); None = single process.
GRADIENT_REDUCER = None


def _one(like: torch.Tensor) -> torch.Tensor:
    """A cached fp32 1.0 on the device of `like`."""
    t = _ONES.get(like.device)
    if t is None:
        t = _ONES[like.device] = torch.ones(1, dtype=torch.float32, device=like.device)
    return t


def _row_sums(q, rotate=None):
    """Sums over the tokens of the matrix a transposed quantization stands for, computed once per tensor (the
    activation's are needed by both weight-gradient products of a fused layer).  Of a rotated quantization
    (blocks b stored as y = H (s . b)): 1^T b = ((H s) / 16)^T y, a weighted row sum with period 16."""
    cached = getattr(q, "_row_sums", None)
    if cached is None:
        weights = None
        if rotate is not None:
            sgn = torch.tensor([-1.0 if (rotate >> i) & 1 else 1.0 for i in range(16)])
            h = LinearLowbitFunction._get_hadamard(16, "cpu", torch.float32)
            weights = ((h @ sgn) / 16.0).repeat(q.shape[1] // 16).to(q.device)
        cached = ops.nvfp4_gemv(q, weights)
        q._row_sums = cached
    else:
        done = getattr(q, "_row_sums_event", None)
        if done is not None:                        # computed on the second stream (_row_sums_beside)
            cur = torch.cuda.current_stream(cached.device)
            cur.wait_event(done)
            cached.record_stream(cur)
    return cached


def _row_sums_beside(op: "PackedOperand"):
    """The token sums of an activation's transposed quantization are needed by the backward pass only: issue
    them on the second stream, after what the current stream has queued so far (the quantization), so that
    they run in the shadow of the forward products instead of in front of the backward ones."""
    x_t = op.transposed()
    if getattr(x_t, "_row_sums", None) is not None:
        return
    dev = x_t.codes.device
    main, aux = torch.cuda.current_stream(dev), _aux_stream(dev)
    queued = torch.cuda.Event()
    queued.record(main)
    aux.wait_event(queued)
    with torch.cuda.stream(aux):
        _row_sums(x_t, op.rotate)
        done = torch.cuda.Event()
        done.record(aux)
    x_t._row_sums_event = done


def _packed_dx(da: PackedOperand, wq: PackedOperand, out_dtype, addend=None, side=None, mean_row=None, sm_limit=0):
    """dX = D^ @ W^ on the FP4 GEMM (bitlinear.py:508): contraction over N, so A = Q(D) [M, N] and
    B = W quantized along N ([K, N], transposed quantizer), plus the row vector mu_D @ W^.
    `side` = (T, U, row_vec) adds a bf16 rank-r product T @ U^T (in this product's accumulator
    units) and another row vector in the same launch."""
    w_t = wq.transposed()                                   # [K, N]
    row = mean_row
    if row is None and da.mean is not None:
        row = ops.nvfp4_gemv(w_t, da.mean)
    lowrank = None
    if side is not None:
        t_acc, u, extra = side
        lowrank = (t_acc, u)
        if extra is not None:
            row = extra if row is None else row + extra
    rank1 = [(None, row)] if row is not None else []
    return _packed_matmul(da.rowmajor(), w_t, rank1=rank1, lowrank=lowrank, c=addend, out_dtype=out_dtype, sm_limit=sm_limit)


def _packed_dw(da: PackedOperand, xa: PackedOperand, M: int, out_dtype=torch.float32, sm_limit=0):
    """dW = D^T @ x^ on the FP4 GEMM (bitlinear.py:502-505), fp32 unless told otherwise: contraction over tokens, so
    A = Q(D)^T [N, M] and B = Q(x)^T [K, M], both from the transposed quantizer, plus the two
    rank-1 terms of  dW = Qd^T Qx + (Qd^T 1) mu_x^T + mu_D (Qx^T 1 + M mu_x)^T."""
    d_t = da.transposed()                                   # [N, M], col_vec = mu_D
    x_t = xa.transposed()                                   # [K, M], col_vec = mu_x
    if da.rotate != xa.rotate:
        raise RuntimeError("the two operands of a weight-gradient product must be rotated alike")
    rank1 = []
    mu_x, mu_d = x_t.col_vec, d_t.col_vec
    if mu_x is not None:
        rank1.append((_row_sums(d_t, da.rotate), mu_x))
    if mu_d is not None:
        tail = _row_sums(x_t, xa.rotate)
        if mu_x is not None:
            tail = torch.add(tail, mu_x, alpha=float(M))          # one kernel: Qx^T 1 + M mu_x
        rank1.append((mu_d, tail))
    # rotated operands: (H s)^T (H s) = 16 I
    return ops.nvfp4_gemm(d_t, x_t, rank1=rank1, out_dtype=out_dtype, sm_limit=sm_limit, alpha=1.0 / 16 if da.rotate is not None else 1.0)


def _grad_dtype(param: torch.Tensor):
    """The reference hands autograd an fp32 weight gradient (bitlinear.py:510), which autograd casts to the
    parameter's dtype.  For a bf16 parameter the product is rounded to bf16 in its own epilogue instead:
    the same single rounding of the fp32 sum, without a 4-byte round trip through memory."""
    return torch.bfloat16 if param.dtype == torch.bfloat16 else torch.float32


def _packed_backward(da: PackedOperand, xa: PackedOperand, wq: PackedOperand, M: int, N: int, K: int, addend=None):
    """Both backward products of one quantized linear, with D^ = 1 mu_D^T + Q(D - mu_D) and
    x^ = 1 mu_x^T + Q(x - mu_x)."""
    out_dtype = xa.dtype if xa.dtype in (torch.bfloat16, torch.float32) else torch.float32
    return _packed_dx(da, wq, out_dtype, addend=addend), _packed_dw(da, xa, M)


class LinearLowbit(torch.nn.Module):
    """Linear layer whose weight and input are quantized on the fly (bitlinear.py:515-595)."""

    def __init__(self, in_features: int, out_features: int, bias=True, args=None, device=None,
                 storage_dtype=torch.float32, compute_dtype=torch.float32) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.storage_dtype = storage_dtype
        self.compute_dtype = compute_dtype
        self.cache_quantized_weight = getattr(args, "cache_quantized_weight", False)
        self._quantized_weight_cache = None
        where = args.device if device is None else device
        self.weight = torch.nn.Parameter(torch.empty((out_features, in_features), dtype=storage_dtype, device=where))
        self.bias = torch.nn.Parameter(torch.empty((out_features,), dtype=storage_dtype, device=where)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            init.uniform_(self.bias, -bound, bound)

    def forward(self, input, quantized_input=None):
        weight_compute = self.weight.to(self.compute_dtype)
        bias_compute = self.bias.to(self.compute_dtype) if self.bias is not None else None
        quantized_weight = self._get_quantized_weight(weight_compute)
        return LinearLowbitFunction.apply(input, weight_compute, bias_compute, quantized_weight, quantized_input)

    def _get_quantized_weight(self, weight_compute):
        """Quantized weight with a one-entry cache keyed on the parameter version.  In packed
        mode the entry is a PackedOperand (codes + scales and the transposed quantization: made in
        the same pass when autograd is recording, on demand otherwise), otherwise the dequantized
        tensor."""
        training = torch.is_grad_enabled()
        with torch.no_grad():
            return self._quantized_weight(weight_compute, training)

    def _quantized_weight(self, weight_compute, training):
        F = LinearLowbitFunction
        packed = F._use_packed(weight_compute, F.q_forward_weight) and not F.enable_nv_recipe
        cache_key = (self.weight._version, weight_compute.device, weight_compute.dtype, F.q_forward_weight,
                     F.enable_nv_recipe, packed)
        if self.cache_quantized_weight and self._quantized_weight_cache is not None:
            cached_key, cached_weight = self._quantized_weight_cache
            if cached_key == cache_key:
                if isinstance(cached_weight, PackedOperand):
                    cached_weight.fresh = False      # quantized in an earlier call: long since complete
                return cached_weight
        if packed:
            source = weight_compute.detach()
            done = None
            if training and _dual_ok(source):        # the input-gradient product contracts over the other dimension
                if F.defer_scale_pass and not self.cache_quantized_weight:
                    # only the backward reads the transposed quantization: its scale pass leaves the forward's path
                    q, qt, finish = F.q_forward_weight.quantize_packed_dual(source, defer="transposed")
                    done = _finish_beside(finish, source.device, index=4)
                else:
                    q, qt = F.q_forward_weight.quantize_packed_dual(source)
            else:
                q, qt = F.q_forward_weight.quantize_packed(source), None
            quantized_weight = PackedOperand(q, source, F.q_forward_weight, source.shape)
            quantized_weight._qt = qt
            quantized_weight._qt_event = done
        else:
            quant_input = weight_compute
            if F.enable_nv_recipe:
                quant_input = F._apply_hadamard_blocks(quant_input, inverse=False)
            quantized_weight = F.q_forward_weight.quantize_dequantize(quant_input)
            if F.enable_nv_recipe:
                quantized_weight = F._apply_hadamard_blocks(quantized_weight, inverse=True)
        if self.cache_quantized_weight:
            self._quantized_weight_cache = (cache_key, quantized_weight)
        return quantized_weight

    def _apply(self, fn, recurse=True):
        self._quantized_weight_cache = None
        return super()._apply(fn, recurse=recurse)


# -----------------------------------------------------------------------------
# fused low-rank + residual product (packed mode of BitLinear.forward)
# -----------------------------------------------------------------------------
class MetisFusedFunction(torch.autograd.Function):
    """y = U (s . (x^ Vq^T)) + x^ Rq^T + b as ONE autograd node on the FP4 GEMM.

    Forward: one small FP4 GEMM gives Yv = x^ Vq^T [M, r]; the residual GEMM then adds the
    bf16 rank-r product (s . Yv) U^T inside the same tensor-memory accumulator, plus the mean and
    bias row vectors in its epilogue.  Backward reproduces, node by node, what autograd derives
    for the reference's chain vlinear -> s -> ulinear -> + warmup_linear (bitlinear.py:752-760):
    ulinear is a plain (unquantized) linear, vlinear and warmup_linear use the quantized
    backward of LinearLowbitFunction."""

    fuse_dx_side_product = True      # bf16 only; False keeps the two dX products as separate launches
    native_lowrank_backward = True   # bf16 only; False leaves the unquantized U branch's backward to torch.matmul
    concurrent_branches = True       # backward of the low-rank branch on a second CUDA stream

    @staticmethod
    def forward(ctx, x, xa: PackedOperand, v_weight, vq: PackedOperand, s, u_weight, r_weight,
                rq: PackedOperand, bias):
        M, K = xa.q.shape
        N = rq.q.shape[0]
        act = xa.dtype if xa.dtype in (torch.bfloat16, torch.float32) else torch.float32
        rank1_v, rank1_r = [], []
        join_residual = None

        def ready(op):
            if op.ready_event is not None:             # quantized on another stream: order this stream after it, once
                torch.cuda.current_stream(xa.q.device).wait_event(op.ready_event)
                op.ready_event = None
        if xa.mean is not None:
            # mu_x V^T and mu_x R^T need the mean only: on the second stream they run beside the
            # quantization of x instead of after it
            # (weights from the cache, or quantized on the second stream itself: fresh ones made on this
            # stream are still being quantized here)
            beside = vq.ready_event is not None and rq.ready_event is not None
            overlap = MetisFusedFunction.concurrent_branches and (beside or (not vq.fresh and not rq.fresh))
            if not overlap:
                ready(vq)
                ready(rq)
            with _beside(xa.mean_event if overlap else None, xa.mean.device) as join:
                if overlap and vq.ready_event is not None:      # quantized on a stream of their own: order this one after each
                    torch.cuda.current_stream(xa.mean.device).wait_event(vq.ready_event)
                row_v = ops.nvfp4_gemv(vq.q, xa.mean)
                # the product with V needs only this one: the pass over the (much larger) residual
                # weight stays off the critical path until the residual product
                v_ready = torch.cuda.Event() if overlap else None
                if v_ready is not None:
                    v_ready.record()
                if overlap and rq.ready_event is not None:
                    torch.cuda.current_stream(xa.mean.device).wait_event(rq.ready_event)
                row_r = ops.nvfp4_gemv(rq.q, xa.mean)
            if v_ready is not None:
                torch.cuda.current_stream(xa.mean.device).wait_event(v_ready)
                row_v.record_stream(torch.cuda.current_stream(xa.mean.device))
                join_residual = lambda: join(row_r)
            rank1_v.append((None, row_v))
            rank1_r.append((None, row_r))
        if bias is not None:
            rank1_r.append((None, bias.float()))
        ready(vq)
        yv = _packed_matmul(xa.q, vq.q, rank1=rank1_v, out_dtype=act)                 # [M, r]
        # torch.mul(self.s, y), in the units the side product accumulates in: 1/(unit_x * unit_R)
        if act == torch.bfloat16:
            lowrank = (ops.lowrank_scale(yv, s, xa.q.unit, rq.q.unit), u_weight.detach().to(torch.bfloat16))
        else:
            ts = yv * s.to(act)
            lowrank = _bf16_factors(ts.float() / (xa.q.unit * rq.q.unit), u_weight.detach(), act)
        if join_residual is not None:
            join_residual()
        ready(rq)
        y = _packed_matmul(xa.q, rq.q, rank1=rank1_r, lowrank=lowrank, out_dtype=act)
        if (MetisFusedFunction.concurrent_branches and xa.q.codes.is_cuda and any(ctx.needs_input_grad)
                and xa._qt is not None and LinearLowbitFunction._backward_centred()):
            _row_sums_beside(xa)        # queued behind the product: it runs as that one drains, not in front of it
        for op in (xa, vq, rq):         # scale passes left to another stream have long finished; this joins that stream
            op.join_deferred()
        ctx.xa, ctx.vq, ctx.rq = xa, vq, rq
        ctx.has_bias = bias is not None
        ctx.dims = (M, N, K)
        ctx.v_weight, ctx.r_weight = v_weight, r_weight        # for their dtypes, and for a reducer that fills .grad itself
        ctx.s_param, ctx.u_param = s, u_weight
        ctx.save_for_backward(yv, s, u_weight)
        return y.reshape(*xa.shape[:-1], N).to(xa.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        F = LinearLowbitFunction
        yv, s, u_weight = ctx.saved_tensors
        xa, vq, rq = ctx.xa, ctx.vq, ctx.rq
        v_weight, r_weight = ctx.v_weight, ctx.r_weight
        M, N, K = ctx.dims
        r = yv.shape[1]
        act = yv.dtype
        g = grad_output.reshape(M, N).to(act)
        grad_bias = g.sum(dim=0).to(torch.float32) if ctx.has_bias else None
        centred = F._backward_centred()
        quantizer = F.q_backward_outputgrad
        reducer = GRADIENT_REDUCER
        # a collective of a layer further up may still be running: leave its kernel some SMs
        busy_limit = reducer.gemm_sm_limit(g.device) if reducer is not None and reducer.pending() else 0

        fuse_dx = MetisFusedFunction.fuse_dx_side_product and act == torch.bfloat16 and r <= 256

        def low_rank_branch(before_weight_gradient=None):
            # ulinear: plain linear on ts = s . yv; vlinear: quantized backward with grad_output = d_yv
            v_t = u_side = None
            if fuse_dx:
                # operand of the bf16 side product of the fused dX launch; it needs nothing of this pass
                v_t = vq.transposed()
                u_side = ops.nvfp4_dequantize(v_t, torch.bfloat16, add_mean=False, unit=_one(v_t.unit))
            if act == torch.bfloat16 and g.is_cuda and r % 8 == 0 and N % 8 == 0 and MetisFusedFunction.native_lowrank_backward:
                # autograd's bf16 ops on the tensor core, one pass over g per product and no transposed copy:
                # dU = g^T ts, then d_ts = g U with d_yv = d_ts . s and ds = sum d_ts . yv in its finishing pass
                one = _one(yv)
                ts = ops.lowrank_scale(yv, s, one, one)
                out_dtype = u_weight.dtype if u_weight.dtype in (torch.bfloat16, torch.float32) else torch.float32
                grad_u = ops.lowrank_du(g, ts, out_dtype=out_dtype).to(u_weight.dtype)
                d_yv, ds32 = ops.lowrank_dts(g, u_weight.detach().to(torch.bfloat16), yv, s)
                grad_s = ds32.to(s.dtype)
            else:
                ts = yv * s.to(act)
                u = u_weight.to(act)
                grad_u = (g.T @ ts).to(u_weight.dtype)
                d_ts = g @ u                                                            # [M, r]
                grad_s = (d_ts * yv).sum(dim=0).to(s.dtype)
                d_yv = d_ts * s.to(act)
            dv = F._pack_centred(d_yv, quantizer, centred, both=True)
            side = None
            if fuse_dx:
                side = (u_side, ops.nvfp4_gemv(v_t, dv.mean) if dv.mean is not None else None)
            # Single process: the input-gradient product is the last big launch and nothing waits for this branch's
            # own weight gradient, so its operands go first.  With a gradient reducer the small gradients' collective
            # should start before that product, in whose shadow it runs: the weight gradient goes first.
            early = before_weight_gradient is not None and reducer is None
            if early:
                before_weight_gradient(dv)
            grad_v = _packed_dw(dv, xa, M, _grad_dtype(v_weight), sm_limit=busy_limit)
            if before_weight_gradient is not None and not early:
                before_weight_gradient(dv)
            return grad_u, grad_s, dv, grad_v, side

        def residual_weight_gradient(dg):
            # warmup_linear (the residual): quantized backward with grad_output = g
            grad_r = _packed_dw(dg, xa, M, _grad_dtype(r_weight), sm_limit=busy_limit)
            if reducer is not None:
                if reducer.across_layers:
                    reducer.adopt(r_weight, grad_r)
                else:
                    reducer.ready(grad_r)   # the big all-reduce starts here and runs beside the dX product
            return grad_r

        def side_operand(dv, dg):
            # D^v in the units the fused dX launch accumulates in.  e2m1 x e4m3 is exact in bf16; the ratio of the
            # two products' units goes into T, rounded once to bf16 (the unfused dX_v would be rounded there too).
            ratio = (dv.q.unit * vq.transposed().unit) / (dg.rowmajor().unit * rq.transposed().unit)
            return ops.nvfp4_dequantize(dv.q, torch.bfloat16, add_mean=False, unit=ratio)

        mean_row = t_acc = None
        concurrent = MetisFusedFunction.concurrent_branches and g.is_cuda
        if concurrent:
            # The low-rank branch is a dozen small kernels that leave most of the GPU idle; on a second
            # stream they run in the shadow of the residual branch's quantizers and weight-gradient
            # GEMM.  Both branches contract over the transposed activation: made once, before the fork.
            x_t = xa.transposed()
            if centred and getattr(x_t, "_row_sums", None) is None:
                _row_sums(x_t, xa.rotate)   # cached on x_t and read by both branches
            main, aux = torch.cuda.current_stream(), _aux_stream(g.device)
            aux.wait_stream(main)
            # the weight-gradient product comes first and reads the transposed output only
            dg = F._pack_centred(g, quantizer, centred, both=True, defer="rowmajor" if F.defer_scale_pass else None)
            dg_done = torch.cuda.Event()
            dg_done.record(main)
            for_dx = {}

            if dg.mean is not None:
                # mu_D R^ for the input gradient needs the mean of g only: a pass over the residual weight that
                # belongs to neither chain, so it gets a stream of its own and runs wherever there is room
                third = _aux_stream(g.device, 1)
                third.wait_event(dg.mean_event)
                with torch.cuda.stream(third):
                    mean_row = ops.nvfp4_gemv(rq.transposed(), dg.mean)
                    mean_row_done = torch.cuda.Event()
                    mean_row_done.record(third)

            def input_gradient_operands(dv):
                # What the input-gradient product needs from this stream goes out ahead of this branch's own
                # weight gradient, which nothing on the other stream waits for until the very end.
                if fuse_dx:
                    aux.wait_event(dg_done)                # the unit of Q(g)
                    for_dx["t_acc"] = side_operand(dv, dg)
                for_dx["ready"] = torch.cuda.Event()
                for_dx["ready"].record(aux)

            with torch.cuda.stream(aux), random_lane(1):
                grad_u, grad_s, dv, grad_v, side = low_rank_branch(input_gradient_operands)
            grad_r = residual_weight_gradient(dg)
            main.wait_event(for_dx["ready"])
            t_acc = for_dx.get("t_acc")
            if mean_row is not None:
                main.wait_event(mean_row_done)
            # allocated on the second stream, read by kernels (or by autograd) on this one: the allocator must
            # not hand their memory to the next second-stream allocation while this stream still uses it
            handed_over = [mean_row, t_acc, dv.q.codes, dv._qt.codes if dv._qt is not None else None]
            if side is not None:
                handed_over += [side[0], side[1]]
            for t in handed_over:
                if t is not None:
                    t.record_stream(main)
        else:
            grad_u, grad_s, dv, grad_v, side = low_rank_branch()
            dg = F._pack_centred(g, quantizer, centred, both=True)
            grad_r = residual_weight_gradient(dg)

        def small_gradients():
            if concurrent:
                main.wait_stream(aux)                           # the low-rank branch's own gradients
                for t in (grad_u, grad_s, grad_v):
                    if t is not None:
                        t.record_stream(main)
            if reducer is not None:
                # the small gradients are final too: their bucket goes out before the input-gradient GEMM
                if reducer.across_layers:
                    for prm, t in ((v_weight, grad_v), (ctx.s_param, grad_s), (ctx.u_param, grad_u)):
                        reducer.adopt(prm, t)
                    reducer.ready(grad_bias)
                else:
                    for t in (grad_v, grad_s, grad_u, grad_bias):
                        reducer.ready(t)
                reducer.start_small()

        if reducer is not None:
            small_gradients()
        # with a gradient all-reduce in flight the input-gradient GEMM leaves it some SMs
        sm_limit = reducer.gemm_sm_limit(g.device) if reducer is not None else 0
        if fuse_dx:
            # dX of both branches in ONE launch: D^v @ V^ enters the residual product as a bf16 rank-r side product
            u_side, extra = side
            if t_acc is None:
                t_acc = side_operand(dv, dg)
            gx = _packed_dx(dg, rq, act, side=(t_acc, u_side, extra), mean_row=mean_row, sm_limit=sm_limit)
        else:
            gx_v = _packed_dx(dv, vq, act, sm_limit=sm_limit)
            gx = _packed_dx(dg, rq, act, addend=gx_v, mean_row=mean_row, sm_limit=sm_limit)          # summed in the epilogue
        if reducer is None:
            small_gradients()
        grad_x = gx.reshape(xa.shape)
        if reducer is not None and reducer.across_layers and reducer.active():
            # the gradients sit in .grad already; the wait for their collectives moves to the end of the pass
            reducer.finish_at_end_of_backward()
            return grad_x, None, None, None, None, None, None, None, grad_bias
        if reducer is not None:
            reducer.flush()
        return grad_x, None, grad_v, None, grad_s, grad_u, grad_r, None, grad_bias


class BitLinear(nn.Module):
    """Drop-in replacement of nn.Linear: W = U diag(s) V + R with V and R in NVFP4
    (reference: bitlinear.py:597-940)."""
    rollout_merge_active = False

    def __init__(self, in_features, out_features, args=None, bias=True, dtype=torch.float32, compute_dtype=None):
        super().__init__()
        self.storage_dtype = dtype
        self.compute_dtype = compute_dtype if compute_dtype is not None else dtype
        if self.compute_dtype not in [torch.float32, torch.float16, torch.bfloat16]:
            raise ValueError(f"Unsupported compute_dtype: {self.compute_dtype}")

        if args.enable_forward_svd == False and args.enable_lowbit == True:  # noqa: E712 (as the reference)
            if args.enable_te:
                raise RuntimeError("enable_te needs transformer_engine, which this build does not use")
            self.warmup_linear = LinearLowbit(in_features, out_features, bias=bias, args=args,
                                              storage_dtype=self.storage_dtype, compute_dtype=self.compute_dtype)
        else:
            self.warmup_linear = nn.Linear(in_features, out_features, bias=bias, device=args.device, dtype=self.storage_dtype)
            init.kaiming_uniform_(self.warmup_linear.weight, a=math.sqrt(5))
            if bias:
                fan_in, _ = init._calculate_fan_in_and_fan_out(self.warmup_linear.weight)
                bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
                init.uniform_(self.warmup_linear.bias, -bound, bound)

        self.ulinear = None
        self.vlinear = None
        self.s = None

        # process-global configuration: the last constructed layer wins (bitlinear.py:634-661)
        F = LinearLowbitFunction
        F.q_forward_input = quant_func[args.q_forward_input]
        F.q_forward_weight = quant_func[args.q_forward_weight]
        compile_qdq = getattr(args, "compile_qdq", False)
        F.q_forward_input.compile_quantize_dequantize = compile_qdq
        F.q_forward_weight.compile_quantize_dequantize = compile_qdq
        F.q_backward_input = quant_func[args.q_backward_input]
        F.q_backward_weight = quant_func[args.q_backward_weight]
        F.q_backward_outputgrad = quant_func[args.q_backward_outputgrad]
        F.enable_backward_svd = args.enable_backward_svd
        F.backward_lowrank_svd = args.backward_lowrank_svd
        F.backward_lowrank_niter = args.backward_lowrank_niter
        F.enable_activation_svd = args.enable_activation_svd
        F.activation_lowrank_svd = args.activation_lowrank_svd
        F.activation_lowrank_niter = args.activation_lowrank_niter
        F.activation_broadcast_dim = args.activation_broadcast_dim
        F.backward_broadcast_dim = args.backward_broadcast_dim
        F.enable_nv_recipe = args.enable_nv_recipe
        F.hadamard_workspace_mb = getattr(args, "hadamard_workspace_mb", 128)
        F.hadamard_tile_size = getattr(args, "hadamard_tile_size", 16)
        F.hadamard_backend = getattr(args, "hadamard_backend", "auto")
        F.tp_simulation = args.tp_simulation      # sic: the reference writes tp_simulation and reads tp_simulate
        F.tp_parts = args.tp_parts
        F.compute_dtype = self.compute_dtype
        F.metis_mode = args.metis_mode
        F.gemm_mode = getattr(args, "gemm_mode", "packed")

        self.args = args
        self.is_svd_quant = False
        if args.forward_svd_warmup_steps <= 0 and args.enable_forward_svd:
            print("split")
            self.split()

        self.mean_cache = {}
        self.activation_group = None
        self._merged_rollout_weight_cache = None
        self.layer_name = ""

    # ---- shared quantized activation (bitlinear.py:676-702) ------------------------------------------------
    def _get_shared_quantized_input(self, x: torch.Tensor):
        group = getattr(self, "activation_group", None)
        if group is None:
            return LinearLowbitFunction.quantize_input(x, mean_cache=self.mean_cache,
                                                       cache_key=f"{self.layer_name}.shared")
        ref = group.get("input_ref")
        if ref is not None and ref() is x:
            return group["quantized_input"]
        quantized = LinearLowbitFunction.quantize_input(x, mean_cache=group["mean_cache"],
                                                        cache_key=f"{group['name']}.shared")

        def forget(dead):
            if group.get("input_ref") is dead:
                group["input_ref"] = None
                group["quantized_input"] = None

        group["input_ref"] = weakref.ref(x, forget)
        group["quantized_input"] = quantized
        return quantized

    # ---- merged weight for rollout (bitlinear.py:704-730) -------------------------------------------------------
    @torch.no_grad()
    def _get_merged_rollout_weight(self, dtype: torch.dtype) -> torch.Tensor:
        F = LinearLowbitFunction
        cache_key = (self.vlinear.weight._version, self.ulinear.weight._version, self.s._version,
                     self.warmup_linear.weight._version, self.vlinear.weight.device, dtype,
                     F.q_forward_weight, F.enable_nv_recipe)
        if self._merged_rollout_weight_cache is not None:
            cached_key, cached_weight = self._merged_rollout_weight_cache
            if cached_key == cache_key:
                return cached_weight

        def dense(w):
            return w.dense(dtype) if isinstance(w, PackedOperand) else w

        v_weight = dense(self.vlinear._get_quantized_weight(self.vlinear.weight.to(dtype)))
        residual = dense(self.warmup_linear._get_quantized_weight(self.warmup_linear.weight.to(dtype)))
        merged = (self.ulinear.weight.to(dtype) * self.s.to(dtype).unsqueeze(0)) @ v_weight + residual
        self._merged_rollout_weight_cache = (cache_key, merged)
        return merged

    def _apply(self, fn, recurse=True):
        self._merged_rollout_weight_cache = None
        return super()._apply(fn, recurse=recurse)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        F = LinearLowbitFunction
        F.mean_cache = self.mean_cache
        if not self.is_svd_quant:
            return self.warmup_linear(x)

        share_activation = (isinstance(self.vlinear, LinearLowbit) and isinstance(self.warmup_linear, LinearLowbit)
                            and self.args.forward_svd_rank > 0)
        if share_activation:
            self._quantize_weights_beside(x)
            shared = self._get_shared_quantized_input(x)
            if isinstance(shared, PackedOperand):
                fused = self._forward_packed(x, shared)
                if fused is not None:
                    return fused
            if BitLinear.rollout_merge_active and not torch.is_grad_enabled():
                dense_in = shared.dense(F.compute_dtype) if isinstance(shared, PackedOperand) else shared
                y = torch.matmul(dense_in, self._get_merged_rollout_weight(dense_in.dtype).T)
                if self.warmup_linear.bias is not None:
                    y = y + self.warmup_linear.bias.to(y.dtype)
                return y
            y = self.vlinear(x, quantized_input=shared)
        else:
            F.mean_cache_key = f"{self.layer_name}.vlinear"
            y = self.vlinear(x)
        y = torch.mul(self.s, y)
        y = self.ulinear(y)
        if self.args.forward_svd_rank > 0:
            if share_activation:
                y = y + self.warmup_linear(x, quantized_input=shared)
            else:
                F.mean_cache_key = f"{self.layer_name}.warmup"
                y = y + self.warmup_linear(x)
        return y

    def _quantize_weights_beside(self, x):
        """With the weight cache off (the reference's default) every forward quantizes V and R again.
        That work does not depend on x: it is issued on the device's second stream, where it runs
        beside the column mean and the quantization of the activation instead of after them.  The
        operands remember the event the current stream has to wait for before it reads them."""
        F = LinearLowbitFunction
        self._prefetched = None
        v, w = self.vlinear, self.warmup_linear
        if not (MetisFusedFunction.concurrent_branches and x.is_cuda and v.weight.is_cuda
                and F._use_packed(v.weight, F.q_forward_weight) and not F.enable_nv_recipe):
            return
        if v.cache_quantized_weight and w.cache_quantized_weight and v._quantized_weight_cache is not None \
                and w._quantized_weight_cache is not None:
            return                                        # (probably) cache hits: nothing to overlap
        # a stream of their own (not the one the mean's row vectors run on: those would queue behind the residual
        # weight's quantization although the first of them needs V only)
        main, aux = torch.cuda.current_stream(x.device), _aux_stream(x.device, 5)
        aux.wait_stream(main)
        with torch.cuda.stream(aux):
            # the small one first: the product with V is the first consumer on the forward's critical path
            vq = v._get_quantized_weight(v.weight.to(v.compute_dtype))
            v_done = torch.cuda.Event()
            v_done.record(aux)
            rq = w._get_quantized_weight(w.weight.to(w.compute_dtype))
            r_done = torch.cuda.Event()
            r_done.record(aux)
        for op, done in ((vq, v_done), (rq, r_done)):
            if isinstance(op, PackedOperand) and op.fresh:
                op.ready_event = done
                for q in (op.q, op._qt):
                    if q is not None:
                        q.codes.record_stream(main)      # one allocation holds codes, scales and unit
        self._prefetched = (vq, rq)

    def _forward_packed(self, x, shared: PackedOperand):
        """Packed mode of the shared-activation branch: both weights as PackedOperand, one fused
        autograd node.  Also serves rollout (no merged bf16 weight is needed: the FP4 weights are
        a quarter of its bytes).  Returns None when a shape does not fit the FP4 GEMM."""
        v, w = self.vlinear, self.warmup_linear
        if getattr(self, "_prefetched", None) is not None:
            vq, rq = self._prefetched
            self._prefetched = None
        else:
            vq = v._get_quantized_weight(v.weight.to(v.compute_dtype))
            rq = w._get_quantized_weight(w.weight.to(w.compute_dtype))
        if not (isinstance(vq, PackedOperand) and isinstance(rq, PackedOperand)):
            return None
        M, K = shared.q.shape
        r, N = vq.q.shape[0], rq.q.shape[0]
        if not (_gemm_ok(M, N, K) and r % 16 == 0 and r <= 256):
            return None
        if torch.is_grad_enabled():
            # the backward products contract over M, N and r and quantize the gradients natively
            if not (M % 32 == 0 and N % 32 == 0 and r % 32 == 0 and _backward_can_pack(shared)):
                return None
        bias = w.bias.to(w.compute_dtype) if w.bias is not None else None
        return MetisFusedFunction.apply(x, shared, v.weight, vq, self.s, self.ulinear.weight, w.weight, rq, bias)

    @staticmethod
    def _init_telinear(w, weight):
        torch.nn.init.ones_(weight)
        weight.mul_(w)

    @torch.no_grad()
    def split(self):
        """One-time W -> U diag(s) V + R by exact fp32 SVD (bitlinear.py:776-924).  Works on any
        device (the reference hard-codes .cuda())."""
        args = self.args
        if not args.enable_forward_svd:
            return
        if self.vlinear is not None:
            u, s, v = torch.linalg.svd(self.ulinear.weight @ torch.diag(self.s) @ self.vlinear.weight, full_matrices=False)
            bias = self.ulinear.bias
            device = self.ulinear.weight.device
            original_dtype = self.ulinear.weight.dtype
        else:
            w = self.warmup_linear.weight
            device, original_dtype = w.device, w.dtype
            u, s, v = torch.linalg.svd(w.to(torch.float32), full_matrices=False)
            u, s, v = (t.to(device=device, dtype=original_dtype) for t in (u, s, v))
            bias = self.warmup_linear.bias.to(device=device) if self.warmup_linear.bias is not None else None
            rank = args.forward_svd_rank
            if rank > 0:
                residual = w - u[:, :rank] @ torch.diag(s[:rank]) @ v[:rank]
                self.warmup_linear = LinearLowbit(w.shape[1], w.shape[0], bias=bias is not None, args=args,
                                                  device=device, storage_dtype=original_dtype,
                                                  compute_dtype=self.compute_dtype)
                if bias is not None:
                    self.warmup_linear.bias.copy_(bias)
                self.warmup_linear.weight.copy_(residual)

        rank = args.forward_svd_rank
        if args.enable_lowbit:
            if args.enable_te:
                raise RuntimeError("enable_te needs transformer_engine, which this build does not use")
            keep = rank if rank > 0 else v.shape[0]
            self.vlinear = LinearLowbit(v.shape[1], keep, bias=False, args=args, device=device,
                                        storage_dtype=original_dtype, compute_dtype=self.compute_dtype)
            # the reference leaves ulinear at the default dtype/device; allocating it beside the
            # weights saves a later .to() and is invisible to callers
            self.ulinear = nn.Linear(keep, u.shape[0], bias=False, device=device, dtype=original_dtype)
            self.vlinear.weight.copy_(v[:keep, :])
            self.ulinear.weight.copy_(u[:, :keep])
        else:
            self.vlinear = nn.Linear(v.shape[1], v.shape[0], bias=False)
            self.ulinear = nn.Linear(u.shape[1], u.shape[0])
            self.vlinear.weight = nn.Parameter(v)
            self.ulinear.weight = nn.Parameter(u)
            if bias is not None:
                self.ulinear.bias = nn.Parameter(bias.clone())

        self.is_svd_quant = True
        if rank > 0:
            self.s = torch.nn.Parameter(s[:rank].clone())
        else:
            self.s = torch.nn.Parameter(s)
            self.warmup_linear = None

    @torch.no_grad()
    def lowrank_initialization(self, rank: int = 32):
        """Replace the weight by its best rank-`rank` approximation (bitlinear.py:926-940)."""
        W = self.warmup_linear.weight
        r = max(1, min(int(rank), min(W.shape)))
        U, S, Vh = torch.linalg.svd(W.detach().to(torch.float32), full_matrices=False)
        W.copy_(((U[:, :r] * S[:r]) @ Vh[:r, :]).to(dtype=W.dtype, device=W.device))
        print(f"[lowrank_init] shape={tuple(W.shape)}  rank={r}")
