"""Quantizer classes of the Metis layer, API-compatible with the reference's
src/Metis/Metis/quant.py (the `QuantFunc` protocol: classmethods get_scalar / quant / rquant /
quantize_dequantize, the `quant_func` registry with the same 11 keys, the compile flag and
`nvfp4_nosr_qdq_compile_status`).

The two NVFP4 block quantizers -- `Cast2NVFp4e2m1BlockNOSR` (round to nearest, quant.py:390-548)
and `Cast2NVFp4e2m1Block` (stochastic rounding, quant.py:273-388) -- run on hand-written sm_100a
kernels through the C ABI and additionally expose `quantize_packed`, which returns real packed
FP4 (codes, E4M3 scales, unit) for the tensor-core GEMM.  They need CUDA tensors; there is no CPU
fallback.  Every other format is outside the accelerated path and is kept as a small pure-torch
class so that registry keys still resolve and stub subclasses (as the reference's tests build
them from `Cast2Fp32`) keep working on any device.
"""
from __future__ import annotations

import torch

from fp4_post_b200 import cabi, ops

_BLOCK = 16


# ---- protocol base ---------------------------------------------------------------------------------

class QuantFunc:
    """Per-tensor absmax scaling; subclasses override the pieces they change (quant.py:69-92)."""
    compile_quantize_dequantize = False

    @classmethod
    @torch.no_grad()
    def quantize_dequantize(cls, x: torch.Tensor):
        s = cls.get_scalar(x)
        return cls.rquant(cls.quant(x, s), s)

    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x: torch.Tensor):
        return x.abs().max() + 1e-6

    @classmethod
    @torch.no_grad()
    def quant(cls, x: torch.Tensor, s: torch.Tensor):
        return x / s

    @classmethod
    @torch.no_grad()
    def rquant(cls, x: torch.Tensor, s: torch.Tensor):
        return x * s


class Cast2Fp32(QuantFunc):
    """Identity-like quantizer (divide and multiply by absmax); the base the tests stub from."""


# ---- shared e2m1 helpers (pure torch, any device) -----------------------------------------------------

def _fold_e2m1(q: torch.Tensor) -> torch.Tensor:
    """[0,12] -> index axis [0,7]: halves the slope above 4 and quarters it above 8 (quant.py:124)."""
    return q - (torch.relu(q - 4) / 2 + torch.relu(q - 8) / 4)


def _unfold_e2m1(r: torch.Tensor) -> torch.Tensor:
    """index 0..7 -> twice the e2m1 magnitude {0,1,2,3,4,6,8,12} (quant.py:126)."""
    return r + (torch.relu(r - 4) + torch.relu(r - 6) * 2)


def _e2m1_grid(x: torch.Tensor, s: torch.Tensor, noise: bool) -> torch.Tensor:
    """x / s snapped to the signed e2m1 grid; `noise` adds U[-.5,.5) on the index axis first."""
    sign = x.sign()
    idx = _fold_e2m1(x.abs() / (s / 2))
    if noise:
        idx = idx + (torch.rand_like(idx) - 0.5)
    return _unfold_e2m1(torch.round(idx)) * sign / 2


def _as_blocks(x: torch.Tensor, s: torch.Tensor):
    rows = x.numel() // x.shape[-1]
    nb = x.shape[-1] // _BLOCK
    return x.reshape(rows, 1, nb, _BLOCK), s.reshape(rows, 1, nb, 1)


def _block_absmax(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    assert cols % _BLOCK == 0
    return x2.abs().view(rows, cols // _BLOCK, _BLOCK).amax(dim=2)


def _pow2_round(s: torch.Tensor) -> torch.Tensor:
    """Nearest power of two in the log domain: the MX (E8M0) scale rule (quant.py:230)."""
    return s.sign() * (2 ** ((s + 1e-127).log2().clamp_(-127, 127).round_()))


def _e4m3_relative(s: torch.Tensor) -> torch.Tensor:
    """Scales rounded to E4M3 relative to max(s)/448 (quant.py:311-320)."""
    unit = s.abs().max() / 448
    return (s / unit).to(torch.float8_e4m3fn).to(s.dtype) * unit


# ---- formats outside the accelerated path (pure torch) ---------------------------------------------------

class WeightQuant(QuantFunc):
    """'1p58bit': ternary-style weight rounding against 2*std of |w| (quant.py:95-110)."""

    @classmethod
    @torch.no_grad()
    def quant(cls, w, eps: float = 1e-6, bits=1):
        mag = w.abs()
        step = (2 * mag.std() + eps) / (2 ** bits)
        return ((w / step).round() / (2 ** bits)).clamp(-1, 1) * mag.mean()


class Cast2Fp4e2m1(QuantFunc):
    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return x.abs().max() / 6 + 1e-6

    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        return _e2m1_grid(x, s, noise=False)


class Cast2Fp4e2m1Random(Cast2Fp4e2m1):
    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        return _e2m1_grid(x, s, noise=True)


class Cast2Fp6e3m2(QuantFunc):
    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return x.abs().max() / 625 + 1e-7

    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        root = ((x / s).clamp(-625, 625).abs() ** 0.25).to(torch.float8_e5m2).to(torch.float32)
        return torch.sign(x) * root ** 4


class Cast2Fp8e4m3(QuantFunc):
    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return x.abs().max() / 448 + 1e-6

    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        return (x / s).to(torch.float8_e4m3fn).to(torch.float32)


class BlockQuantFunc(QuantFunc):
    """1 x 16 blocks along the last dimension (quant.py:180-195)."""
    block_shape = (1, _BLOCK)
    _denominator = 6.0
    _epsilon = 1e-9
    _element = Cast2Fp4e2m1

    @classmethod
    @torch.no_grad()
    def _reshape(cls, x, s):
        return _as_blocks(x, s)

    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return _block_absmax(x) / cls._denominator + cls._epsilon

    @classmethod
    def _stored_scale(cls, s):
        return s

    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        xb, sb = _as_blocks(x, s)
        return cls._element.quant(xb, sb).view(x.shape)

    @classmethod
    @torch.no_grad()
    def rquant(cls, x, s):
        xb, sb = _as_blocks(x, cls._stored_scale(s))
        return (xb * sb).view(x.shape)


class Cast2Fp4e2m1Block(BlockQuantFunc):
    _element = Cast2Fp4e2m1Random


class Cast2MXFp4e2m1Block(BlockQuantFunc):
    _element = Cast2Fp4e2m1Random
    _stored_scale = classmethod(lambda cls, s: _pow2_round(s))


class Cast2MXFp4e2m1BlockNOSR(BlockQuantFunc):
    _element = Cast2Fp4e2m1
    _stored_scale = classmethod(lambda cls, s: _pow2_round(s))


class Cast2Fp6e3m2Block(BlockQuantFunc):
    _denominator, _epsilon, _element = 625.0, 1e-7, Cast2Fp6e3m2

    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return super().get_scalar(x).to(torch.float16).to(torch.float32)


class Cast2Fp8e4m3Block(BlockQuantFunc):
    _denominator, _epsilon, _element = 448.0, 1e-7, Cast2Fp8e4m3

    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        return super().get_scalar(x).to(torch.float16).to(torch.float32)


# ---- NVFP4: the accelerated path ------------------------------------------------------------------------------

_native_qdq_validated = False
_native_qdq_disabled_reason = None


def nvfp4_nosr_qdq_compile_status():
    """Same three answers as the reference (quant.py:61-66).  Here "validated" means that the
    native kernel's output was compared once, bit for bit, with the eager op-by-op graph."""
    if _native_qdq_disabled_reason is not None:
        return f"disabled: {_native_qdq_disabled_reason}"
    return "validated" if _native_qdq_validated else "not validated"


def _eager_nosr_graph(x: torch.Tensor) -> torch.Tensor:
    """Op-by-op statement of the round-to-nearest fake quantization, in x's dtype, used only to
    validate the native kernel when `compile_quantize_dequantize` asks for it.  Divisors are
    tensors so that CUDA performs true divisions as the CPU does."""
    rows = x.numel() // x.shape[-1]
    blocks = x.reshape(rows, -1, _BLOCK)
    six, two, top = (torch.tensor(v, dtype=x.dtype, device=x.device) for v in (6.0, 2.0, 448.0))
    s = blocks.abs().amax(dim=2, keepdim=True) / six + 1e-9
    unit = s.amax() / top
    d = (s / unit).to(torch.float8_e4m3fn).to(x.dtype) * unit
    r = torch.round(_fold_e2m1(blocks.abs() / (s / two)))
    return (_unfold_e2m1(r) * blocks.sign() / two * d).reshape(x.shape)


class random_lane:
    """Context manager: stochastic quantizations issued inside use their own Philox key and their own
    device-side offset counter.  Work that runs on a second CUDA stream takes a lane of its own, so that
    two streams never read and bump one counter at the same time (and never share random bits)."""

    def __init__(self, lane: int):
        self.lane = int(lane)

    def __enter__(self):
        self.saved = _NativeNVFP4._lane
        _NativeNVFP4._lane = self.lane
        return self

    def __exit__(self, *exc):
        _NativeNVFP4._lane = self.saved
        return False


class _NativeNVFP4(BlockQuantFunc):
    """Common part of the two NVFP4 quantizers: CUDA only, kernels behind the C ABI."""
    stochastic = False
    sr_bits = 8          # random bits per element of the stochastic rounding: 8 (hardware) or 16 (software)
    _seed = 0x5EED
    _calls = 0

    @classmethod
    def _check(cls, x: torch.Tensor):
        rows = x.numel() // x.shape[-1]
        cols = x.shape[-1]
        br, bc = cls.block_shape
        if rows % br != 0 or cols % bc != 0:
            raise ValueError(f"NVFP4 block shape {cls.block_shape} does not divide tensor shape {tuple(x.shape)}")
        if not x.is_cuda:
            raise RuntimeError(f"{cls.__name__} runs on sm_100a kernels only: got a {x.device.type} tensor "
                               "(there is no CPU fallback)")

    @classmethod
    def _native_input(cls, x: torch.Tensor) -> torch.Tensor:
        return x if x.dtype in (torch.bfloat16, torch.float32) else x.float()

    @classmethod
    def philox_key(cls) -> int:
        """Philox key of the stochastic calls being issued now: the class seed and the random lane in the
        low word, the data-parallel rank in the high word, so that ranks that quantize the same element
        index with the same call number draw independent bits (the reference's ranks each have their own
        torch generator stream)."""
        rank = 0
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            rank = torch.distributed.get_rank()
        return ((cls._seed + _NativeNVFP4._lane) & 0xFFFFFFFF) | (rank << 32)

    _counters = {}          # (device, lane) -> int64 [1]: the Philox offset of the next stochastic call
    _lane = 0               # random lane of the calls being issued now (see random_lane)

    @classmethod
    def _offset_counter(cls, device: torch.device) -> torch.Tensor:
        """Per-device call counter kept ON the device (like torch's graph-safe Philox offset): every
        stochastic quantization reads and bumps it, so eager calls and replays of a captured CUDA
        graph both draw fresh random bits.  Created on first use: run one step before capturing."""
        key = (device, _NativeNVFP4._lane)
        ctr = _NativeNVFP4._counters.get(key)
        if ctr is None:
            ctr = _NativeNVFP4._counters[key] = torch.ones(1, dtype=torch.int64, device=device)
        return ctr

    @classmethod
    @torch.no_grad()
    def quantize_packed(cls, x: torch.Tensor, *, transpose: bool = False, mean: torch.Tensor | None = None,
                        sf_layout: int = cabi.SF_MMA, hadamard_signs: int | None = None) -> ops.NVFP4Tensor:
        """Real FP4: packed codes + E4M3 scales + unit of x viewed as [rows, cols] (or of its
        transpose).  `mean` (fp32 [cols]) is subtracted first and recorded on the result."""
        cls._check(x)
        return ops.nvfp4_quantize(cls._native_input(x), transpose=transpose, stochastic=cls.stochastic,
                                  seed=cls.philox_key(), sf_layout=sf_layout, mean=mean,
                                  offset_counter=cls._offset_counter(x.device) if cls.stochastic else None,
                                  hadamard_signs=hadamard_signs if transpose else None, sr_bits=cls.sr_bits)

    @classmethod
    @torch.no_grad()
    def quantize_packed_dual(cls, x: torch.Tensor, *, mean: torch.Tensor | None = None, sf_layout: int = cabi.SF_MMA,
                             hadamard_signs: int | None = None, token_sums: bool = False, defer: str | None = None):
        """(quantize_packed(x), quantize_packed(x, transpose=True)) from one pass over x: what a training
        step needs of every operand (the products of the backward contract over the other dimension).
        token_sums, defer: see ops.nvfp4_quantize_dual."""
        cls._check(x)
        return ops.nvfp4_quantize_dual(cls._native_input(x), stochastic=cls.stochastic,
                                       seed=cls.philox_key(), sf_layout=sf_layout, mean=mean,
                                       offset_counter=cls._offset_counter(x.device) if cls.stochastic else None,
                                       hadamard_signs=hadamard_signs, token_sums=token_sums, defer=defer, sr_bits=cls.sr_bits)

    @classmethod
    @torch.no_grad()
    def quantize_dequantize(cls, x: torch.Tensor):
        cls._check(x)
        q = cls.quantize_packed(x, sf_layout=cabi.SF_ROWMAJOR)
        out_dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.float32
        return q.dequantize(out_dtype).reshape(x.shape).to(x.dtype)

    # The three-call protocol is kept for callers that still use it (bitlinear.py:294-301,
    # 398-402).  It is not the accelerated path: plain torch ops with tensor divisors.
    @classmethod
    @torch.no_grad()
    def get_scalar(cls, x):
        cls._check(x)
        six = torch.tensor(6.0, dtype=x.dtype, device=x.device)
        return _block_absmax(x) / six + 1e-9

    @classmethod
    @torch.no_grad()
    def quant(cls, x, s):
        xb, sb = _as_blocks(x, s)
        two = torch.tensor(2.0, dtype=x.dtype, device=x.device)
        sign = xb.sign()
        idx = _fold_e2m1(xb.abs() / (sb / two))
        if cls.stochastic:
            idx = idx + (torch.rand_like(idx) - 0.5)
        return (_unfold_e2m1(torch.round(idx)) * sign / two).view(x.shape)

    @classmethod
    @torch.no_grad()
    def rquant(cls, x, s):
        top = torch.tensor(448.0, dtype=s.dtype, device=s.device)
        unit = s.abs().max() / top
        s.div_(unit)                                   # the reference rescales its argument in place (quant.py:313)
        stored = s.to(torch.float8_e4m3fn).to(s.dtype) * unit
        xb, sb = _as_blocks(x, stored)
        return (xb * sb).view(x.shape)


class Cast2NVFp4e2m1BlockNOSR(_NativeNVFP4):
    """Round-to-nearest NVFP4 (registry key 'nvfp4e2m1bnosr')."""
    stochastic = False

    @classmethod
    @torch.no_grad()
    def quantize_dequantize(cls, x: torch.Tensor):
        global _native_qdq_validated, _native_qdq_disabled_reason
        out = super().quantize_dequantize(x)
        if cls.compile_quantize_dequantize and not _native_qdq_validated and _native_qdq_disabled_reason is None:
            # The reference validates its torch.compile'd graph against the eager one on first use
            # (quant.py:420-432); the native kernel is validated the same way.  It computes in
            # fp32, so the comparison runs on the fp32 view of the input.
            xf = x.float()
            eager = _eager_nosr_graph(xf)
            native = super().quantize_dequantize(xf)
            if torch.equal(native, eager):
                _native_qdq_validated = True
            else:
                bad = int((native != eager).sum())
                _native_qdq_disabled_reason = f"native output differed from eager output at {bad}/{x.numel()} elements"
        return out


class Cast2NVFp4e2m1Block(_NativeNVFP4):
    """Stochastic-rounding NVFP4 (registry key 'nvfp4e2m1b'), the backward default.  `sr_bits`: 8 uses the
    hardware's stochastic e2m1 conversion (8 random bits per element: a value goes up with probability
    floor(256 p) / 256, p its position between its neighbours); 16 the software form (2^-16 steps)."""
    stochastic = True


@torch.no_grad()
def cast_2_fp32(x):
    return x


quant_func = {
    "fp4e2m1": Cast2Fp4e2m1,
    "nvfp4e2m1b": Cast2NVFp4e2m1Block,
    "mxfp4e2m1b": Cast2MXFp4e2m1Block,
    "mxfp4e2m1bnosr": Cast2MXFp4e2m1BlockNOSR,
    "nvfp4e2m1bnosr": Cast2NVFp4e2m1BlockNOSR,
    "fp6e3m2": Cast2Fp6e3m2,
    "fp6e3m2b": Cast2Fp6e3m2Block,
    "fp8e4m3": Cast2Fp8e4m3,
    "fp8e4m3b": Cast2Fp8e4m3Block,
    "fp32": Cast2Fp32,
    "1p58bit": WeightQuant,
}


def is_native(quantizer) -> bool:
    """True for quantizer classes that can emit packed FP4 for the tensor-core path."""
    return isinstance(quantizer, type) and issubclass(quantizer, _NativeNVFP4)
