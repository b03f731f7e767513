"""Tensor-level wrappers over the C ABI: PyTorch supplies device memory and streams only.

Every function needs CUDA tensors and the built library; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import cabi

_DTYPES = {torch.bfloat16: cabi.DTYPE_BF16, torch.float32: cabi.DTYPE_F32}

# Kernels of this library launched since import, by entry point (two per quantizer call: the
# streaming pass and the scale pass; the memset between them is not a kernel).
LAUNCHES = {"quantize": 0, "rmsnorm_quantize": 0, "dequantize": 0, "col_mean": 0, "gemv": 0, "gemm": 0, "lowrank_bwd": 0}


def launch_count() -> int:
    return sum(LAUNCHES.values())


def _dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"{what} must be bfloat16 or float32, got {t.dtype}") from None


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: the NVFP4 path has no CPU fallback")


def _stream() -> int:
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


class _on_device:
    """Makes `dev` current for the calls inside; free when it already is (the common case)."""
    __slots__ = ("guard",)

    def __init__(self, dev: torch.device):
        self.guard = None if dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _packed_buffers(L, R: int, Cc: int, sf_layout: int, dev):
    """codes, scales and unit of one quantized tensor as views of a single allocation."""
    n_codes = R * (Cc // 2)
    n_scales = L.metis_nvfp4_sf_bytes(R, Cc, sf_layout)
    o_scales = (n_codes + 255) & ~255
    o_unit = (o_scales + n_scales + 255) & ~255
    buf = torch.empty(o_unit + 16, dtype=torch.uint8, device=dev)
    return buf[:n_codes].view(R, Cc // 2), buf[o_scales:o_scales + n_scales], buf[o_unit:o_unit + 4].view(torch.float32)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _rows2d(x: torch.Tensor) -> torch.Tensor:
    """View x as [rows, cols] with unit stride along cols (copy only if it has to)."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < x2.shape[1]):
        x2 = x2.contiguous()
    return x2


@dataclass
class NVFP4Tensor:
    """A quantized [R, C] matrix: packed e2m1 codes, E4M3 block scales, fp32 unit.

    `row_vec` (fp32 [C]) is the mean that was subtracted before quantization; the represented
    matrix is value(codes, scales, unit) + 1 * row_vec (bitlinear.py:330-332).  For a
    transposed quantization of x [M, K] with column means, `col_vec` (fp32 [R]) holds them
    instead: the represented matrix is value + col_vec * 1^T.
    """
    codes: torch.Tensor          # uint8 [R, C/2]
    scales: torch.Tensor         # uint8, flat
    unit: torch.Tensor           # float32 [1]
    shape: tuple
    sf_layout: int
    row_vec: Optional[torch.Tensor] = None
    col_vec: Optional[torch.Tensor] = None
    token_sums: Optional[torch.Tensor] = None     # fp32 [R]: sums of the rows' quantized values, when the quantizer formed them

    @property
    def device(self):
        return self.codes.device

    def dequantize(self, dtype: torch.dtype = torch.float32, add_mean: bool = True) -> torch.Tensor:
        return nvfp4_dequantize(self, dtype, add_mean=add_mean)


def col_mean(x: torch.Tensor) -> torch.Tensor:
    """Column means of x viewed as [rows, cols], fp32 (input_flat.mean(dim=0), bitlinear.py:326)."""
    _need_cuda(x, "x")
    x2 = _rows2d(x)
    rows, cols = x2.shape
    L = cabi.lib()
    with _on_device(x2.device):
        mean = torch.empty(cols, dtype=torch.float32, device=x2.device)
        ws_bytes = L.metis_col_mean_workspace_bytes(rows, cols)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x2.device)
        rc = L.metis_col_mean(x2.data_ptr(), _dtype_code(x2, "x"), rows, cols, x2.stride(0), mean.data_ptr(),
                              ws.data_ptr(), ws.numel(), _stream())
    cabi.check(rc, "metis_col_mean")
    LAUNCHES["col_mean"] += 2
    return mean


def _hadamard_flags(sign_mask: Optional[int]) -> int:
    """Flag bits that make the transposed quantizer rotate its blocks: sign_mask has bit i set where position
    i of every block of 16 is negated before the Hadamard butterfly; None: no rotation."""
    if sign_mask is None:
        return 0
    if not 0 <= sign_mask < 1 << 16:
        raise ValueError("sign_mask holds one bit per position of a block of 16")
    return cabi.Q_HADAMARD | (sign_mask << 16)


def _sr_flags(stochastic: bool, sr_bits: int) -> int:
    if sr_bits not in (8, 16):
        raise ValueError(f"sr_bits must be 8 (hardware conversion) or 16 (software), not {sr_bits}")
    return cabi.Q_SR16 if stochastic and sr_bits == 16 else 0


def nvfp4_quantize(x: torch.Tensor, *, transpose: bool = False, stochastic: bool = False, seed: int = 0,
                   offset: int = 0, sf_layout: int = cabi.SF_MMA,
                   mean: Optional[torch.Tensor] = None,
                   offset_counter: Optional[torch.Tensor] = None,
                   hadamard_signs: Optional[int] = None, sr_bits: int = 8) -> NVFP4Tensor:
    """Quantize x (viewed as [rows, cols]) or, with transpose=True, its transpose.
    sr_bits: random bits per element of the stochastic rounding, 8 (the hardware conversion) or 16 (software).

    `mean` (fp32 [cols]) is subtracted from every row of x first.  Stochastic rounding draws
    Philox(seed; element, offset); with `offset_counter` (int64 [1] on x's device) the offset is that
    counter's value and the call increments it, so the call can sit in a CUDA graph that is replayed."""
    _need_cuda(x, "x")
    x2 = _rows2d(x)
    rows, cols = x2.shape
    R, Cc = (cols, rows) if transpose else (rows, cols)
    if Cc % 16 != 0 or R == 0:
        raise ValueError(f"NVFP4 block shape (1, 16) does not divide tensor shape {(R, Cc)}")
    L = cabi.lib()
    flags = (cabi.Q_TRANSPOSE if transpose else 0) | (cabi.Q_STOCHASTIC if stochastic else 0) | _hadamard_flags(hadamard_signs)
    flags |= _sr_flags(stochastic, sr_bits)
    dev = x2.device
    if stochastic and offset_counter is not None:
        if offset_counter.dtype != torch.int64 or offset_counter.device != dev or offset_counter.numel() != 1:
            raise ValueError("offset_counter must be an int64 tensor with one element on the device of x")
        flags |= cabi.Q_OFFSET_ON_DEVICE
        offset = offset_counter.data_ptr()
    if mean is not None:
        _need_cuda(mean, "mean")
        mean = mean.reshape(-1).to(torch.float32).contiguous()
        assert mean.numel() == cols
    with _on_device(dev):
        codes, scales, unit = _packed_buffers(L, R, Cc, sf_layout, dev)
        ws = torch.empty(L.metis_nvfp4_quantize_workspace_bytes(R, Cc), dtype=torch.uint8, device=dev)
        rc = L.metis_nvfp4_quantize(x2.data_ptr(), _dtype_code(x2, "x"), rows, cols, x2.stride(0), _ptr(mean),
                                    flags, seed & (2**64 - 1), offset & (2**64 - 1), sf_layout,
                                    codes.data_ptr(), scales.data_ptr(), unit.data_ptr(), ws.data_ptr(),
                                    ws.numel(), _stream())
    cabi.check(rc, "metis_nvfp4_quantize")
    LAUNCHES["quantize"] += 2
    q = NVFP4Tensor(codes, scales, unit, (R, Cc), sf_layout)
    if mean is not None:
        if transpose:
            q.col_vec = mean
        else:
            q.row_vec = mean
    return q


def nvfp4_quantize_dual(x: torch.Tensor, *, stochastic: bool = False, seed: int = 0, offset: int = 0,
                        sf_layout: int = cabi.SF_MMA, mean: Optional[torch.Tensor] = None,
                        offset_counter: Optional[torch.Tensor] = None, hadamard_signs: Optional[int] = None,
                        token_sums: bool = False, defer: Optional[str] = None, sr_bits: int = 8):
    """Both quantizations of x viewed as [rows, cols] from one pass over it: (Q of x, Q of x^T), each
    bit-identical to the separate call (round to nearest).  rows and cols must be multiples of 16.
    With token_sums the second result carries `token_sums` (fp32 [cols]), the sums of its rows' quantized
    values, formed by the scale pass (where the shape allows it: rows a multiple of 64, no rotation).
    defer = "rowmajor" or "transposed": the scale pass of that output (its scales, unit, token sums) is left
    out; a third value is returned, a function that launches it on the stream that is current when it is
    called (the caller orders that stream after this call and its consumers after that launch)."""
    _need_cuda(x, "x")
    x2 = _rows2d(x)
    rows, cols = x2.shape
    if rows % 16 != 0 or cols % 16 != 0 or rows == 0:
        raise ValueError(f"NVFP4 block shape (1, 16) does not divide both dimensions of tensor shape {(rows, cols)}")
    L = cabi.lib()
    flags = (cabi.Q_STOCHASTIC if stochastic else 0) | _hadamard_flags(hadamard_signs)      # rotation: the transposed output only
    flags |= _sr_flags(stochastic, sr_bits)
    if defer not in (None, "rowmajor", "transposed"):
        raise ValueError(f"defer must be 'rowmajor' or 'transposed', not {defer!r}")
    deferred = {None: 0, "rowmajor": cabi.Q_DEFER_ROWMAJOR, "transposed": cabi.Q_DEFER_TRANSPOSED}[defer]
    flags |= deferred
    dev = x2.device
    if stochastic and offset_counter is not None:
        if offset_counter.dtype != torch.int64 or offset_counter.device != dev or offset_counter.numel() != 1:
            raise ValueError("offset_counter must be an int64 tensor with one element on the device of x")
        flags |= cabi.Q_OFFSET_ON_DEVICE
        offset = offset_counter.data_ptr()
    if mean is not None:
        _need_cuda(mean, "mean")
        mean = mean.reshape(-1).to(torch.float32).contiguous()
        assert mean.numel() == cols
    with _on_device(dev):
        codes, scales, unit = _packed_buffers(L, rows, cols, sf_layout, dev)
        codes_t, scales_t, unit_t = _packed_buffers(L, cols, rows, sf_layout, dev)
        ws = torch.empty(L.metis_nvfp4_quantize_dual_workspace_bytes(rows, cols), dtype=torch.uint8, device=dev)
        sums = None
        if token_sums and rows % 64 == 0 and hadamard_signs is None:
            sums = torch.empty(cols, dtype=torch.float32, device=dev)
        rc = L.metis_nvfp4_quantize_dual(x2.data_ptr(), _dtype_code(x2, "x"), rows, cols, x2.stride(0), _ptr(mean),
                                         flags, seed & (2**64 - 1), offset & (2**64 - 1), sf_layout,
                                         codes.data_ptr(), scales.data_ptr(), unit.data_ptr(),
                                         codes_t.data_ptr(), scales_t.data_ptr(), unit_t.data_ptr(), _ptr(sums),
                                         ws.data_ptr(), ws.numel(), _stream())
    cabi.check(rc, "metis_nvfp4_quantize_dual")
    LAUNCHES["quantize"] += 2
    q = NVFP4Tensor(codes, scales, unit, (rows, cols), sf_layout)
    qt = NVFP4Tensor(codes_t, scales_t, unit_t, (cols, rows), sf_layout)
    if mean is not None:
        q.row_vec = mean
        qt.col_vec = mean
    qt.token_sums = sums
    if defer is None:
        return q, qt

    def finish():
        with _on_device(dev):
            rc2 = L.metis_nvfp4_quantize_dual_finish(rows, cols, deferred, sf_layout, scales.data_ptr(), unit.data_ptr(),
                                                     codes_t.data_ptr(), scales_t.data_ptr(), unit_t.data_ptr(), _ptr(sums),
                                                     ws.data_ptr(), ws.numel(), _stream())
        cabi.check(rc2, "metis_nvfp4_quantize_dual_finish")
        # the buffers were allocated on the quantizing call's stream and are now also used on this one
        cur = torch.cuda.current_stream(dev)
        for t in (ws, scales, unit, codes_t, scales_t, unit_t, sums):
            if t is not None:
                t.record_stream(cur)
        LAUNCHES["quantize"] += 1
    return q, qt, finish


def rmsnorm_nvfp4_quantize(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, *,
                           sf_layout: int = cabi.SF_MMA, return_norm: bool = False):
    """Fused RMSNorm -> NVFP4 quantization of x viewed as [rows, cols] (llama.py:23-31 then
    quant.py:6-36).  Returns the NVFP4Tensor, and the normalised tensor too if asked."""
    _need_cuda(x, "x")
    _need_cuda(gamma, "gamma")
    x2 = _rows2d(x)
    rows, cols = x2.shape
    if cols % 16 != 0 or rows == 0:
        raise ValueError(f"NVFP4 block shape (1, 16) does not divide tensor shape {(rows, cols)}")
    gamma = gamma.contiguous()
    assert gamma.numel() == cols
    L = cabi.lib()
    dev = x2.device
    with _on_device(dev):
        codes, scales, unit = _packed_buffers(L, rows, cols, sf_layout, dev)
        ws = torch.empty(L.metis_nvfp4_quantize_workspace_bytes(rows, cols), dtype=torch.uint8, device=dev)
        norm = None
        if return_norm:
            out_dtype = torch.bfloat16 if (x2.dtype == torch.bfloat16 and gamma.dtype == torch.bfloat16) else torch.float32
            norm = torch.empty((rows, cols), dtype=out_dtype, device=dev)
        rc = L.metis_rmsnorm_nvfp4_quantize(x2.data_ptr(), _dtype_code(x2, "x"), rows, cols, x2.stride(0),
                                            gamma.data_ptr(), _dtype_code(gamma, "gamma"), float(eps), sf_layout,
                                            codes.data_ptr(), scales.data_ptr(), unit.data_ptr(), _ptr(norm),
                                            ws.data_ptr(), ws.numel(), _stream())
    cabi.check(rc, "metis_rmsnorm_nvfp4_quantize")
    LAUNCHES["rmsnorm_quantize"] += 2
    q = NVFP4Tensor(codes, scales, unit, (rows, cols), sf_layout)
    return (q, norm.reshape(x.shape)) if return_norm else q


def rmsnorm_mean(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, *, want_rstd: bool = True):
    """RMSNorm of x viewed as [rows, cols] with the column mean of its output from the same pass:
    (y shaped like x, mean fp32 [cols], rstd fp32 [rows] or None).  First pass of the mean-centred
    activation path; nvfp4_quantize[_dual](y, mean=mean) is the second."""
    _need_cuda(x, "x")
    _need_cuda(gamma, "gamma")
    x2 = _rows2d(x)
    rows, cols = x2.shape
    if cols % 16 != 0 or rows == 0:
        raise ValueError(f"NVFP4 block shape (1, 16) does not divide tensor shape {(rows, cols)}")
    gamma = gamma.contiguous()
    assert gamma.numel() == cols
    L = cabi.lib()
    dev = x2.device
    with _on_device(dev):
        out_dtype = torch.bfloat16 if (x2.dtype == torch.bfloat16 and gamma.dtype == torch.bfloat16) else torch.float32
        y = torch.empty((rows, cols), dtype=out_dtype, device=dev)
        mean = torch.empty(cols, dtype=torch.float32, device=dev)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev) if want_rstd else None
        ws = torch.empty(max(16, L.metis_rmsnorm_mean_workspace_bytes(rows, cols)), dtype=torch.uint8, device=dev)
        rc = L.metis_rmsnorm_mean(x2.data_ptr(), _dtype_code(x2, "x"), rows, cols, x2.stride(0), gamma.data_ptr(),
                                  _dtype_code(gamma, "gamma"), float(eps), y.data_ptr(), _ptr(rstd), mean.data_ptr(),
                                  ws.data_ptr(), ws.numel(), _stream())
    cabi.check(rc, "metis_rmsnorm_mean")
    LAUNCHES["rmsnorm_quantize"] += 2
    return y.reshape(x.shape), mean, rstd


def nvfp4_dequantize(q: NVFP4Tensor, dtype: torch.dtype = torch.float32, add_mean: bool = True,
                     unit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense [R, C] tensor of q.  `unit` (fp32 [1], device) replaces q's own unit, e.g. to express the
    values in another product's accumulator units."""
    R, Cc = q.shape
    L = cabi.lib()
    with _on_device(q.device):
        out = torch.empty((R, Cc), dtype=dtype, device=q.device)
        rv = q.row_vec if add_mean else None
        rc = L.metis_nvfp4_dequantize(q.codes.data_ptr(), q.scales.data_ptr(), (q.unit if unit is None else unit).data_ptr(), q.sf_layout, R, Cc,
                                      _ptr(rv), out.data_ptr(), _DTYPES[dtype], out.stride(0), _stream())
    cabi.check(rc, "metis_nvfp4_dequantize")
    LAUNCHES["dequantize"] += 1
    if add_mean and q.col_vec is not None:
        out += q.col_vec.to(dtype)[:, None]
    return out


def nvfp4_gemv(q: NVFP4Tensor, v: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = sum_c v[c] * value(q)[r, c] (v None: row sums), fp32; the mean vectors of q are ignored."""
    R, Cc = q.shape
    L = cabi.lib()
    if v is not None:
        v = v.reshape(-1).to(torch.float32).contiguous()
        assert v.numel() == Cc
    with _on_device(q.device):
        out = torch.empty(R, dtype=torch.float32, device=q.device)
        rc = L.metis_nvfp4_gemv(q.codes.data_ptr(), q.scales.data_ptr(), q.unit.data_ptr(), q.sf_layout, R, Cc,
                                _ptr(v), out.data_ptr(), _stream())
    cabi.check(rc, "metis_nvfp4_gemv")
    LAUNCHES["gemv"] += 1
    return out


def lowrank_scale(yv: torch.Tensor, s: torch.Tensor, unit_a: torch.Tensor, unit_b: torch.Tensor) -> torch.Tensor:
    """bf16( (yv * s).float() / (unit_a * unit_b) ) for bf16 yv [M, r]: torch.mul(self.s, y) of the
    low-rank branch, in the accumulator units of the GEMM whose side product it feeds (one kernel)."""
    _need_cuda(yv, "yv")
    if yv.dtype != torch.bfloat16 or yv.dim() != 2 or yv.stride(1) != 1:
        raise TypeError("yv must be a bf16 matrix with contiguous rows")
    if s.dtype not in (torch.bfloat16, torch.float32):
        s = s.float()
    s = s.reshape(-1).contiguous()
    M, r = yv.shape
    assert s.numel() == r and s.device == yv.device
    with _on_device(yv.device):
        out = torch.empty((M, r), dtype=torch.bfloat16, device=yv.device)
        rc = cabi.lib().metis_lowrank_scale(yv.data_ptr(), M, r, yv.stride(0), s.data_ptr(), _dtype_code(s, "s"),
                                            unit_a.data_ptr(), unit_b.data_ptr(), out.data_ptr(), _stream())
    cabi.check(rc, "metis_lowrank_scale")
    LAUNCHES["gemv"] += 1
    return out


def nvfp4_gemm(a: NVFP4Tensor, b: NVFP4Tensor, *, lowrank=None, rank1=(), c: Optional[torch.Tensor] = None,
               out_dtype: torch.dtype = torch.bfloat16, alpha: float = 1.0,
               status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               sm_limit: int = 0, _debug: int = 0) -> torch.Tensor:
    """D = alpha*ua*ub * (A @ B^T + T @ U^T) + sum_i cvec_i (x) rvec_i (+ c), see metis_nvfp4_gemm.

    a: [M, K], b: [N, K] (both METIS_SF_MMA).  lowrank = (T [M, r] bf16, U [N, r] bf16), already in
    accumulator units.  rank1 = up to two (cvec or None, rvec) pairs of fp32 vectors.
    Only the packed parts of a and b enter the product; their mean vectors do not.
    sm_limit > 0 caps the SMs this launch occupies (room for a collective's kernel beside it)."""
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: {K} vs {K2}")
    if a.sf_layout != cabi.SF_MMA or b.sf_layout != cabi.SF_MMA:
        raise ValueError("GEMM operands need METIS_SF_MMA scales")
    dev = a.device
    args = cabi.GemmArgs()
    args.M, args.N, args.K = M, N, K
    args.a_codes, args.a_scales, args.a_unit = a.codes.data_ptr(), a.scales.data_ptr(), a.unit.data_ptr()
    args.b_codes, args.b_scales, args.b_unit = b.codes.data_ptr(), b.scales.data_ptr(), b.unit.data_ptr()
    args.alpha = float(alpha)
    keep = []
    if lowrank is not None:
        T, U = lowrank
        if T.dtype != torch.bfloat16 or U.dtype != torch.bfloat16:
            raise TypeError("low-rank factors must be bfloat16")
        T, U = _rows2d(T), _rows2d(U)
        if T.shape[0] != M or U.shape[0] != N or T.shape[1] != U.shape[1]:
            raise ValueError(f"low-rank shapes {tuple(T.shape)} / {tuple(U.shape)} do not fit [{M}, r] / [{N}, r]")
        keep += [T, U]
        args.rank = T.shape[1]
        args.lr_t, args.ldt = T.data_ptr(), T.stride(0)
        args.lr_u, args.ldu = U.data_ptr(), U.stride(0)
    if len(rank1) > 2:
        raise ValueError("at most two rank-1 terms")
    for i, (cv, rv) in enumerate(rank1):
        rv = rv.reshape(-1).to(torch.float32).contiguous()
        assert rv.numel() == N and rv.is_cuda
        keep.append(rv)
        if cv is not None:
            cv = cv.reshape(-1).to(torch.float32).contiguous()
            assert cv.numel() == M and cv.is_cuda
            keep.append(cv)
        setattr(args, f"cvec{i}", _ptr(cv))
        setattr(args, f"rvec{i}", rv.data_ptr())
    with _on_device(dev):
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=dev)
        else:
            assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
        if c is not None:
            assert c.shape == (M, N) and c.dtype == out_dtype and c.stride(1) == 1 and c.is_cuda
            args.c, args.ldc = c.data_ptr(), c.stride(0)
        args.d, args.ldd = out.data_ptr(), out.stride(0)
        args.d_dtype = _DTYPES[out_dtype]
        args.reserved = int(_debug)
        args.sm_limit = int(sm_limit)
        args.status = _ptr(status)
        args.stream = _stream()
        ws_bytes = cabi.lib().metis_nvfp4_gemm_workspace_bytes(M, N, K) if M <= 128 else 0
        if ws_bytes > 0:                      # decode-sized product: scratch for its split-K partial sums
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            keep.append(ws)
            args.workspace, args.workspace_bytes = ws.data_ptr(), ws_bytes
        rc = cabi.lib().metis_nvfp4_gemm(C.byref(args))
    cabi.check(rc, "metis_nvfp4_gemm")
    LAUNCHES["gemm"] += 2 if ws_bytes > 0 else 1
    return out


def _bf16_rows(t: torch.Tensor, what: str) -> torch.Tensor:
    _need_cuda(t, what)
    if t.dtype != torch.bfloat16 or t.dim() != 2:
        raise TypeError(f"{what} must be a bf16 matrix")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def bf16_panel_gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
                    status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """D = A_op B_op^T in bf16 on the tensor core, fp32 out, at most 256 columns.  a is [Mg, Kg], or
    [Kg, Mg] with a_mn_major; b is [Ng, Kg], or [Kg, Ng] with b_mn_major."""
    a, b = _bf16_rows(a, "a"), _bf16_rows(b, "b")
    Mg, Kg = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    Ng, Kb = (b.shape[1], b.shape[0]) if b_mn_major else b.shape
    if Kg != Kb:
        raise ValueError(f"inner dimensions differ: {Kg} vs {Kb}")
    L = cabi.lib()
    with _on_device(a.device):
        out = torch.empty((Mg, Ng), dtype=torch.float32, device=a.device)
        ws = torch.empty(max(16, L.metis_bf16_panel_gemm_workspace_bytes(Mg, Ng, Kg)), dtype=torch.uint8, device=a.device)
        rc = L.metis_bf16_panel_gemm(a.data_ptr(), int(a_mn_major), a.stride(0), b.data_ptr(), int(b_mn_major), b.stride(0),
                                     Mg, Ng, Kg, out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(), _ptr(status), _stream())
    cabi.check(rc, "metis_bf16_panel_gemm")
    LAUNCHES["lowrank_bwd"] += 2
    return out


def lowrank_dts(g: torch.Tensor, u: torch.Tensor, yv: torch.Tensor, s: torch.Tensor, status: Optional[torch.Tensor] = None):
    """(d_yv, ds) of the low-rank branch from one pass over g [M, N]: d_ts = bf16(g @ u), d_yv = bf16(d_ts * s),
    ds = sum over rows of bf16(d_ts * yv) in fp32.  u [N, r], yv [M, r] bf16; s [r] bf16 or fp32."""
    g, u, yv = _bf16_rows(g, "g"), _bf16_rows(u, "u"), _bf16_rows(yv, "yv")
    M, N = g.shape
    r = u.shape[1]
    if u.shape[0] != N or yv.shape != (M, r) or s.numel() != r:
        raise ValueError(f"shapes do not fit: g {tuple(g.shape)}, u {tuple(u.shape)}, yv {tuple(yv.shape)}, s {tuple(s.shape)}")
    if s.dtype not in (torch.bfloat16, torch.float32):
        s = s.float()
    s = s.reshape(-1).contiguous()
    L = cabi.lib()
    with _on_device(g.device):
        d_yv = torch.empty((M, r), dtype=torch.bfloat16, device=g.device)
        ds = torch.empty(r, dtype=torch.float32, device=g.device)
        ws = torch.empty(L.metis_lowrank_dts_workspace_bytes(M, N, r), dtype=torch.uint8, device=g.device)
        rc = L.metis_lowrank_dts(g.data_ptr(), g.stride(0), M, N, u.data_ptr(), u.stride(0), r, yv.data_ptr(), yv.stride(0),
                                 s.data_ptr(), _dtype_code(s, "s"), d_yv.data_ptr(), d_yv.stride(0), ds.data_ptr(),
                                 ws.data_ptr(), ws.numel(), _ptr(status), _stream())
    cabi.check(rc, "metis_lowrank_dts")
    LAUNCHES["lowrank_bwd"] += 2
    return d_yv, ds


def lowrank_du(g: torch.Tensor, ts: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dU = g^T @ ts [N, r] for g [M, N] and ts [M, r] (bf16), one pass over g, no transposed copies."""
    g, ts = _bf16_rows(g, "g"), _bf16_rows(ts, "ts")
    M, N = g.shape
    r = ts.shape[1]
    if ts.shape[0] != M:
        raise ValueError(f"shapes do not fit: g {tuple(g.shape)}, ts {tuple(ts.shape)}")
    L = cabi.lib()
    with _on_device(g.device):
        out = torch.empty((N, r), dtype=out_dtype, device=g.device)
        ws = torch.empty(L.metis_lowrank_du_workspace_bytes(M, N, r), dtype=torch.uint8, device=g.device)
        rc = L.metis_lowrank_du(g.data_ptr(), g.stride(0), M, N, ts.data_ptr(), ts.stride(0), r, out.data_ptr(), _DTYPES[out_dtype],
                                out.stride(0), ws.data_ptr(), ws.numel(), _ptr(status), _stream())
    cabi.check(rc, "metis_lowrank_du")
    LAUNCHES["lowrank_bwd"] += 2
    return out
