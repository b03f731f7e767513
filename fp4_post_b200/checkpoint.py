"""State-dict bridge for Metis layers.

A BitLinear stores `ulinear.weight [N, r]`, `s [r]`, `vlinear.weight [r, K]` and
`warmup_linear.weight [N, K]` (+ biases): the same parameter names as the reference, so checkpoints
move between the two builds unchanged.  Two conversions sit on top of that contract:

merge_state_dict    folds every BitLinear back into a plain `weight` (+ `bias`) of a standard
                    nn.Linear: W = U diag(s) V + R in fp32, cast back to the residual's dtype.  Same key
                    handling as the reference's converter (tools/convert_bitlinear_to_standard.py:80-172).
export_packed       what a native NVFP4 inference engine loads: for every BitLinear the residual and
                    the V factor as packed e2m1 codes + E4M3 block scales + fp32 unit (row-major
                    scales, the portable layout), U and s in their stored dtype.  The draft paper's
                    "native NVFP4 inference" evaluation (fp4_post_aaai_draft.tex:234) needs exactly this.
import_packed       the inverse: dequantized weights for a standard state dict, or (on a CUDA device)
                    packed operands that a BitLinear's weight cache can serve directly.
"""
from __future__ import annotations

import re
from collections import OrderedDict
from typing import Dict, Iterable, Mapping, Optional, Set

import torch

_FACTOR_SUFFIXES = ("ulinear.weight", "ulinear.bias", "vlinear.weight", "vlinear.bias", "s",
                    "warmup_linear.weight", "warmup_linear.bias")
_PACKED_PARTS = ("codes", "scales", "unit")


def bitlinear_prefixes(keys: Iterable[str]) -> Set[str]:
    """Module paths that own a ulinear / vlinear / warmup_linear child."""
    found = set()
    for key in keys:
        m = re.match(r"(.+)\.(ulinear|vlinear|warmup_linear)\.", key)
        if m:
            found.add(m.group(1))
    return found


def merged_weight(u: torch.Tensor, s: torch.Tensor, v: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
    """U diag(s) V (+ R), accumulated in fp32; the dtype of the residual (else of U) comes back."""
    w = (u.float() * s.float().unsqueeze(0)) @ v.float()
    if residual is not None:
        return (w + residual.float()).to(residual.dtype)
    return w.to(u.dtype)


def _cast(t: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    return t.to(dtype) if dtype is not None and torch.is_floating_point(t) else t


def merge_state_dict(state_dict: Mapping[str, torch.Tensor], target_dtype: Optional[torch.dtype] = None,
                     report: Optional[list] = None) -> "OrderedDict[str, torch.Tensor]":
    """Every BitLinear becomes `prefix.weight` (+ `prefix.bias`: the residual's bias, else the U
    branch's); a module with only a residual is copied; everything else passes through.  `report`
    collects one line per module."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    consumed = set()
    for prefix in sorted(bitlinear_prefixes(state_dict.keys())):
        get = lambda suffix: state_dict.get(f"{prefix}.{suffix}")
        u, v, s, r = get("ulinear.weight"), get("vlinear.weight"), get("s"), get("warmup_linear.weight")
        bias = get("warmup_linear.bias")
        if bias is None:
            bias = get("ulinear.bias")
        consumed.update(f"{prefix}.{x}" for x in _FACTOR_SUFFIXES if f"{prefix}.{x}" in state_dict)
        if u is not None and v is not None and s is not None:
            out[f"{prefix}.weight"] = _cast(merged_weight(u, s, v, r), target_dtype)
            note = "merged U diag(s) V" + (" + residual" if r is not None else "")
        elif r is not None:
            out[f"{prefix}.weight"] = _cast(r, target_dtype)
            bias = get("warmup_linear.bias")
            note = "copied the residual"
        else:
            missing = [n for n, t in (("ulinear.weight", u), ("s", s), ("vlinear.weight", v), ("warmup_linear.weight", r)) if t is None]
            note = f"skipped, missing {missing}"
            bias = None
        if bias is not None:
            out[f"{prefix}.bias"] = _cast(bias, target_dtype)
        if report is not None:
            report.append(f"{prefix}: {note}")
    for key, value in state_dict.items():
        if key not in consumed:
            out[key] = _cast(value, target_dtype)
    return out


def export_packed(state_dict: Mapping[str, torch.Tensor], device: torch.device | str = "cuda") -> "OrderedDict[str, torch.Tensor]":
    """Packed NVFP4 export: `prefix.{warmup_linear,vlinear}.weight` of every BitLinear become
    `….weight.nvfp4.codes` (uint8 [rows, cols/2]), `.scales` (E4M3 bytes [rows, cols/16]), `.unit` (fp32 [1])
    and `.shape`; all other entries pass through.  Quantization is the round-to-nearest weight quantizer
    of the forward pass (the sm_100a kernel: needs a CUDA device and the built library)."""
    from fp4_post_b200 import cabi, ops
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    packed_keys = set()
    for prefix in bitlinear_prefixes(state_dict.keys()):
        for child in ("warmup_linear", "vlinear"):
            key = f"{prefix}.{child}.weight"
            w = state_dict.get(key)
            if w is not None and w.dim() == 2 and w.shape[1] % 16 == 0:
                packed_keys.add(key)
    for key, value in state_dict.items():
        if key not in packed_keys:
            out[key] = value
            continue
        w = value.to(device)
        if w.dtype not in (torch.bfloat16, torch.float32):
            w = w.float()
        q = ops.nvfp4_quantize(w.contiguous(), sf_layout=cabi.SF_ROWMAJOR)
        out[f"{key}.nvfp4.codes"] = q.codes.cpu()
        out[f"{key}.nvfp4.scales"] = q.scales.cpu()
        out[f"{key}.nvfp4.unit"] = q.unit.cpu()
        out[f"{key}.nvfp4.shape"] = torch.tensor(list(value.shape), dtype=torch.int64)
    return out


_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def dequantize_packed(codes: torch.Tensor, scales: torch.Tensor, unit: torch.Tensor, shape) -> torch.Tensor:
    """fp32 values of a packed NVFP4 tensor with row-major scales; plain torch, any device (the
    decoder a checkpoint reader needs: value = e2m1(code) * e4m3(scale) * unit)."""
    rows, cols = int(shape[0]), int(shape[1])
    c = codes.reshape(rows, cols // 2).to(torch.int64)
    nib = torch.stack((c & 0xF, c >> 4), dim=-1).reshape(rows, cols)        # element 2i in the low nibble
    mag = _E2M1.to(codes.device)[nib & 7]
    val = torch.where((nib & 8) != 0, -mag, mag)
    sc = scales.reshape(rows, cols // 16).view(torch.float8_e4m3fn).float()
    return val.reshape(rows, cols // 16, 16).mul(sc.unsqueeze(-1)).mul(unit.float().reshape(())).reshape(rows, cols)


def import_packed(state_dict: Mapping[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16) -> "OrderedDict[str, torch.Tensor]":
    """A standard Metis state dict from a packed export: the packed weights are dequantized to `dtype`
    (exactly representable in bf16: e2m1 x e4m3 has 5 significant bits; the unit multiplies in fp32 and
    the product is rounded once)."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    groups: Dict[str, Dict[str, torch.Tensor]] = {}
    for key, value in state_dict.items():
        m = re.match(r"(.+)\.nvfp4\.(codes|scales|unit|shape)$", key)
        if m:
            groups.setdefault(m.group(1), {})[m.group(2)] = value
        else:
            out[key] = value
    for key, parts in groups.items():
        missing = [p for p in (*_PACKED_PARTS, "shape") if p not in parts]
        if missing:
            raise KeyError(f"packed tensor {key} lacks {missing}")
        out[key] = dequantize_packed(parts["codes"], parts["scales"], parts["unit"], parts["shape"].tolist()).to(dtype)
    return out
