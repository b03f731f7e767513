"""The reference's own BitLinear, assembled on the CPU from the modules oracle/build_ref.py placed in
oracle/_ref/ (decisivemoments/fp4-post src/Metis/Metis/bitlinear.py and quant.py, unmodified).

TEST INFRASTRUCTURE ONLY: the timed CPU baseline of the benchmark and a cross-check of the restated
oracle.  BitLinear.split() of the reference cannot run on the CPU (bitlinear.py:800-802 hard-codes
.cuda()), so the layer is put together the way the reference's own tests do it
(tests/test_metis_quant_cache.py:198-208): __new__, then the sub-modules by hand, with the class-level
configuration of LinearLowbitFunction (bitlinear.py:28-73) set to the GRPO defaults
(src/grpo/grpo.py:62-103): NVFP4 round-to-nearest forward, stochastic-rounding backward, mean mode.
"""
from __future__ import annotations

import importlib
import sys
from types import SimpleNamespace

import torch

from . import build_ref

_mods = None


def modules():
    """(bitlinear module, quant module) of the reference, imported under a private name so that they
    never shadow the package's own `Metis` aliases."""
    global _mods
    if _mods is None:
        if not build_ref.available():
            raise RuntimeError("oracle/_ref is empty: run `python -m oracle.build_ref <checkout>` where the reference is present")
        saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "Metis" or k.startswith("Metis.")}
        sys.path.insert(0, str(build_ref.OUT))
        try:
            bl = importlib.import_module("Metis.Metis.bitlinear")
            qt = importlib.import_module("Metis.Metis.quant")
        finally:
            sys.path.remove(str(build_ref.OUT))
            for k in [k for k in sys.modules if k == "Metis" or k.startswith("Metis.")]:
                sys.modules["_reference_" + k] = sys.modules.pop(k)
            sys.modules.update(saved)
        _mods = (bl, qt)
    return _mods


def configure(compute_dtype=torch.float32, stochastic_backward=True, rank=64):
    bl, qt = modules()
    F = bl.LinearLowbitFunction
    rtn, sr = qt.Cast2NVFp4e2m1BlockNOSR, qt.Cast2NVFp4e2m1Block
    back = sr if stochastic_backward else rtn
    F.compute_dtype = compute_dtype
    F.q_forward_input = F.q_forward_weight = rtn
    F.q_backward_input = F.q_backward_weight = F.q_backward_outputgrad = back
    F.enable_activation_svd, F.activation_lowrank_svd, F.activation_lowrank_niter, F.activation_broadcast_dim = True, rank, 0, -1
    F.enable_backward_svd, F.backward_lowrank_svd, F.backward_lowrank_niter, F.backward_broadcast_dim = True, rank, 0, -1
    F.tp_simulate, F.tp_parts, F.metis_mode, F.enable_nv_recipe = False, 1, "mean", False
    return F


def assemble(U, s, V, R, bias=None, dtype=torch.float32, stochastic_backward=True):
    """BitLinear with the given factors: U [N, r], s [r], V [r, K], R [N, K]."""
    bl, _ = modules()
    N, r = U.shape
    K = V.shape[1]
    configure(dtype, stochastic_backward, r)
    args = SimpleNamespace(device="cpu", cache_quantized_weight=False, forward_svd_rank=r)
    layer = bl.BitLinear.__new__(bl.BitLinear)
    torch.nn.Module.__init__(layer)
    layer.args = args
    layer.is_svd_quant = True
    layer.mean_cache = {}
    layer.activation_group = None
    layer._merged_rollout_weight_cache = None
    layer.layer_name = "reference.layer"
    layer.vlinear = bl.LinearLowbit(K, r, bias=False, args=args, storage_dtype=dtype, compute_dtype=dtype)
    layer.ulinear = torch.nn.Linear(r, N, bias=False, dtype=dtype)
    layer.warmup_linear = bl.LinearLowbit(K, N, bias=bias is not None, args=args, storage_dtype=dtype, compute_dtype=dtype)
    layer.s = torch.nn.Parameter(s.to(dtype).clone())
    with torch.no_grad():
        layer.vlinear.weight.copy_(V)
        layer.ulinear.weight.copy_(U)
        layer.warmup_linear.weight.copy_(R)
        if bias is not None:
            layer.warmup_linear.bias.copy_(bias)
    return layer
