"""Generates the golden vectors under tests/golden/ by running the REFERENCE itself.

Run once, in a container that has the reference checked out (it is not needed afterwards and
is never read by the tests, the smoke check or the benchmark):

    python tests/golden/make_golden.py --reference /path/to/fp4-post

What is recorded (all inputs seeded; everything the reference computes is computed by the
reference's own code, imported from <reference>/src):
  quant_cases.npz    x -> Cast2NVFp4e2m1BlockNOSR.quantize_dequantize(x) (quant.py:393-433), plus
                     the packed codes / E4M3 bytes / unit derived from the reference's own
                     intermediates get_scalar (quant.py:437-455) and quant (quant.py:459-466);
                     mean-centred cases go through LinearLowbitFunction.svd_quant(metis_mode="mean")
                     (bitlinear.py:311-336).
  rmsnorm_cases.npz  RMSNorm.forward (src/Metis/models/llama.py:16-31; the class body is executed
                     from the file's text because the module imports packages that are absent)
                     followed by the same quantizer on .float().
  layer_cases.npz    BitLinear forward + backward (bitlinear.py:736-769, 407-513) assembled the way
                     the reference's tests do (tests/test_metis_quant_cache.py:198-208), fp32,
                     round-to-nearest quantizers everywhere, mean mode.
"""
from __future__ import annotations

import argparse
import ast
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LUT = {0: 0, 1: 1, 2: 2, 3: 3, 4: 4, 6: 5, 8: 6, 12: 7}


def derive_packed(Q, x: torch.Tensor):
    """codes / scale bytes / unit from the reference's own intermediates."""
    s = Q.get_scalar(x)
    v = Q.quant(x.clone(), s.clone()) * 2           # in {0, +-1, 2, 3, 4, 6, 8, 12}
    lut = torch.zeros(13, dtype=torch.uint8)
    for k, c in LUT.items():
        lut[k] = c
    mag = lut[v.abs().to(torch.int64)]
    nib = (mag | (torch.signbit(v).to(torch.uint8) << 3)).reshape(-1, x.shape[-1])
    codes = nib[:, 0::2] | (nib[:, 1::2] << 4)
    unit = s.max() / 448
    scales = (s / unit).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.numpy(), scales.numpy(), np.float32(unit.item()), s.numpy()


def quant_inputs():
    g = torch.Generator().manual_seed(0)
    cases = {}
    cases["randn_64x256"] = torch.randn(64, 256, generator=g)
    x = torch.randn(32, 512, generator=g)
    x[:, torch.randperm(512, generator=g)[:5]] *= 20
    cases["outliers_32x512"] = x
    t = torch.distributions.StudentT(3.0)
    torch.manual_seed(1)
    xb = (t.sample((48, 1536)) + 2.0 * torch.randn(1, 1536)).to(torch.bfloat16).float()
    cases["bf16valued_48x1536"] = xb
    cases["weights_128x256"] = 0.02 * torch.randn(128, 256, generator=g)
    # special values: exact ties, zeros, negative zero, tiny and huge blocks
    sp = torch.zeros(8, 64)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    sp[0, 0:16] = ties                 # s == 1 exactly, every element on a rounding tie
    sp[0, 16:32] = ties * 3.0
    sp[1, 0:16] = ties * 1e-3
    sp[1, 16:32] = ties.flip(0) * 7.0
    sp[2, 0:16] = 0.0                  # all-zero block
    sp[2, 16] = -0.0
    sp[2, 17] = 1e-30
    sp[2, 18] = -1e-30
    sp[3, :] = torch.randn(64, generator=g) * 1e-6   # block scales that flush to zero in E4M3
    sp[4, :] = torch.randn(64, generator=g) * 1e4
    sp[5, :] = torch.randn(64, generator=g)
    sp[5, 3] = -0.0
    sp[6, :] = torch.linspace(-6, 6, 64)
    sp[7, :] = torch.linspace(-1, 1, 64) ** 3 * 50
    cases["special_8x64"] = sp
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of decisivemoments/fp4-post (the directory that holds src/)")
    ref = Path(ap.parse_args().reference)
    sys.path.insert(0, str(ref / "src"))
    from Metis.Metis.bitlinear import BitLinear, LinearLowbit, LinearLowbitFunction
    from Metis.Metis.quant import Cast2NVFp4e2m1BlockNOSR as Q

    torch.set_num_threads(1)   # one summation order for the recorded means

    # ---- quantizer ---------------------------------------------------------------------------------
    out = {}
    for name, x in quant_inputs().items():
        codes, scales, unit, bs = derive_packed(Q, x)
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/qdq"] = Q.quantize_dequantize(x.clone()).numpy()
        out[f"{name}/codes"], out[f"{name}/scales"], out[f"{name}/unit"], out[f"{name}/block_scale"] = codes, scales, unit, bs
    # mean-centred (activation path of metis_mode="mean")
    g = torch.Generator().manual_seed(2)
    xm = torch.randn(2, 48, 256, generator=g) + 3.0 * torch.randn(1, 1, 256, generator=g)
    cache = {}
    xhat = LinearLowbitFunction.svd_quant(xm.clone(), quant_func=Q, metis_mode="mean", mean_cache=cache, cache_key="k")
    me, count = cache["k"]
    codes, scales, unit, bs = derive_packed(Q, xm.reshape(-1, 256) - me)
    out["mean_96x256/x"] = xm.reshape(-1, 256).numpy()
    out["mean_96x256/mean"] = me.reshape(-1).numpy()
    out["mean_96x256/qdq"] = xhat.reshape(-1, 256).numpy()
    out["mean_96x256/codes"], out["mean_96x256/scales"], out["mean_96x256/unit"], out["mean_96x256/block_scale"] = codes, scales, unit, bs
    assert count == 96
    np.savez_compressed(HERE / "quant_cases.npz", **out)

    # ---- RMSNorm -> quant --------------------------------------------------------------------------
    src = (ref / "src/Metis/models/llama.py").read_text()
    cls = next(n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == "RMSNorm")
    ns = {"torch": torch, "nn": torch.nn}
    exec(compile(ast.Module(body=[cls], type_ignores=[]), "llama.py:RMSNorm", "exec"), ns)
    RMSNorm = ns["RMSNorm"]
    out = {}
    torch.manual_seed(3)
    t = torch.distributions.StudentT(3.0)
    for name, (rows, cols, gdt) in {"bf16_gbf16_40x1536": (40, 1536, torch.bfloat16),
                                    "bf16_gf32_24x512": (24, 512, torch.float32)}.items():
        x = (t.sample((rows, cols)) + 2.0 * torch.randn(1, cols)).to(torch.bfloat16)
        norm = RMSNorm(cols, eps=1e-6, device="cpu")
        with torch.no_grad():
            norm.weight.copy_(1.0 + 0.1 * torch.randn(cols))
        if gdt == torch.bfloat16:
            norm = norm.to(torch.bfloat16)
        with torch.no_grad():
            y = norm(x)
        yf = y.float()
        codes, scales, unit, bs = derive_packed(Q, yf)
        out[f"{name}/x"] = x.float().numpy()                  # bf16 values, stored widened
        out[f"{name}/gamma"] = norm.weight.detach().float().numpy()
        out[f"{name}/y"] = yf.numpy()
        out[f"{name}/qdq"] = Q.quantize_dequantize(yf.clone()).numpy()
        out[f"{name}/codes"], out[f"{name}/scales"], out[f"{name}/unit"] = codes, scales, unit
    np.savez_compressed(HERE / "rmsnorm_cases.npz", **out)

    # ---- the Metis layer, forward + backward ---------------------------------------------------------
    g = torch.Generator().manual_seed(4)
    B, T, K, N, r = 2, 32, 128, 96, 16
    x = torch.randn(B, T, K, generator=g)
    x[..., torch.randperm(K, generator=g)[:2]] *= 20
    W = 0.02 * torch.randn(N, K, generator=g)
    bias = 0.1 * torch.randn(N, generator=g)
    grad_out = torch.randn(B, T, N, generator=g)
    U, S, Vh = torch.linalg.svd(W, full_matrices=False)
    R = W - U[:, :r] @ torch.diag(S[:r]) @ Vh[:r]
    args = SimpleNamespace(device="cpu", cache_quantized_weight=False, forward_svd_rank=r)
    layer = BitLinear.__new__(BitLinear)
    torch.nn.Module.__init__(layer)
    layer.args = args
    layer.is_svd_quant = True
    layer.mean_cache = {}
    layer.activation_group = None
    layer._merged_rollout_weight_cache = None
    layer.layer_name = "golden.layer"
    layer.vlinear = LinearLowbit(K, r, bias=False, args=args)
    layer.ulinear = torch.nn.Linear(r, N, bias=False)
    layer.warmup_linear = LinearLowbit(K, N, bias=True, args=args)
    layer.s = torch.nn.Parameter(S[:r].clone())
    with torch.no_grad():
        layer.vlinear.weight.copy_(Vh[:r])
        layer.ulinear.weight.copy_(U[:, :r])
        layer.warmup_linear.weight.copy_(R)
        layer.warmup_linear.bias.copy_(bias)
    F = LinearLowbitFunction
    F.compute_dtype = torch.float32
    F.q_forward_input = Q
    F.q_forward_weight = Q
    F.q_backward_input = Q
    F.q_backward_weight = Q
    F.q_backward_outputgrad = Q           # round to nearest so that the record is deterministic
    F.enable_activation_svd = True
    F.activation_lowrank_svd = r
    F.activation_lowrank_niter = 0
    F.activation_broadcast_dim = -1
    F.enable_backward_svd = True
    F.backward_lowrank_svd = r
    F.backward_lowrank_niter = 0
    F.backward_broadcast_dim = -1
    F.tp_simulate = False
    F.tp_parts = 1
    F.metis_mode = "mean"
    F.enable_nv_recipe = False
    xr = x.clone().requires_grad_(True)
    y = layer(xr)
    y.backward(grad_out)
    np.savez_compressed(
        HERE / "layer_cases.npz",
        x=x.numpy(), W=W.numpy(), bias=bias.numpy(), grad_out=grad_out.numpy(), rank=np.int64(r),
        U=U[:, :r].contiguous().numpy(), S=S[:r].numpy(), V=Vh[:r].contiguous().numpy(), R=R.numpy(),
        y=y.detach().numpy(), dx=xr.grad.numpy(), dR=layer.warmup_linear.weight.grad.numpy(),
        dV=layer.vlinear.weight.grad.numpy(), dU=layer.ulinear.weight.grad.numpy(), ds=layer.s.grad.numpy(),
        dbias=layer.warmup_linear.bias.grad.numpy())
    for f in ("quant_cases.npz", "rmsnorm_cases.npz", "layer_cases.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
