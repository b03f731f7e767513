"""Packed NVFP4 export of a Metis state dict through the sm_100a quantizer (fp4_post_b200/checkpoint.py)."""
import pytest
import torch

import fp4_post_b200
from fp4_post_b200 import checkpoint as CK

fp4_post_b200.install_reference_aliases()

from Metis.Metis.bitlinear import BitLinear  # noqa: E402
from Metis.Metis.quant import Cast2NVFp4e2m1BlockNOSR  # noqa: E402
from grpo.grpo import MetisArgs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def test_export_then_import_gives_the_quantized_weights_of_the_forward_pass():
    torch.manual_seed(0)
    args = MetisArgs(forward_svd_rank=32)
    args.device = "cuda"
    block = torch.nn.Module()
    block.proj = BitLinear(256, 192, args=args, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    block.proj.layer_name = "proj"
    block.proj.split()
    block.norm = torch.nn.LayerNorm(256)
    sd = block.state_dict()
    packed = CK.export_packed(sd)
    for child in ("warmup_linear", "vlinear"):
        key = f"proj.{child}.weight"
        assert key not in packed
        rows, cols = sd[key].shape
        assert packed[f"{key}.nvfp4.codes"].shape == (rows, cols // 2) and packed[f"{key}.nvfp4.codes"].dtype == torch.uint8
        assert packed[f"{key}.nvfp4.scales"].numel() == rows * cols // 16
        assert packed[f"{key}.nvfp4.shape"].tolist() == [rows, cols]
    assert torch.equal(packed["proj.ulinear.weight"], sd["proj.ulinear.weight"]) and "norm.weight" in packed
    # 0.5 + 1/16 bytes per weight instead of 2
    nbytes = lambda d, k: sum(v.numel() * v.element_size() for n, v in d.items() if n.startswith(k))
    assert nbytes(packed, "proj.warmup_linear.weight") < 0.3 * nbytes(sd, "proj.warmup_linear.weight")

    restored = CK.import_packed(packed, dtype=torch.bfloat16)
    assert set(restored) == set(sd)
    for child in ("warmup_linear", "vlinear"):
        key = f"proj.{child}.weight"
        want = Cast2NVFp4e2m1BlockNOSR.quantize_dequantize(sd[key].cuda()).cpu()
        assert torch.equal(restored[key], want), key
    block.load_state_dict(restored)                      # same keys, same shapes: loads into the module
