"""State-dict bridge (fp4_post_b200/checkpoint.py): merging BitLinear factors into plain weights with the
reference converter's key contract (tools/convert_bitlinear_to_standard.py:80-172), and the packed
NVFP4 export format against the oracle and the reference's own fake-quant vectors."""
from collections import OrderedDict

import numpy as np
import pytest
import torch

from fp4_post_b200 import checkpoint as CK
from oracle import nvfp4_oracle as O


def _state_dict():
    g = torch.Generator().manual_seed(0)
    sd = OrderedDict()
    sd["model.embed.weight"] = torch.randn(10, 8, generator=g)
    # a full BitLinear: U [N, r], s [r], V [r, K], residual [N, K], residual bias
    sd["model.layers.0.q_proj.ulinear.weight"] = torch.randn(12, 4, generator=g).to(torch.bfloat16)
    sd["model.layers.0.q_proj.vlinear.weight"] = torch.randn(4, 32, generator=g).to(torch.bfloat16)
    sd["model.layers.0.q_proj.s"] = torch.rand(4, generator=g).to(torch.bfloat16)
    sd["model.layers.0.q_proj.warmup_linear.weight"] = torch.randn(12, 32, generator=g).to(torch.bfloat16)
    sd["model.layers.0.q_proj.warmup_linear.bias"] = torch.randn(12, generator=g).to(torch.bfloat16)
    # low-rank only, bias on the U branch
    sd["model.layers.0.k_proj.ulinear.weight"] = torch.randn(6, 2, generator=g)
    sd["model.layers.0.k_proj.ulinear.bias"] = torch.randn(6, generator=g)
    sd["model.layers.0.k_proj.vlinear.weight"] = torch.randn(2, 32, generator=g)
    sd["model.layers.0.k_proj.s"] = torch.rand(2, generator=g)
    # residual only (rank 0)
    sd["model.layers.0.o_proj.warmup_linear.weight"] = torch.randn(8, 16, generator=g)
    # incomplete: skipped, its tensors dropped like the reference tool does
    sd["model.layers.0.up_proj.vlinear.weight"] = torch.randn(2, 16, generator=g)
    sd["model.norm.weight"] = torch.ones(8)
    return sd


def test_merge_follows_the_reference_key_contract():
    sd = _state_dict()
    report = []
    out = CK.merge_state_dict(sd, report=report)
    assert CK.bitlinear_prefixes(sd) == {"model.layers.0.q_proj", "model.layers.0.k_proj", "model.layers.0.o_proj",
                                         "model.layers.0.up_proj"}
    p = "model.layers.0.q_proj"
    want = (sd[f"{p}.ulinear.weight"].float() @ torch.diag(sd[f"{p}.s"].float()) @ sd[f"{p}.vlinear.weight"].float()
            + sd[f"{p}.warmup_linear.weight"].float()).to(torch.bfloat16)
    assert out[f"{p}.weight"].dtype == torch.bfloat16
    torch.testing.assert_close(out[f"{p}.weight"].float(), want.float(), rtol=0, atol=2 ** -6)
    assert torch.equal(out[f"{p}.bias"], sd[f"{p}.warmup_linear.bias"])
    k = "model.layers.0.k_proj"
    want_k = sd[f"{k}.ulinear.weight"] @ torch.diag(sd[f"{k}.s"]) @ sd[f"{k}.vlinear.weight"]
    torch.testing.assert_close(out[f"{k}.weight"], want_k, rtol=1e-5, atol=1e-6)
    assert torch.equal(out[f"{k}.bias"], sd[f"{k}.ulinear.bias"])
    assert torch.equal(out["model.layers.0.o_proj.weight"], sd["model.layers.0.o_proj.warmup_linear.weight"])
    assert "model.layers.0.o_proj.bias" not in out
    assert not any(key.startswith("model.layers.0.up_proj") for key in out)
    assert not any(".ulinear." in key or ".vlinear." in key or ".warmup_linear." in key or key.endswith(".s") for key in out)
    assert torch.equal(out["model.embed.weight"], sd["model.embed.weight"]) and "model.norm.weight" in out
    assert len(report) == 4 and any("skipped" in line for line in report)
    # order: merged modules first (sorted), then the untouched tensors in their original order
    assert list(out)[-2:] == ["model.embed.weight", "model.norm.weight"]


def test_merge_casts_floating_tensors_only():
    sd = _state_dict()
    sd["model.step"] = torch.tensor(7)
    out = CK.merge_state_dict(sd, target_dtype=torch.float16)
    assert out["model.layers.0.q_proj.weight"].dtype == torch.float16 and out["model.norm.weight"].dtype == torch.float16
    assert out["model.step"].dtype == torch.int64


def test_packed_decoder_matches_the_oracle_and_the_reference_vectors(quant_golden):
    g = quant_golden["weights_128x256"]
    codes, scales, unit, _ = O.quantize(g["x"])
    got = CK.dequantize_packed(torch.from_numpy(codes), torch.from_numpy(scales), torch.tensor([unit]), g["x"].shape)
    assert np.array_equal(got.numpy(), g["qdq"])               # the reference's own fake-quant output


def test_import_packed_restores_a_standard_state_dict(quant_golden):
    g = quant_golden["weights_128x256"]
    codes, scales, unit, _ = O.quantize(g["x"])
    sd = OrderedDict()
    key = "model.layers.3.down_proj.warmup_linear.weight"
    sd[f"{key}.nvfp4.codes"] = torch.from_numpy(codes)
    sd[f"{key}.nvfp4.scales"] = torch.from_numpy(scales)
    sd[f"{key}.nvfp4.unit"] = torch.tensor([unit])
    sd[f"{key}.nvfp4.shape"] = torch.tensor(list(g["x"].shape))
    sd["model.layers.3.down_proj.s"] = torch.ones(4)
    out = CK.import_packed(sd, dtype=torch.float32)
    assert set(out) == {key, "model.layers.3.down_proj.s"}
    assert np.array_equal(out[key].numpy(), g["qdq"])
    del sd[f"{key}.nvfp4.unit"]
    with pytest.raises(KeyError):
        CK.import_packed(sd)
