"""A whole forward + backward of the Metis layer captured into a CUDA graph (fp4_post_b200.graphs):
the replay must compute what the eager step computes, follow the static inputs, and draw fresh
stochastic-rounding bits on every replay (the Philox offset lives on the device)."""
import pytest
import torch

import fp4_post_b200
from fp4_post_b200 import ops
from fp4_post_b200.graphs import GraphedStep

fp4_post_b200.install_reference_aliases()

from Metis.Metis.bitlinear import BitLinear, LinearLowbitFunction  # noqa: E402
from Metis.Metis.quant import Cast2NVFp4e2m1Block  # noqa: E402
from grpo.grpo import MetisArgs  # noqa: E402
from gpu_helpers import rel_l2  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _lib(built_library):
    return built_library


def make_layer(cache):
    torch.manual_seed(7)
    args = MetisArgs(forward_svd_rank=64, activation_lowrank_svd=64, backward_lowrank_svd=64, cache_quantized_weight=cache)
    args.device = DEV
    layer = BitLinear(512, 384, args=args, bias=True, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.layer_name = "graphed"
    layer.split()
    return layer.to(DEV)


def test_replay_matches_eager_follows_the_inputs_and_redraws_the_rounding_bits():
    layer = make_layer(cache=False)          # weight quantization inside the graph: safe when weights change
    assert LinearLowbitFunction.q_backward_outputgrad is Cast2NVFp4e2m1Block      # stochastic backward (GRPO default)
    params = list(layer.parameters())
    x = torch.randn(2, 256, 512, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    g = torch.randn(2, 256, 384, device=DEV, dtype=torch.bfloat16)

    def step():
        for p in params:
            p.grad = None
        x.grad = None
        y = layer(x)
        y.backward(g)
        return y, x.grad, layer.warmup_linear.weight.grad

    graphed = GraphedStep(step)
    y1, gx1, gw1 = (t.clone() for t in graphed())
    y2, gx2, gw2 = (t.clone() for t in graphed())
    y_e, gx_e, gw_e = (t.clone() for t in step())
    # forward: round to nearest everywhere, so eager and both replays agree bit for bit
    assert torch.equal(y1, y2) and torch.equal(y1, y_e)
    # backward: stochastic rounding with a fresh Philox offset per call, in replays too
    assert not torch.equal(gx1, gx2) and not torch.equal(gw1, gw2)
    for a in (gx1, gx2):
        assert rel_l2(a.float().cpu().numpy(), gx_e.float().cpu().numpy()) <= 0.2
    for a in (gw1, gw2):
        assert rel_l2(a.float().cpu().numpy(), gw_e.float().cpu().numpy()) <= 0.2

    # new contents of the static input tensors, same graph
    with torch.no_grad():
        x.copy_(torch.randn_like(x))
        g.copy_(torch.randn_like(g))
    y3 = graphed()[0].clone()
    assert not torch.equal(y3, y1)
    assert torch.equal(y3, step()[0])

    # the weights changed: with the cache off the replay re-quantizes them
    with torch.no_grad():
        layer.warmup_linear.weight.mul_(1.5)
    y4 = graphed()[0].clone()
    assert torch.equal(y4, step()[0]) and not torch.equal(y4, y3)


def test_stochastic_quantizer_counter_advances_once_per_call():
    ctr = torch.full((1,), 5, dtype=torch.int64, device=DEV)
    x = torch.randn(64, 256, device=DEV, dtype=torch.bfloat16)
    a = ops.nvfp4_quantize(x, stochastic=True, seed=1, offset_counter=ctr)
    b = ops.nvfp4_quantize(x, stochastic=True, seed=1, offset_counter=ctr)
    torch.cuda.synchronize()
    assert ctr.item() == 7
    assert not torch.equal(a.codes, b.codes)
    # the same bits as the host-side offset of the same value
    c = ops.nvfp4_quantize(x, stochastic=True, seed=1, offset=5)
    assert torch.equal(a.codes, c.codes) and torch.equal(a.scales, c.scales)
    with pytest.raises(ValueError):
        ops.nvfp4_quantize(x, stochastic=True, offset_counter=torch.zeros(1, dtype=torch.int32, device=DEV))
