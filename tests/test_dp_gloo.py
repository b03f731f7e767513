"""Data-parallel path on two CPU ranks (gloo): sharded tokens, replicated weights, one gradient
all-reduce.  With identity quantizers the layer is linear in the batch, so the all-reduced weight
gradients must equal the single-process gradients of the whole batch."""
import os
import socket
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_layer():
    import fp4_post_b200
    fp4_post_b200.install_reference_aliases()
    from Metis.Metis.bitlinear import BitLinear, LinearLowbit, LinearLowbitFunction as F
    from Metis.Metis.quant import Cast2Fp32
    F.compute_dtype = torch.float32
    for k in ("q_forward_input", "q_forward_weight", "q_backward_input", "q_backward_weight", "q_backward_outputgrad"):
        setattr(F, k, Cast2Fp32)
    F.enable_activation_svd = F.enable_backward_svd = F.enable_nv_recipe = False
    torch.manual_seed(0)
    args = SimpleNamespace(device="cpu", cache_quantized_weight=False, forward_svd_rank=4)
    layer = BitLinear.__new__(BitLinear)
    torch.nn.Module.__init__(layer)
    layer.args, layer.is_svd_quant, layer.mean_cache = args, True, {}
    layer.activation_group, layer._merged_rollout_weight_cache, layer.layer_name = None, None, "dp"
    layer.vlinear = LinearLowbit(16, 4, bias=False, args=args)
    layer.ulinear = torch.nn.Linear(4, 8, bias=False)
    layer.warmup_linear = LinearLowbit(16, 8, bias=True, args=args)
    layer.s = torch.nn.Parameter(torch.rand(4) + 0.5)
    return layer


def _batch():
    g = torch.Generator().manual_seed(1)
    return torch.randn(6, 5, 16, generator=g), torch.randn(6, 5, 8, generator=g)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fp4_post_b200.dp import allreduce_gradients, shard_tokens
        layer = _make_layer()
        x, g = _batch()
        xs, gs = shard_tokens(x, rank, world), shard_tokens(g, rank, world)
        layer(xs).backward(gs)
        nbytes = allreduce_gradients(layer.parameters())
        if rank == 0:
            out.put(({n: p.grad.clone() for n, p in layer.named_parameters()}, nbytes, tuple(xs.shape)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_full_batch_weight_gradients():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    grads, nbytes, shard_shape = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert shard_shape == (3, 5, 16)
    layer = _make_layer()
    x, g = _batch()
    layer(x).backward(g)
    assert nbytes == sum(p.numel() * 4 for p in layer.parameters())
    for name, p in layer.named_parameters():
        torch.testing.assert_close(grads[name], p.grad, rtol=1e-5, atol=1e-5, msg=name)


def _reducer_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fp4_post_b200.dp import GradientReducer
        red = GradientReducer(small_bytes=1024)
        big = torch.full((64, 64), float(rank + 1))             # 16 KiB: its own asynchronous all-reduce
        small = [torch.full((5,), float(rank + 1)), torch.full((3, 2), 10.0 * (rank + 1))]
        red.ready(big)
        for t in small:
            red.ready(t)
        red.ready(None)                                           # an absent gradient (no bias) is skipped
        red.flush()
        # every rank draws its stochastic-rounding bits from its own Philox key
        from fp4_post_b200.Metis.Metis.quant import Cast2NVFp4e2m1Block, random_lane
        keys = torch.tensor([Cast2NVFp4e2m1Block.philox_key()], dtype=torch.int64)
        with random_lane(1):
            keys = torch.cat([keys, torch.tensor([Cast2NVFp4e2m1Block.philox_key()], dtype=torch.int64)])
        gathered = [torch.zeros_like(keys) for _ in range(world)]
        dist.all_gather(gathered, keys)
        if rank == 0:
            out.put((big.clone(), [t.clone() for t in small], red.bytes_reduced, torch.stack(gathered)))
    finally:
        dist.destroy_process_group()


def test_gradient_reducer_sums_large_tensors_in_place_and_small_ones_in_one_bucket():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_reducer_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    big, small, nbytes, keys = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert keys.unique().numel() == 4                 # 2 ranks x 2 random lanes: four different Philox keys
    assert torch.equal(big, torch.full((64, 64), 3.0))
    assert torch.equal(small[0], torch.full((5,), 3.0)) and torch.equal(small[1], torch.full((3, 2), 30.0))
    assert nbytes == (64 * 64 + 5 + 6) * 4


def test_gradient_reducer_is_inert_without_a_process_group():
    from fp4_post_b200.dp import GradientReducer
    red = GradientReducer()
    t = torch.ones(4)
    red.ready(t)
    red.flush()
    assert torch.equal(t, torch.ones(4)) and red.bytes_reduced == 0


def test_sharding_covers_the_batch_once_and_allreduce_is_a_noop_without_a_group():
    from fp4_post_b200.dp import allreduce_gradients, shard_tokens
    x = torch.arange(7 * 3).reshape(7, 3)
    parts = [shard_tokens(x, r, 3) for r in range(3)]
    assert torch.equal(torch.cat(parts), x) and [p.shape[0] for p in parts] == [2, 2, 3]
    assert allreduce_gradients([torch.nn.Parameter(torch.zeros(2))]) == 0


class _Adopting(torch.autograd.Function):
    """y = x * w whose backward hands w's gradient to the reducer instead of to autograd (what the fused
    Metis backward does with GradientReducer(across_layers=True))."""

    @staticmethod
    def forward(ctx, x, w, reducer):
        ctx.save_for_backward(x, w)
        ctx.w_param, ctx.reducer = w, reducer
        return x * w

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        ctx.reducer.adopt(ctx.w_param, (gy * x).sum(0))
        ctx.reducer.finish_at_end_of_backward()
        return gy * w, None, None


def _across_layers_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fp4_post_b200.dp import GradientReducer
        red = GradientReducer(small_bytes=64, across_layers=True)
        w1 = torch.nn.Parameter(torch.full((32,), 2.0))          # 128 bytes: its own collective
        w2 = torch.nn.Parameter(torch.full((4,), 3.0))           # 16 bytes: the flat bucket
        x = torch.full((3, 32), float(rank + 1), requires_grad=True)
        h = _Adopting.apply(x, w1, red)                           # two "layers": both collectives are waited for once,
        y = _Adopting.apply(h[:, :4], w2, red)                    # after the whole backward pass
        assert not red.pending()
        y.sum().backward()
        assert not red.pending() and x.grad is not None
        if rank == 0:
            out.put((w1.grad.clone(), w2.grad.clone()))
    finally:
        dist.destroy_process_group()


def test_reducer_across_layers_fills_grad_itself_and_waits_once_at_the_end_of_backward():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_across_layers_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    g1, g2 = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # rank r: x = r + 1; dw2 = sum over 3 rows of h = 3 * 2 (r+1) -> summed over ranks 6 * (1 + 2) = 18
    assert torch.equal(g2, torch.full((4,), 18.0))
    # dw1 = sum over rows of gy1 * x with gy1 = w2 on the first 4 columns (0 elsewhere): 3 * 3 * (r+1) -> 27
    want = torch.zeros(32)
    want[:4] = 27.0
    assert torch.equal(g1, want)
