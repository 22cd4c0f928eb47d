"""Expert-parallel MoE layer on GPUs.  With one visible GPU the layer runs with world size 1 (every
"peer" store lands in the rank's own buffers), which still exercises dispatch, the signal/wait pair,
the masked grouped GEMMs, the return path and the weighted sum.  With two or more GPUs a second test
spawns one process per GPU and checks every rank's output against the single-process oracle."""
import os

import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close

pytestmark = pytest.mark.gpu


def ep_case(world, t_per_rank, h, i, e, topk, seed):
    from kb_nano_b200 import inputs
    xs = [inputs.activations(t_per_rank, h, seed=seed + r) for r in range(world)]
    routes = [inputs.route_sigmoid_topk(inputs.router_logits(t_per_rank, e, seed=seed + r), topk) for r in range(world)]
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=seed + 100, std=0.05)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=seed + 200, std=0.05)
    return xs, routes, (w13_q, w13_s, w2_q, w2_s)


def inputs_logits(rank, t, e, seed):
    from kb_nano_b200 import inputs
    return inputs.router_logits(t, e, seed=seed + rank)


def test_ep_world1_matches_oracle(cuda_dev):
    from kb_nano_b200 import ep, ops
    t, h, i, e, topk = 96, 512, 256, 16, 4
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(1, t, h, i, e, topk, seed=3)
    d = cuda_dev
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    ref = to.moe_layer(xs[0], w13_q, w13_s, w2_q, w2_s, routes[0][0], routes[0][1])
    # max_m = 64 is not a multiple of 128: the expert GEMMs use the fp32-scale kernels
    slow = ep.EpMoe(0, 1, e, h, i, max_tokens=128, topk=topk, max_m=64, device=d)
    out = slow.forward(xs[0].to(d), routes[0][1].to(d), routes[0][0].to(d), *wd)
    slow.check()
    assert_gemm_close(out.cpu(), ref, "EP world=1, fp32-scale GEMMs")
    slow.close()
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=128, topk=topk, max_m=128, device=d)
    for it in range(3):        # repeated calls reuse buffers, counters and flags
        out = layer.forward(xs[0].to(d), routes[0][1].to(d), routes[0][0].to(d), *[wd[j] for j in (0, 1, 2, 3)])
        layer.check()
        assert ops.gemm_status(d) == 0
        assert_gemm_close(out.cpu(), ref, f"EP world=1, call {it}")
    # BASELINE configs[3]: "output is checked against the single-GPU result" -- the expert-contiguous pipeline on one
    # GPU gives the same bits (same per-row arithmetic, same slot order in the weighted sum)
    from kb_nano_b200 import moe
    single = moe.fused_experts_fp8(xs[0].to(d), wd[0], wd[2], routes[0][0].to(d), routes[0][1].to(d), e, wd[1], wd[3])
    assert torch.equal(out.view(torch.int16), single.view(torch.int16))
    # fewer tokens than max_tokens, then none at all
    out = layer.forward(xs[0][:5].to(d), routes[0][1][:5].to(d), routes[0][0][:5].to(d), *wd)
    assert_gemm_close(out.cpu(), ref[:5], "EP world=1, 5 tokens")
    out = layer.forward(xs[0][:0].to(d), routes[0][1][:0].to(d), routes[0][0][:0].to(d), *wd)
    assert out.shape == (0, h)
    layer.check()
    layer.close()


def test_ep_many_rows_per_expert_uses_the_plain_operand_order(cuda_dev):
    """256 tokens x top-2 over 4 experts: about 128 rows per expert, more than the layer expects the swapped operand
    order of the masked GEMMs to pay for, so it runs them in the plain order; same bits as the one-GPU pipeline."""
    from kb_nano_b200 import ep, moe
    t, h, i, e, topk = 256, 512, 256, 4, 2
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(1, t, h, i, e, topk, seed=41)
    d = cuda_dev
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=t, topk=topk, max_m=256, device=d)
    out = layer.forward(xs[0].to(d), routes[0][1].to(d), routes[0][0].to(d), *wd)
    layer.check()
    ref = to.moe_layer(xs[0], w13_q, w13_s, w2_q, w2_s, routes[0][0], routes[0][1])
    assert_gemm_close(out.cpu(), ref, "EP world=1, 128 rows per expert")
    single = moe.fused_experts_fp8(xs[0].to(d), wd[0], wd[2], routes[0][0].to(d), routes[0][1].to(d), e, wd[1], wd[3])
    assert torch.equal(out.view(torch.int16), single.view(torch.int16))
    # the same layer with a handful of tokens takes the swapped order: same bits again
    out5 = layer.forward(xs[0][:5].to(d), routes[0][1][:5].to(d), routes[0][0][:5].to(d), *wd)
    layer.check()
    single5 = moe.fused_experts_fp8(xs[0][:5].to(d), wd[0], wd[2], routes[0][0][:5].to(d), routes[0][1][:5].to(d), e, wd[1], wd[3])
    assert torch.equal(out5.view(torch.int16), single5.view(torch.int16))
    layer.close()


def test_ep_forward_replays_from_a_cuda_graph(cuda_dev):
    """kb-nano runs decode steps from CUDA graphs (infra/engine.py:2410-2427): the layer's step counter lives on the
    device, so a captured forward can be replayed with new inputs in the same buffers."""
    from kb_nano_b200 import ep
    t, h, i, e, topk = 32, 512, 256, 16, 4
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(3, t, h, i, e, topk, seed=21)
    d = cuda_dev
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=t, topk=topk, max_m=128, device=d)
    x, tw, ti = xs[0].to(d), routes[0][0].to(d).contiguous(), routes[0][1].to(d).contiguous()
    out = torch.empty(t, h, dtype=torch.bfloat16, device=d)
    layer.forward(x, ti, tw, *wd, out=out)                 # warm-up outside the capture (table, attributes, packed scales)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer.forward(x, ti, tw, *wd, out=out)
    for r in range(3):
        x.copy_(xs[r].to(d))
        tw.copy_(routes[r][0].to(d))
        ti.copy_(routes[r][1].to(d))
        graph.replay()
        layer.check()
        ref = to.moe_layer(xs[r], w13_q, w13_s, w2_q, w2_s, routes[r][0], routes[r][1])
        assert_gemm_close(out.cpu(), ref, f"graph replay {r}")
    eager = layer.forward(x, ti, tw, *wd).clone()          # eager calls and replays interleave
    graph.replay()
    assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
    layer.close()


@pytest.mark.parametrize("depth,copy_streams", [(2, 2), (2, 1), (1, 1), (3, 2)])
def test_ep_host_pipeline_matches_forward(cuda_dev, depth, copy_streams):
    """Host-resident inputs and results: the pipeline's staged copies on side streams give the bits of forward() on
    device tensors, step after step over its rotating buffers, eagerly and replayed from a CUDA graph."""
    from kb_nano_b200 import ep
    t, h, i, e, topk = 32, 512, 256, 16, 4
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(5, t, h, i, e, topk, seed=31)
    d = cuda_dev
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=t, topk=topk, max_m=128, device=d)
    want = [layer.forward(xs[r].to(d), routes[r][1].to(d), routes[r][0].to(d), *wd).cpu() for r in range(5)]
    pipe = ep.EpMoeHostPipeline(layer, depth=depth, copy_streams=copy_streams)
    bufs = [pipe.new_host_buffers() for _ in range(5)]
    for r, (blob, _) in enumerate(bufs):
        pipe.pack(blob, xs[r], routes[r][0], routes[r][1])
    pipe.begin()
    for blob, hout in bufs:
        pipe.submit(blob, hout, *wd)
    pipe.join()
    torch.cuda.synchronize()
    layer.check()
    for r, (_, hout) in enumerate(bufs):
        assert torch.equal(hout.view(torch.int16), want[r].view(torch.int16)), f"eager step {r}"
        hout.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pipe.begin()
        for blob, hout in bufs:
            pipe.submit(blob, hout, *wd)
        pipe.join()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    layer.check()
    for r, (_, hout) in enumerate(bufs):
        assert torch.equal(hout.view(torch.int16), want[r].view(torch.int16)), f"replayed step {r}"
    with pytest.raises(ValueError):
        pipe.submit(torch.empty(pipe.blob_bytes, dtype=torch.uint8), bufs[0][1], *wd)      # not pinned
    layer.close()


@pytest.mark.parametrize("e,topk,scoring,n_group,topk_group,use_bias,bf16_logits", [
    (16, 4, "softmax", 1, 1, False, False),          # TopKSoftmax-style routing (Qwen3 / Mixtral layers)
    (64, 6, "sigmoid", 8, 3, True, True),            # GroupedTopK-style routing on bf16 logits (DeepSeek layer)
    (256, 8, "sigmoid", 8, 4, True, False),
])
def test_ep_forward_routed_equals_route_then_forward(cuda_dev, e, topk, scoring, n_group, topk_group, use_bias, bf16_logits):
    """Routing inside the dispatch kernel: the same choice as the stand-alone routing kernel, bit for bit, and the same
    layer output as routing first and calling forward() with the result; also replayed from a CUDA graph."""
    from kb_nano_b200 import ep, inputs, ops
    t, h, i = 48, 512, 256
    d = cuda_dev
    x = inputs.activations(t, h, seed=1).to(d)
    lg = inputs.router_logits(t, e, seed=2).to(d)
    lg = lg.to(torch.bfloat16) if bf16_logits else lg
    bias = (0.1 * torch.randn(e, generator=torch.Generator().manual_seed(3))).to(d) if use_bias else None
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=4, std=0.05)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=5, std=0.05)
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    route = dict(scoring=scoring, bias=bias, n_group=n_group, topk_group=topk_group, renormalize=True, scale=1.5, round_bf16=bf16_logits)
    tw, ti = ops.moe_route_topk(lg, topk, **route)
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=64, topk=topk, max_m=128, device=d)
    want = layer.forward(x, ti, tw, *wd).clone()
    got = layer.forward_routed(x, lg, *wd, **route)
    layer.check()
    rw, ri = layer.last_routing(t)
    assert torch.equal(ri, ti) and torch.equal(rw.view(torch.int32), tw.view(torch.int32))
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    out = torch.empty_like(got)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer.forward_routed(x, lg, *wd, out=out, **route)
    graph.replay()
    layer.check()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    with pytest.raises(ValueError):
        layer.forward_routed(x, lg[:, :8].contiguous(), *wd, **route)
    layer.close()


def test_ep_overflow_is_reported_not_fatal(cuda_dev):
    """More rows for one expert than max_m: the status word says so and the context stays usable."""
    from kb_nano_b200 import ep
    t, h, i, e, topk = 64, 256, 128, 4, 1
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(1, t, h, i, e, topk, seed=5)
    d = cuda_dev
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=64, topk=topk, max_m=8, device=d)
    ids = torch.zeros(t, 1, dtype=torch.int32)        # all 64 tokens to expert 0, room for 8
    layer.forward(xs[0].to(d), ids.to(d), torch.ones(t, 1).to(d), w13_q.to(d), w13_s.to(d), w2_q.to(d), w2_s.to(d))
    st = layer.status()
    assert st["code"] == 10 and st["detail"] == 0
    with pytest.raises(ep.EpStatusError):
        layer.check()
    # the report is cleared on request and a well-formed step then passes its check
    layer.clear_status()
    ids = (torch.arange(t, dtype=torch.int32) % e).view(t, 1)     # 16 tokens per expert would still overflow: send 8 x 4
    layer.forward(xs[0][:32].to(d), ids[:32].to(d), torch.ones(32, 1).to(d), w13_q.to(d), w13_s.to(d), w2_q.to(d), w2_s.to(d))
    layer.check()
    layer.close()


def test_ep_wait_for_a_silent_rank_times_out(cuda_dev):
    """A world of two in which rank 1 never runs (its handle is all zero, so its slots alias this rank's own
    buffer): the waits for its dispatch and combine signals give up after their time limit and record
    {code 20, phase, peer 1}; nothing faults and the context and the GPU stay usable."""
    import time
    from kb_nano_b200 import ep
    t, h, i, e, topk = 16, 256, 128, 8, 2
    xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(1, t, h, i, e, topk, seed=9)
    d = cuda_dev
    layer = ep.EpMoe(0, 2, e, h, i, max_tokens=t, topk=topk, max_m=128, device=d, handles=b"\x01" * 64 + b"\x00" * 64)
    tw, ti = routes[0]
    t0 = time.time()
    layer.forward(xs[0].to(d), ti.to(d), tw.to(d), w13_q[: e // 2].to(d), w13_s[: e // 2].to(d), w2_q[: e // 2].to(d), w2_s[: e // 2].to(d))
    st = layer.status()
    assert st["code"] == 20 and st["phase"] == 1 and st["peer"] == 1, st
    assert time.time() - t0 < 30
    with pytest.raises(ep.EpStatusError):
        layer.check()
    layer.close()
    # the device still works
    assert float(torch.ones(8, device=d).sum()) == 8.0


def _ep_worker(rank, world, port, t, h, i, e, topk, seed, q):
    import torch.distributed as dist
    from kb_nano_b200 import ep, ops
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    d = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=d)
    try:
        xs, routes, (w13_q, w13_s, w2_q, w2_s) = ep_case(world, t, h, i, e, topk, seed)
        lo, hi = ep.expert_range(rank, world, e)
        layer = ep.EpMoe(rank, world, e, h, i, max_tokens=t, topk=topk, max_m=256, device=d)   # 8 ranks x 64 tokens x 4 slots over 16 experts: 128 rows per expert on average
        loc = [w[lo:hi].contiguous().to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
        ref = to.moe_layer(xs[rank], w13_q, w13_s, w2_q, w2_s, routes[rank][0], routes[rank][1])
        ok, msg = True, ""
        for it in range(3):
            out = layer.forward(xs[rank].to(d), routes[rank][1].to(d), routes[rank][0].to(d), *loc)
            st = layer.status()
            if st["code"] != 0 or ops.gemm_status(d) != 0:
                ok, msg = False, f"status {st}"
                break
            try:
                assert_gemm_close(out.cpu(), ref, f"rank {rank} call {it}")
            except AssertionError as ex:
                ok, msg = False, str(ex)
                break
        if ok:
            # routing inside the dispatch kernel, from the logits whose sigmoid top-k is this rank's routing (the router
            # weights may differ from torch's in the last place, so the tolerance applies, not bit equality)
            lg = inputs_logits(rank, t, e, seed).to(d)
            got = layer.forward_routed(xs[rank].to(d), lg, *loc, scoring="sigmoid", renormalize=True)
            try:
                assert layer.status()["code"] == 0, layer.status()
                assert_gemm_close(got.cpu(), ref, f"rank {rank} forward_routed")
            except AssertionError as ex:
                ok, msg = False, str(ex)
        if ok:
            # the same tokens through the one-GPU pipeline with all experts on this GPU: identical bits
            from kb_nano_b200 import moe
            allw = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
            single = moe.fused_experts_fp8(xs[rank].to(d), allw[0], allw[2], routes[rank][0].to(d), routes[rank][1].to(d), e, allw[1], allw[3])
            if not torch.equal(out.view(torch.int16), single.view(torch.int16)):
                ok, msg = False, f"rank {rank}: expert-parallel result differs from the single-GPU result in {int((out != single).sum())} elements"
        dist.barrier()
        layer.close()
        q.put((rank, ok, msg))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_multi_gpu_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + world
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, 64, 512, 256, 16, 4, 11, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    results = [q.get(timeout=5) for _ in range(world)]
    for p in procs:
        assert p.exitcode == 0
    for rank, ok, msg in sorted(results):
        assert ok, f"rank {rank}: {msg}"
