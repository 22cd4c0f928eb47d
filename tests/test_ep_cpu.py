"""Host-side logic of the expert-parallel layer with two gloo ranks on CPU: the placement rule
(`ep.expert_range`, `ep.plan`) that the dispatch kernel applies, the 64-byte handle exchange pattern,
and that a layer computed as "each rank runs its own experts on the rows routed to it, results go back
to the token's rank and are summed in slot order" equals the single-process oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import torch_oracle as to
from tests.util import assert_gemm_close


def _case(world, t, h, i, e, topk, seed):
    from kb_nano_b200 import inputs
    xs = [inputs.activations(t, h, seed=seed + r) for r in range(world)]
    routes = [inputs.route_softmax_topk(inputs.router_logits(t, e, seed=seed + r), topk) for r in range(world)]
    w13 = inputs.expert_weights(e, 2 * i, h, seed=seed + 100, std=0.05)
    w2 = inputs.expert_weights(e, h, i, seed=seed + 200, std=0.05)
    return xs, routes, w13, w2


def _worker(rank, world, port, q):
    from kb_nano_b200 import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        t, h, i, e, topk = 12, 256, 128, 8, 2
        xs, routes, (w13_q, w13_s), (w2_q, w2_s) = _case(world, t, h, i, e, topk, seed=9)
        lo, hi = ep.expert_range(rank, world, e)
        # handle exchange as EpMoe does it: fixed-size blobs gathered in rank order
        blobs = [None] * world
        dist.all_gather_object(blobs, bytes([rank]) * 64)
        assert [b[0] for b in blobs] == list(range(world)) and all(len(b) == 64 for b in blobs)
        # dispatch: quantised rows go to the rank that owns their expert
        a_q, a_s = to.quant_1x128(xs[rank])
        dst, le = ep.plan(routes[rank][1], world, e)
        send = [[] for _ in range(world)]
        for tok in range(t):
            for s in range(topk):
                send[int(dst[tok, s])].append((rank, tok, s, int(le[tok, s]), a_q[tok].view(torch.uint8).clone(), a_s[tok].clone()))
        gathered = [None] * world
        dist.all_gather_object(gathered, send)
        mine = [row for src in gathered for row in src[rank]]
        # local experts in the masked layout, row order = arrival order
        back = [[] for _ in range(world)]
        for l in range(hi - lo):
            rows = [r for r in mine if r[3] == l]
            if not rows:
                continue
            aq = torch.stack([r[4] for r in rows]).view(torch.float8_e4m3fn)
            asc = torch.stack([r[5] for r in rows])
            h1 = (to.dequant_rows(aq, asc) @ to.dequant_blocks(w13_q[lo + l], w13_s[lo + l]).t()).to(torch.bfloat16)
            q2, s2 = to.silu_mul_quant_1x128(h1)
            h2 = (to.dequant_rows(q2, s2) @ to.dequant_blocks(w2_q[lo + l], w2_s[lo + l]).t()).to(torch.bfloat16)
            for r, y in zip(rows, h2):
                back[r[0]].append((r[1], r[2], y))
        returned = [None] * world
        dist.all_gather_object(returned, back)
        comb = torch.zeros(t, topk, h, dtype=torch.bfloat16)
        for src in returned:
            for tok, s, y in src[rank]:
                comb[tok, s] = y
        out = (comb.float() * routes[rank][0].unsqueeze(-1)).sum(1).to(torch.bfloat16)
        ref = to.moe_layer(xs[rank], w13_q, w13_s, w2_q, w2_s, routes[rank][0], routes[rank][1])
        # per-rank view of the oracle: the layer restricted to this rank's experts, summed over ranks
        part = to.moe_layer(xs[0], w13_q, w13_s, w2_q, w2_s, routes[0][0], routes[0][1], experts=range(lo, hi)).float()
        dist.all_reduce(part)
        full0 = to.moe_layer(xs[0], w13_q, w13_s, w2_q, w2_s, routes[0][0], routes[0][1]).float()
        ok = True
        msg = ""
        try:
            assert_gemm_close(out, ref, f"rank {rank} emulated EP")
            assert_gemm_close(part.to(torch.bfloat16), full0.to(torch.bfloat16), "sum of per-rank partial layers")
        except AssertionError as ex:
            ok, msg = False, str(ex)
        q.put((rank, ok, msg))
    finally:
        dist.destroy_process_group()


def test_expert_placement_rule():
    from kb_nano_b200 import ep
    assert ep.expert_range(0, 8, 256) == (0, 32) and ep.expert_range(7, 8, 256) == (224, 256)
    with pytest.raises(ValueError):
        ep.expert_range(0, 3, 256)
    ids = torch.tensor([[0, 31, 32], [255, 128, 64]], dtype=torch.int32)
    dst, le = ep.plan(ids, 8, 256)
    assert dst.tolist() == [[0, 0, 1], [7, 4, 2]] and le.tolist() == [[0, 31, 0], [31, 0, 0]]


def test_emulated_ep_layer_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29611, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, msg in sorted(res):
        assert ok, f"rank {rank}: {msg}"
