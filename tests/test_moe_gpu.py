"""GPU parity of the MoE permutation kernels (bit-exact against kb-nano's own permute, from the
golden fixture) and of the whole FP8 expert pipeline (tolerance rule of the GEMMs)."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close, bf16_from_bits, fp8_from_bits, golden

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def run_permute(a_q, a_s, ids, e, dev):
    from kb_nano_b200 import ops
    t, k = a_q.shape
    topk = ids.shape[1]
    m_cap = ops.moe_aligned_rows(t, topk, e)
    a_perm = torch.zeros(m_cap, k, dtype=torch.uint8, device=dev).view(FP8)
    s_perm = torch.zeros(m_cap, k // 128, device=dev)
    row_expert = torch.full((m_cap,), -7, dtype=torch.int32, device=dev)
    dest = torch.full((t, topk), -7, dtype=torch.int32, device=dev)
    ws = torch.empty(ops.moe_permute_workspace_bytes(t, topk, e), dtype=torch.uint8, device=dev)
    ops.moe_permute(a_q.to(dev), a_s.to(dev), ids.to(dev), e, a_perm, s_perm, row_expert, dest, ws)
    return a_perm.cpu(), s_perm.cpu(), row_expert.cpu(), dest.cpu()


def test_permute_matches_reference_layout(cuda_dev):
    g = golden("permute")
    e = 4
    a_perm, s_perm, row_expert, dest = run_permute(fp8_from_bits(g["a_q"]), torch.from_numpy(g["a_s"]),
                                                   torch.from_numpy(g["topk_ids"]), e, cuda_dev)
    assert a_perm.shape[0] == g["a_perm"].shape[0]
    assert (row_expert.numpy() == g["row_expert"]).all()
    assert (dest.numpy() == g["inv_perm"]).all()
    valid = g["row_expert"] >= 0
    assert (a_perm.view(torch.uint8).numpy()[valid] == g["a_perm"][valid]).all()
    assert (s_perm.numpy()[valid] == g["as_perm"][valid]).all()


@pytest.mark.parametrize("t,topk,e,k", [(37, 3, 5, 256), (700, 8, 64, 512), (1, 2, 4, 128)])
def test_permute_emits_packed_scales(cuda_dev, t, topk, e, k):
    """The packed UE8M0 copy of the scales written by the permute equals packing the permuted fp32 scales
    afterwards; the id tensor starts 12 bytes into an allocation in the first case (unaligned ranking path)."""
    from kb_nano_b200 import ops
    gen = torch.Generator().manual_seed(t + k)
    a_q = torch.randint(0, 255, (t, k), dtype=torch.uint8, generator=gen).view(FP8).to(cuda_dev)
    a_s = torch.exp2(torch.randint(-20, 10, (t, k // 128), generator=gen).float()).to(cuda_dev)
    ids_all = torch.randint(0, e, (t + 1, topk), dtype=torch.int32, generator=gen).to(cuda_dev)
    ids = ids_all[1:]
    m_cap = ops.moe_aligned_rows(t, topk, e)
    outs = []
    for fused in (False, True):
        a_perm = torch.zeros(m_cap, k, dtype=torch.uint8, device=cuda_dev).view(FP8)
        s_perm = torch.zeros(m_cap, k // 128, device=cuda_dev)
        row_expert = torch.empty(m_cap, dtype=torch.int32, device=cuda_dev)
        dest = torch.empty(t, topk, dtype=torch.int32, device=cuda_dev)
        ws = torch.empty(ops.moe_permute_workspace_bytes(t, topk, e), dtype=torch.uint8, device=cuda_dev)
        sf = torch.zeros(ops.packed_sf_rows_bytes(m_cap, k), dtype=torch.uint8, device=cuda_dev)
        ops.moe_permute(a_q, a_s, ids, e, a_perm, s_perm, row_expert, dest, ws, sf if fused else None)
        outs.append((a_perm.view(torch.uint8).cpu(), s_perm.cpu(), row_expert.cpu(), dest.cpu(), sf.cpu(), ops.pack_sf_rows(s_perm, k).cpu()))
    for x, y in zip(outs[0][:4], outs[1][:4]):
        assert torch.equal(x, y)
    assert not outs[0][4].any()                        # not requested: untouched
    assert torch.equal(outs[1][4], outs[1][5])         # padding rows: scale 0.0 packs to exponent byte 0 = the pre-zeroed buffer
    assert outs[1][4].any()


def test_combine_matches_reference(cuda_dev):
    from kb_nano_b200 import ops
    g = golden("permute")
    mm2 = bf16_from_bits(g["mm2"]).to(cuda_dev)
    out = torch.empty(g["combined"].shape, dtype=torch.bfloat16, device=cuda_dev)
    ops.moe_unpermute_combine(mm2, torch.from_numpy(g["inv_perm"]).to(cuda_dev), torch.from_numpy(g["topk_w"]).to(cuda_dev), out)
    ref = bf16_from_bits(g["combined"])
    # same products; the reference rounds the fp32 sum once as well, only the summation order may differ
    assert float((out.cpu().float() - ref.float()).abs().max()) <= 2.0 ** -7 * float(ref.float().abs().max())
    assert_gemm_close(out.cpu(), ref, "combine")


@pytest.mark.parametrize("t,topk,e", [(1, 1, 1), (7, 2, 3), (300, 8, 64), (128, 8, 256), (64, 4, 5), (1000, 3, 17), (2048, 8, 256)])
def test_permute_properties(cuda_dev, t, topk, e):
    """Stable grouping with 128-aligned segments, for shapes with empty experts and every token on one expert."""
    gen = torch.Generator().manual_seed(t * 31 + e)
    k = 256
    a_q = torch.randint(0, 255, (t, k), dtype=torch.uint8, generator=gen).view(FP8)
    a_s = torch.rand(t, k // 128, generator=gen)
    if e == 5:
        ids = torch.full((t, topk), 3, dtype=torch.int32)          # everything to one expert
    else:
        ids = torch.stack([torch.randperm(e, generator=gen)[:topk] for _ in range(t)]).to(torch.int32) if topk <= e else torch.zeros(t, topk, dtype=torch.int32)
    a_perm, s_perm, row_expert, dest = run_permute(a_q, a_s, ids, e, cuda_dev)
    flat = ids.reshape(-1)
    counts = torch.bincount(flat.long(), minlength=e)
    off = torch.zeros(e + 1, dtype=torch.long)
    off[1:] = torch.cumsum((counts + 127) // 128 * 128, 0)
    exp_rows = torch.full_like(row_expert, -1)
    for x in range(e):
        exp_rows[off[x]:off[x] + counts[x]] = x
    assert (row_expert == exp_rows).all()
    seen = {}
    for i in range(flat.numel()):
        x = int(flat[i])
        r = seen.get(x, 0)
        seen[x] = r + 1
        assert int(dest.reshape(-1)[i]) == int(off[x]) + r
    d = dest.reshape(-1).long()
    assert (a_perm.view(torch.uint8)[d] == a_q.view(torch.uint8).repeat_interleave(topk, 0)).all()
    assert (s_perm[d] == a_s.repeat_interleave(topk, 0)).all()


def moe_case(t, h, i, e, topk, seed, routing):
    from kb_nano_b200 import inputs
    x = inputs.activations(t, h, seed=seed)
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=seed + 1, std=0.05)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=seed + 2, std=0.05)
    logits = inputs.router_logits(t, e, seed=seed)
    tw, ti = (inputs.route_sigmoid_topk if routing == "sigmoid" else inputs.route_softmax_topk)(logits, topk)
    return x, w13_q, w13_s, w2_q, w2_s, tw, ti


@pytest.mark.parametrize("t,h,i,e,topk,routing", [(64, 512, 256, 8, 2, "softmax"), (200, 1024, 256, 32, 8, "sigmoid"), (1, 256, 128, 4, 2, "softmax")])
def test_moe_layer_vs_oracle(cuda_dev, t, h, i, e, topk, routing):
    from kb_nano_b200 import moe
    x, w13_q, w13_s, w2_q, w2_s, tw, ti = moe_case(t, h, i, e, topk, seed=t + e, routing=routing)
    ref = to.moe_layer(x, w13_q, w13_s, w2_q, w2_s, tw, ti)
    d = cuda_dev
    for fast in (True, False):      # UE8M0 block-scaled GEMMs, then the fp32-scale kernels
        out = moe.fused_experts_fp8(x.to(d), w13_q.to(d), w2_q.to(d), tw.to(d), ti.to(d), e, w13_s.to(d), w2_s.to(d), use_ue8m0=fast)
        assert_gemm_close(out.cpu(), ref, f"moe layer t={t} e={e} ue8m0={fast}")
    # bf16 router weights (as MixtralMoE casts them) and int64 ids go through the same path
    out2 = moe.fused_experts_fp8(x.to(d), w13_q.to(d), w2_q.to(d), tw.to(torch.bfloat16).to(d), ti.long().to(d), e, w13_s.to(d), w2_s.to(d))
    ref2 = to.moe_layer(x, w13_q, w13_s, w2_q, w2_s, tw.to(torch.bfloat16), ti)
    assert_gemm_close(out2.cpu(), ref2, "moe layer, bf16 weights")


def test_moe_layer_fused_activation_matches_unfused(cuda_dev):
    """The layer with the activation inside GEMM1's epilogue returns the bits of the layer with the
    stand-alone activation kernel."""
    from kb_nano_b200 import inputs, moe
    t, h, i, e, topk, d = 300, 1024, 512, 16, 4, cuda_dev
    x = inputs.activations(t, h, seed=5, device=d)
    tw, ti = inputs.route_sigmoid_topk(inputs.router_logits(t, e, seed=5, device=d), topk)
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=6, device=d)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=7, device=d)
    a = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s, fuse_activation=True).clone()
    b = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s, fuse_activation=False).clone()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert bool(a.float().abs().sum() > 0)


@pytest.mark.parametrize("t,topk,e,bm", [(37, 4, 8, 16), (256, 8, 64, 64), (1, 2, 4, 16), (300, 1, 3, 128)])
def test_pair_experts_from_sorted_lists(cuda_dev, t, topk, e, bm):
    """kbn_moe_pair_experts against the layout kb-nano's moe_align_block_size produces (pairs sorted by expert, every
    expert's run padded to a multiple of the block size with the value n_pairs; tasks/baseline/L1/moe_grouped_gemm.py
    :111-127 reads it that way): every pair gets the expert of the block its position lies in; a pair left out of
    the list gets -1; without a list block i is pair i."""
    from kb_nano_b200 import ops
    gen = torch.Generator().manual_seed(t * 131 + e)
    ids = torch.stack([torch.randperm(e, generator=gen)[:topk] if topk <= e else torch.randint(0, e, (topk,), generator=gen) for _ in range(t)])
    n_pairs = t * topk
    flat = ids.reshape(-1)
    dropped = int(torch.randint(0, n_pairs, (1,), generator=gen)) if n_pairs > 4 else -1
    sorted_ids, blocks = [], []
    for ex in range(e):
        mine = [p for p in torch.nonzero(flat == ex).flatten().tolist() if p != dropped]
        pad = (-len(mine)) % bm
        sorted_ids += mine + [n_pairs] * pad
        blocks += [ex] * ((len(mine) + pad) // bm)
    want = flat.clone().to(torch.int32)
    if dropped >= 0:
        want[dropped] = -1
    out = torch.full((n_pairs,), 77, dtype=torch.int32, device=cuda_dev)
    ops.moe_pair_experts(torch.tensor(sorted_ids, dtype=torch.int32, device=cuda_dev), torch.tensor(blocks, dtype=torch.int32, device=cuda_dev), bm, out)
    assert torch.equal(out.cpu(), want)
    out2 = torch.full((n_pairs,), 77, dtype=torch.int32, device=cuda_dev)
    ops.moe_pair_experts(None, flat.to(torch.int32).to(cuda_dev), bm, out2)
    assert torch.equal(out2.cpu(), flat.to(torch.int32))


def test_moe_grouped_gemm_candidate_golden(cuda_dev):
    """The MoeGroupedGemm drop-in (sorted-token layout of kb-nano's Triton path) on the fixture produced by
    the reference's MoeGroupedGemm, with and without the routed-weight multiply, and in the one-row-per-block
    form (sorted_token_ids=None)."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_moe_grouped_gemm", os.path.join(candidate_dir(), "L1", "moe_grouped_gemm.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    g = golden("grouped_gemm")
    d = cuda_dev
    a_q, a_s = fp8_from_bits(g["a_q"]).to(d), torch.from_numpy(g["a_s"]).to(d)
    b_q, b_s = fp8_from_bits(g["b_q"]).to(d), torch.from_numpy(g["b_s"]).to(d)
    tw = torch.from_numpy(g["topk_w"]).to(d)
    sorted_ids, blk = torch.from_numpy(g["sorted_ids"]).to(d), torch.from_numpy(g["blk_experts"]).to(d)
    t, topk = g["topk_ids"].shape
    ntpp = torch.tensor([sorted_ids.numel()], dtype=torch.int32, device=d)
    ref = bf16_from_bits(g["c"])
    gg = mod.MoeGroupedGemm()
    c = torch.full((t * topk, b_q.shape[1]), 3.0, dtype=torch.bfloat16, device=d)
    a0 = a_q.clone()
    gg(a_q, b_q, c, tw, sorted_ids, blk, ntpp, False, topk, config={"BLOCK_SIZE_M": 16}, a_scale=a_s, b_scale=b_s,
       use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(c.cpu(), ref, "MoeGroupedGemm golden")
    assert bool((a_q.view(torch.uint8) == a0.view(torch.uint8)).all())
    c2 = torch.zeros_like(c)
    gg(a_q, b_q, c2, tw, sorted_ids, blk, ntpp, True, topk, config={"BLOCK_SIZE_M": 16}, a_scale=a_s, b_scale=b_s,
       use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(c2.cpu(), (ref.float() * torch.from_numpy(g["topk_w"]).reshape(-1, 1)).to(torch.bfloat16), "MoeGroupedGemm x routed weight")
    # naive block assignment: block i = row i, expert_ids has one entry per row
    c3 = torch.zeros_like(c)
    gg(a_q, b_q, c3, tw, None, torch.from_numpy(g["topk_ids"]).reshape(-1).to(d), ntpp, False, topk, config={"BLOCK_SIZE_M": 16},
       a_scale=a_s, b_scale=b_s, use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(c3.cpu(), ref, "MoeGroupedGemm naive")
    # weight scales that are not powers of two take the fp32-scale kernels
    b_s2 = b_s * 1.3
    c4 = torch.zeros_like(c)
    gg(a_q, b_q, c4, tw, sorted_ids, blk, ntpp, False, topk, config={"BLOCK_SIZE_M": 16}, a_scale=a_s, b_scale=b_s2,
       use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(c4.cpu(), (ref.float() * 1.3).to(torch.bfloat16), "MoeGroupedGemm, arbitrary weight scales")
    with pytest.raises(NotImplementedError):
        gg(a_q.float(), b_q, c, tw, sorted_ids, blk, ntpp, False, topk)


def test_fused_experts_candidate_golden(cuda_dev):
    """The FusedExperts drop-in class on the reference-generated fixture."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir
    spec = importlib.util.spec_from_file_location("_candidate_impl_L2_fused_experts", os.path.join(candidate_dir(), "L2", "fused_experts.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    g = golden("fused_experts")
    d = cuda_dev
    x = bf16_from_bits(g["x"]).to(d)
    x0 = x.clone()
    out = mod.FusedExperts()(x, fp8_from_bits(g["w13_q"]).to(d), fp8_from_bits(g["w2_q"]).to(d), torch.from_numpy(g["topk_w"]).to(d),
                             torch.from_numpy(g["topk_ids"]).to(d), 4, w13_scale=torch.from_numpy(g["w13_s"]).to(d),
                             w2_scale=torch.from_numpy(g["w2_s"]).to(d), use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(out.cpu(), bf16_from_bits(g["out"]), "FusedExperts golden")
    assert bool((x == x0).all())
    with pytest.raises(NotImplementedError):
        mod.FusedExperts()(x, x, x, x, x, 4)


def test_vllm_fused_experts_candidate_golden(cuda_dev):
    """The VllmFusedExperts drop-in class (DeepSeek's expert path) on the reference-generated fixture, whose
    operation order (routed weight applied at GEMM2, sum over the slots) is that class's."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir
    spec = importlib.util.spec_from_file_location("_candidate_impl_L2_vllm_fused_experts", os.path.join(candidate_dir(), "L2", "vllm_fused_experts.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    g = golden("fused_experts")
    d = cuda_dev
    x = bf16_from_bits(g["x"]).to(d)
    x0 = x.clone()
    args = (fp8_from_bits(g["w13_q"]).to(d), fp8_from_bits(g["w2_q"]).to(d), torch.from_numpy(g["topk_w"]).to(d),
            torch.from_numpy(g["topk_ids"]).to(d), 4, torch.from_numpy(g["w13_s"]).to(d), torch.from_numpy(g["w2_s"]).to(d))
    out = mod.VllmFusedExperts()(x, *args, [128, 128])
    assert_gemm_close(out.cpu(), bf16_from_bits(g["out"]), "VllmFusedExperts golden")
    assert bool((x == x0).all())
    with pytest.raises(NotImplementedError):
        mod.VllmFusedExperts()(x, *args, [64, 64])
