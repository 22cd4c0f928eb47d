"""Generate the golden fixtures in this directory by running kb-nano's own Python reference.

Run once in a container that has the kb-nano tree (first argument, or $KB_NANO_REF); the .npz
files it writes are committed and are what the tests read, so the tests never need the reference
tree.

    python tests/golden/make_golden.py [/path/to/kb_nano]

Every array is produced by reference code, imported from the tree as it lies:
  quant_1x128.npz     tasks/reference/L1/fp8_linear.py  PerTokenGroupQuantFp8 / _quantize_fp8_per_token_group
  silu_table.npz      tasks/reference/L1/silu_and_mul.py SiluAndMul on every bf16 gate bit pattern (up = 1)
  silu_mul_quant.npz  SiluAndMul (bf16) followed by _quantize_fp8_per_token_group
  block_quant.npz     bench/kernels/scenario_registry.py _quantize_fp8_per_block / _quantize_fp8_per_token_group
  fp8_linear.npz      tasks/reference/L1/fp8_linear.py Fp8Linear.forward on dequant(quant(A))
  grouped_gemm.npz    tasks/reference/L1/moe_grouped_gemm.py MoeGroupedGemm.forward (FP8 block-scaled)
  permute.npz         tasks/reference/L2/fused_experts.py _deepgemm_permute / _deepgemm_unpermute_and_reduce
  fused_experts.npz   the op sequence of tasks/reference/L2/fused_experts.py FusedExperts._forward_triton, run
                      with that file's own MoeAlign / MoeGroupedGemm / SiluAndMul / PerTokenGroupQuantFp8 / MoeSum
  routing.npz         tasks/reference/L1/topk_softmax.py TopKSoftmax.forward (renormalised and raw weights)
  grouped_topk.npz    tasks/baseline/L1/grouped_topk.py GroupedTopK.forward, eager branch (:117-174; kb-nano has no
                      reference/ edition of this operator).  The file imports a compiled extension at module level
                      that only its CUDA fast path uses: the import is satisfied with an empty stand-in and, with no
                      CUDA device, forward() takes the eager branch.  VLLM_BATCH_INVARIANT=1 makes its top-k sorted.
                      `--only-grouped-topk` writes this fixture alone.
Inputs are seeded; bf16 tensors are stored as uint16 bit patterns, fp8 as uint8.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ONLY_GROUPED_TOPK = "--only-grouped-topk" in sys.argv
_args = [a for a in sys.argv[1:] if not a.startswith("--")]
if not _args and "KB_NANO_REF" not in os.environ:
    sys.exit("usage: make_golden.py [--only-grouped-topk] /path/to/kb_nano   (or set KB_NANO_REF)")
REF = os.path.abspath(_args[0] if _args else os.environ["KB_NANO_REF"])


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def make_grouped_topk():
    import types
    os.environ["VLLM_BATCH_INVARIANT"] = "1"
    pkg = types.ModuleType("_ref_l1")
    pkg.__path__ = [os.path.join(REF, "tasks", "baseline", "L1")]
    sys.modules["_ref_l1"] = pkg
    csrc = types.ModuleType("_ref_l1.csrc")
    csrc._C = None                                 # the compiled extension: used by the CUDA fast path only
    sys.modules["_ref_l1.csrc"] = csrc
    spec = importlib.util.spec_from_file_location("_ref_l1.grouped_topk", os.path.join(REF, "tasks/baseline/L1/grouped_topk.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    assert not torch.cuda.is_available(), "the eager branch is what is recorded: run without a CUDA device"
    gen = torch.Generator().manual_seed(20250)
    out = {}
    # DeepSeek-V3-like: 256 experts in 8 groups, 4 groups kept, top-8, sigmoid, selection bias, x 2.5
    lg = torch.randn(48, 256, generator=gen)
    bias = torch.randn(256, generator=gen) * 0.1
    w, ids = mod.GroupedTopK("sigmoid", True, 2.5)(lg, bias, 8, 4, 8)
    out.update(a_logits=bits(lg), a_bias=bits(bias), a_w=bits(w), a_ids=bits(ids))
    # no bias (group score = max), softmax, no renormalisation
    lg = torch.randn(32, 64, generator=gen)
    w, ids = mod.GroupedTopK("softmax", False, 1.0)(lg, None, 4, 2, 6)
    out.update(b_logits=bits(lg), b_w=bits(w), b_ids=bits(ids))
    # bf16 logits: the scores are computed in bf16 (ids can tie there; the fixture keeps the weights' multiset per token)
    lg = torch.randn(40, 128, generator=gen).to(torch.bfloat16)
    bias = torch.randn(128, generator=gen) * 0.05
    w, ids = mod.GroupedTopK("sigmoid", True, 1.0)(lg, bias, 4, 2, 8)
    out.update(c_logits=bits(lg), c_bias=bits(bias), c_w=bits(w), c_ids=bits(ids))
    np.savez_compressed(os.path.join(HERE, "grouped_topk.npz"), **out)


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def edge_activations(gen: torch.Generator, m: int, k: int) -> torch.Tensor:
    """bf16 [m,k] ~N(0,1) with rows that hit the scale formula's corner cases."""
    x = torch.randn(m, k, generator=gen)
    x[0] = 0.0                                   # all-zero groups -> eps clamp
    x[1, :128] = torch.linspace(-3.5, 3.5, 128)  # absmax/448 exactly a power of two
    x[2, :128] = 7.0 * torch.sign(x[2, :128])
    x[3, :128] *= 1e-3
    x[3, 7] = 14.0 * 2.0 ** -10
    x[4, 5] = 448.0
    x[5, 9] = -448.0 * 64
    x[6] *= 1e-12                                # below eps
    x[7] *= 1e-9                                 # around eps
    x[8, ::3] *= 50.0                            # outliers
    x[9, :128] = 3.515625                        # mantissa just above 1.75
    x[10, :128] = 3.484375                       # mantissa just below 1.75
    x[11] *= 3.0e4
    return x.to(torch.bfloat16)


def main() -> None:
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    ref_lin = _load("tasks/reference/L1/fp8_linear.py", "_ref_fp8_linear")
    ref_act = _load("tasks/reference/L1/silu_and_mul.py", "_ref_silu_and_mul")
    ref_gg = _load("tasks/reference/L1/moe_grouped_gemm.py", "_ref_moe_grouped_gemm")
    ref_fe = _load("tasks/reference/L2/fused_experts.py", "_ref_fused_experts")
    pkg_dir = tempfile.mkdtemp()
    os.symlink(REF, os.path.join(pkg_dir, "kb_nano"))
    sys.path.insert(0, pkg_dir)
    ref_reg = importlib.import_module("kb_nano.bench.kernels.scenario_registry")

    gen = torch.Generator().manual_seed(20240607)

    # ---- a1: per-token-group quant ------------------------------------------------------
    x = edge_activations(gen, 48, 640)
    q = torch.empty(48, 640, dtype=torch.float8_e4m3fn)
    s = torch.empty(48, 5, dtype=torch.float32)
    ref_lin.PerTokenGroupQuantFp8()(x, q, s)
    x_r = torch.randn(16, 200, generator=gen).to(torch.bfloat16)    # ragged K (not a multiple of 128)
    q_r = torch.empty(16, 200, dtype=torch.float8_e4m3fn)
    s_r = torch.empty(16, 2, dtype=torch.float32)
    ref_lin._quantize_fp8_per_token_group(x_r, q_r, s_r)
    np.savez_compressed(os.path.join(HERE, "quant_1x128.npz"), x=bits(x), q=bits(q), s=bits(s),
                        x_ragged=bits(x_r), q_ragged=bits(q_r), s_ragged=bits(s_r))

    # ---- silu(gate)->bf16 for every gate bit pattern -----------------------------------
    g_all = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    tab = ref_act.SiluAndMul()(torch.stack([g_all, torch.ones_like(g_all)], dim=1)).reshape(-1)
    np.savez_compressed(os.path.join(HERE, "silu_table.npz"), table=bits(tab))

    # ---- a2: silu*up (bf16) then quant -------------------------------------------------
    xin = torch.randn(128, 2 * 384, generator=gen)
    mask = torch.rand(128, 2 * 384, generator=gen) < 1e-3
    xin = torch.where(mask, xin * 50.0, xin)
    xin[0] = 0.0
    xin[1, :384] = 30.0
    xin[2, :384] = -30.0
    xin[3, :384] = -100.0
    xin = xin.to(torch.bfloat16)
    y = ref_act.SiluAndMul()(xin)
    q2 = torch.empty(128, 384, dtype=torch.float8_e4m3fn)
    s2 = torch.empty(128, 3, dtype=torch.float32)
    ref_lin._quantize_fp8_per_token_group(y, q2, s2)
    np.savez_compressed(os.path.join(HERE, "silu_mul_quant.npz"), x=bits(xin), y=bits(y), q=bits(q2), s=bits(s2))

    # ---- weight 128x128 block quant (the harness's coherent-input generator) ------------
    w = (0.02 * torch.randn(3, 256, 384, generator=gen)).to(torch.bfloat16)
    wq, ws = ref_reg._quantize_fp8_per_block(w, torch.float8_e4m3fn)
    w_r = (0.02 * torch.randn(200, 300, generator=gen)).to(torch.bfloat16)
    wq_r, ws_r = ref_reg._quantize_fp8_per_block(w_r, torch.float8_e4m3fn)
    aq_h, as_h = ref_reg._quantize_fp8_per_token_group(x, torch.float8_e4m3fn)
    np.savez_compressed(os.path.join(HERE, "block_quant.npz"), w=bits(w), q=bits(wq), s=bits(ws),
                        w_ragged=bits(w_r), q_ragged=bits(wq_r), s_ragged=bits(ws_r),
                        act_q=bits(aq_h), act_s=bits(as_h))

    # ---- a3: dense linear = Fp8Linear.forward on the dequantised quantised A ------------
    a = torch.randn(40, 384, generator=gen).to(torch.bfloat16)
    wl = (0.02 * torch.randn(256, 384, generator=gen)).to(torch.bfloat16)
    wlq, wls = ref_reg._quantize_fp8_per_block(wl, torch.float8_e4m3fn)
    aq = torch.empty(40, 384, dtype=torch.float8_e4m3fn)
    asc = torch.empty(40, 3, dtype=torch.float32)
    ref_lin._quantize_fp8_per_token_group(a, aq, asc)
    a_deq = aq.float() * asc.repeat_interleave(128, dim=-1)
    # Fp8Linear.forward does F.linear(x.float(), dequant(W)) and casts to x.dtype; feeding it the
    # fp32 dequantised A gives fp32 out, rounded to bf16 here exactly as the layer would.
    c = ref_lin.Fp8Linear()(a_deq, wlq, wls).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "fp8_linear.npz"), a=bits(a), a_q=bits(aq), a_s=bits(asc),
                        w_q=bits(wlq), w_s=bits(wls), c=bits(c))

    # ---- a4/a6: grouped GEMM via the reference MoeGroupedGemm (sorted-token layout) -----
    E, T, H, I, TOPK, BM = 4, 24, 256, 128, 2, 16
    hs = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    w13 = (0.05 * torch.randn(E, 2 * I, H, generator=gen)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(E, H, I, generator=gen)).to(torch.bfloat16)
    w13q, w13s = ref_reg._quantize_fp8_per_block(w13, torch.float8_e4m3fn)
    w2q, w2s = ref_reg._quantize_fp8_per_block(w2, torch.float8_e4m3fn)
    logits = torch.randn(T, E, generator=gen)
    tw, ti = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
    tw = (tw / tw.sum(-1, keepdim=True)).float()
    ti = ti.to(torch.int32)
    hq = torch.empty(T, H, dtype=torch.float8_e4m3fn)
    hsc = torch.empty(T, H // 128, dtype=torch.float32)
    ref_lin._quantize_fp8_per_token_group(hs, hq, hsc)
    sorted_ids, blk_experts, ntpp = ref_fe.MoeAlign()(ti, BM, E)
    c1 = torch.zeros(T * TOPK, 2 * I, dtype=torch.bfloat16)
    # The torch MoeGroupedGemm expands a [T, K/128] activation scale as if it were a 128x128 block
    # scale when block_shape is given (tasks/reference/L1/moe_grouped_gemm.py:60-63: row r reads
    # a_scale[r // 128]), unlike the Triton kernel it stands for, which reads one scale per token and
    # K-group (tasks/baseline/L1/moe_grouped_gemm.py:159-167).  Handing it the scale already expanded
    # to A's shape takes its `scale.shape == x.shape` branch (:49-50) and gives per-token-group
    # dequantisation with the reference's own code.
    ref_gg.MoeGroupedGemm()(hq, w13q, c1, tw, sorted_ids, blk_experts, ntpp, False, TOPK,
                            config={"BLOCK_SIZE_M": BM}, a_scale=hsc.repeat_interleave(128, dim=1), b_scale=w13s,
                            use_fp8_w8a8=True, block_shape=[128, 128])
    np.savez_compressed(os.path.join(HERE, "grouped_gemm.npz"), a_q=bits(hq), a_s=bits(hsc), b_q=bits(w13q),
                        b_s=bits(w13s), topk_ids=bits(ti), topk_w=bits(tw), c=bits(c1),
                        sorted_ids=bits(sorted_ids), blk_experts=bits(blk_experts))

    # ---- permute / unpermute helpers of the DeepGEMM-layout path ------------------------
    a_perm, as_perm, row_expert, inv_perm = ref_fe._deepgemm_permute(hq, hsc, ti, E, 128)
    mm2 = torch.randn(a_perm.shape[0], H, generator=gen).to(torch.bfloat16)
    comb = torch.empty(T, H, dtype=torch.bfloat16)
    ref_fe._deepgemm_unpermute_and_reduce(mm2, ti, tw, inv_perm, comb)
    np.savez_compressed(os.path.join(HERE, "permute.npz"), a_q=bits(hq), a_s=bits(hsc), topk_ids=bits(ti),
                        topk_w=bits(tw), a_perm=bits(a_perm), as_perm=bits(as_perm), row_expert=bits(row_expert),
                        inv_perm=bits(inv_perm), mm2=bits(mm2), combined=bits(comb))

    # ---- a7: whole FP8 expert pipeline ---------------------------------------------------
    # The sequence of FusedExperts._forward_triton (tasks/reference/L2/fused_experts.py:810-872) run
    # with the reference's own modules, activation scales passed expanded for the reason given above
    # (FusedExperts.forward itself would hit the row//128 expansion in both GEMMs).
    gg = ref_fe.MoeGroupedGemm()
    inter1 = torch.zeros(T * TOPK, 2 * I, dtype=torch.bfloat16)
    gg(hq, w13q, inter1, tw, sorted_ids, blk_experts, ntpp, False, TOPK, config={"BLOCK_SIZE_M": BM},
       a_scale=hsc.repeat_interleave(128, dim=1), b_scale=w13s, use_fp8_w8a8=True, block_shape=[128, 128])
    inter2 = ref_fe.SiluAndMul()(inter1)
    a2q = torch.empty(T * TOPK, I, dtype=torch.float8_e4m3fn)
    a2s = torch.empty(T * TOPK, I // 128, dtype=torch.float32)
    ref_fe.PerTokenGroupQuantFp8()(inter2, a2q, a2s)
    inter3 = torch.zeros(T * TOPK, H, dtype=torch.bfloat16)
    gg(a2q, w2q, inter3, tw, sorted_ids, blk_experts, ntpp, True, 1, config={"BLOCK_SIZE_M": BM},
       a_scale=a2s.repeat_interleave(128, dim=1), b_scale=w2s, use_fp8_w8a8=True, block_shape=[128, 128])
    out = ref_fe.MoeSum()(inter3, TOPK)
    np.savez_compressed(os.path.join(HERE, "fused_experts.npz"), x=bits(hs), w13_q=bits(w13q), w13_s=bits(w13s),
                        w2_q=bits(w2q), w2_s=bits(w2s), topk_w=bits(tw), topk_ids=bits(ti), inter1=bits(inter1),
                        a2_q=bits(a2q), a2_s=bits(a2s), out=bits(out))
    # routing: the reference TopKSoftmax on fp32 logits (Mixtral-like 8 experts / top-2 and 256 experts / top-8)
    ref_tk = _load("tasks/reference/L1/topk_softmax.py", "_ref_topk_softmax")
    router = ref_tk.TopKSoftmax()
    lg8 = torch.randn(64, 8, generator=gen)
    lg256 = torch.randn(48, 256, generator=gen)
    w8, i8 = router(lg8, 2, True)
    w8, i8 = w8.clone(), i8.clone()
    router = ref_tk.TopKSoftmax()             # its output buffers keep the first call's top_k: one instance per top_k
    w256, i256 = router(lg256, 8, True)
    w256, i256 = w256.clone(), i256.clone()
    w256n, i256n = router(lg256, 8, False)
    np.savez_compressed(os.path.join(HERE, "routing.npz"), logits8=bits(lg8), w8=bits(w8), ids8=bits(i8), logits256=bits(lg256),
                        w256=bits(w256), ids256=bits(i256), w256_raw=bits(w256n.clone()), ids256_raw=bits(i256n.clone()))
    make_grouped_topk()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if ONLY_GROUPED_TOPK:
        make_grouped_topk()
        print("grouped_topk.npz", os.path.getsize(os.path.join(HERE, "grouped_topk.npz")))
    else:
        main()
