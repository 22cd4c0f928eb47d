"""CPU oracle, torch edition.  TEST INFRASTRUCTURE ONLY.

A restatement, in plain torch CPU ops, of the torch path kb-nano's reference uses to
define the FP8 W8A8 hot path.  Only tests/, the smoke check and bench.py's CPU-baseline
legs may import this module; the product package never does.

Reference lines each function follows (paths relative to the kb-nano tree):
  quant_1x128           tasks/reference/L1/fp8_linear.py:41-64
  silu_mul_bf16         tasks/baseline/L1/silu_mul_quant_fp8.py:54-60
                        (== tasks/reference/L1/silu_and_mul.py:18-21 on bf16 input)
  silu_mul_quant_1x128  tasks/baseline/L1/silu_mul_quant_fp8.py:54-76
  block_quant_128x128   bench/kernels/scenario_registry.py:185-221
  dequant_rows/_blocks  tasks/reference/L1/fp8_linear.py:26-38
  gemm_nt_dequant       tasks/reference/L1/fp8_linear.py:100-104 applied to quantised A
  grouped_gemm_contig   tasks/reference/L1/moe_grouped_gemm.py:39-91 (per-expert matmul)
  grouped_gemm_masked   same arithmetic in the [E, max_m, K] layout (no reference call site)
  route_sigmoid_topk    tasks/baseline/L1/grouped_topk.py:119-174 with n_group=1, no bias
  route_softmax_topk    tasks/reference/L1/topk_softmax.py:46-52
  requant_weights_ue8m0 tasks/baseline/L1/fp8_linear.py:453-512 with DeepGEMM's published per_block_cast_to_fp8
                        (v2.1.1.post3: block max clamped at 1e-4, scale = 2^ceil(log2(max/448)), x * (1/scale))
  rmsnorm_quant         tasks/baseline/L1/csrc/rmsnorm_quant.cu:22-97,125-204 (fp32 arithmetic of the CUDA
                        kernel; there is no torch reference of the fused op in the tree)
  moe_layer             tasks/baseline/L2/fused_experts.py:246-283,119-136
                        (quant -> GEMM1 -> silu*up+quant -> GEMM2 -> weighted sum over top-k
                        in the activation dtype)
"""
from __future__ import annotations

import torch

GROUP = 128
FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def _scale_from_absmax(absmax: torch.Tensor, eps: float, ue8m0: bool) -> torch.Tensor:
    s = absmax.clamp_min(eps) / FP8_MAX
    if ue8m0:
        s = torch.pow(2.0, torch.ceil(torch.log2(s)))
    return s


def quant_1x128(x: torch.Tensor, eps: float = 1e-10, ue8m0: bool = True):
    """x [M,K] (bf16/fp32) -> (q e4m3 [M,K], scale fp32 [M, ceil(K/128)])."""
    m, k = x.shape
    g = (k + GROUP - 1) // GROUP
    xf = x.float()
    if g * GROUP != k:
        pad = xf.new_zeros(m, g * GROUP)
        pad[:, :k] = xf
    else:
        pad = xf
    s = _scale_from_absmax(pad.view(m, g, GROUP).abs().amax(dim=-1), eps, ue8m0)
    full = s.repeat_interleave(GROUP, dim=-1)[:, :k]
    q = torch.clamp(xf / full, -FP8_MAX, FP8_MAX).to(FP8)
    return q, s


def silu_mul_bf16(x: torch.Tensor) -> torch.Tensor:
    """x [M, 2*N2] bf16 -> bf16 [M, N2]: silu in fp32, rounded to bf16, times up in bf16."""
    n2 = x.shape[-1] // 2
    g = x[..., :n2].float()
    s = (g / (1.0 + torch.exp(-g))).to(x.dtype)
    return s * x[..., n2:]


def silu_mul_quant_1x128(x: torch.Tensor, eps: float = 1e-10, ue8m0: bool = True):
    return quant_1x128(silu_mul_bf16(x), eps, ue8m0)


def block_quant_128x128(w: torch.Tensor, eps: float = 1e-10, ue8m0: bool = True):
    """w [..., R, C] -> (q e4m3 same shape, scale fp32 [..., ceil(R/128), ceil(C/128)])."""
    shp = w.shape
    r, c = shp[-2], shp[-1]
    rb, cb = (r + 127) // 128, (c + 127) // 128
    flat = w.reshape(-1, r, c).float()
    pad = flat.new_zeros(flat.shape[0], rb * 128, cb * 128)
    pad[:, :r, :c] = flat
    s = _scale_from_absmax(pad.view(-1, rb, 128, cb, 128).abs().amax(dim=(2, 4)), eps, ue8m0)
    full = s.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)[:, :r, :c]
    q = torch.clamp(flat / full, -FP8_MAX, FP8_MAX).to(FP8).reshape(shp)
    return q, s.reshape(*shp[:-2], rb, cb)


def dequant_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    k = q.shape[-1]
    return q.float() * s.float().repeat_interleave(GROUP, dim=-1)[..., :k]


def dequant_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    r, c = q.shape[-2], q.shape[-1]
    full = s.float().repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)[..., :r, :c]
    return q.float() * full


def gemm_nt_dequant(a_q, sa, w_q, sw, bias=None) -> torch.Tensor:
    out = torch.nn.functional.linear(dequant_rows(a_q, sa), dequant_blocks(w_q, sw),
                                     bias.float() if bias is not None else None)
    return out.to(torch.bfloat16)


def fp8_linear(x_bf16, w_q, sw, bias=None) -> torch.Tensor:
    k = w_q.shape[-1]
    x2 = x_bf16.reshape(-1, k)
    a_q, sa = quant_1x128(x2)
    out = gemm_nt_dequant(a_q, sa, w_q, sw, bias)
    return out.view(*x_bf16.shape[:-1], w_q.shape[0])


def grouped_gemm_contig(a_q, sa, b_q, sb, row_expert, out=None) -> torch.Tensor:
    """Rows with row_expert < 0 are left untouched (zero if `out` is not given)."""
    m, n = a_q.shape[0], b_q.shape[1]
    if out is None:
        out = torch.zeros(m, n, dtype=torch.bfloat16)
    a_d = dequant_rows(a_q, sa)
    for e in torch.unique(row_expert).tolist():
        if e < 0:
            continue
        rows = (row_expert == e).nonzero().flatten()
        out[rows] = (a_d[rows] @ dequant_blocks(b_q[e], sb[e]).t()).to(torch.bfloat16)
    return out


def grouped_gemm_masked(a_q, sa, b_q, sb, masked_m, out=None) -> torch.Tensor:
    e_l, max_m, _ = a_q.shape
    n = b_q.shape[1]
    if out is None:
        out = torch.zeros(e_l, max_m, n, dtype=torch.bfloat16)
    for e in range(e_l):
        mm = int(masked_m[e])
        if mm == 0:
            continue
        out[e, :mm] = (dequant_rows(a_q[e, :mm], sa[e, :mm]) @ dequant_blocks(b_q[e], sb[e]).t()).to(torch.bfloat16)
    return out


def route_sigmoid_topk(logits: torch.Tensor, k: int):
    scores = torch.sigmoid(logits.float())
    w, ids = torch.topk(scores, k, dim=-1, sorted=True)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def route_softmax_topk(logits: torch.Tensor, k: int):
    probs = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(probs, k, dim=-1, sorted=True)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def moe_layer(x, w13_q, w13_s, w2_q, w2_s, topk_w, topk_ids, experts=None) -> torch.Tensor:
    """FP8 MoE expert pipeline on CPU, per expert.

    `experts` restricts the computation to a subset of expert ids (pairs routed elsewhere
    contribute nothing); used for bounded CPU samples and for the per-rank view of the
    expert-parallel layer.
    """
    t, h = x.shape
    a_q, sa = quant_1x128(x)
    a_d = dequant_rows(a_q, sa)
    acc = torch.zeros(t, topk_ids.shape[1], h, dtype=x.dtype)
    ids = topk_ids.long()
    todo = torch.unique(ids).tolist() if experts is None else list(experts)
    for e in todo:
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h1 = (a_d[tok] @ dequant_blocks(w13_q[e], w13_s[e]).t()).to(torch.bfloat16)
        q2, s2 = silu_mul_quant_1x128(h1)
        h2 = (dequant_rows(q2, s2) @ dequant_blocks(w2_q[e], w2_s[e]).t()).to(torch.bfloat16)
        acc[tok, slot] = h2
    # dtype promotion as in the reference: bf16 rows times the router's weights (fp32 or bf16)
    return (acc * topk_w.unsqueeze(-1)).sum(dim=1).to(x.dtype)


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None):
    """(q, scale[, new_residual, normalised_x]) of the fused (add +) RMSNorm + 1x128 quant."""
    if residual is not None:
        s = residual.float() + x.float()
        row = s.to(torch.bfloat16)
        sum_sq = (s * s).sum(dim=-1, keepdim=True)
    else:
        row = x
        sum_sq = (x.float() * x.float()).sum(dim=-1, keepdim=True)
    rms_inv = torch.rsqrt(sum_sq / x.shape[-1] + eps)
    v = (row.float() * rms_inv) * weight.float()
    q, sc = quant_1x128(v)
    if residual is not None:
        return q, sc, row, v.to(torch.bfloat16)
    return q, sc


def requant_weights_ue8m0(w_q: torch.Tensor, s: torch.Tensor, eps: float = 1e-4):
    """(new e4m3 weights, new power-of-two fp32 scales) of block-scaled weights [..., N, K]."""
    w = dequant_blocks(w_q, s)
    return block_quant_128x128(w, eps=eps, ue8m0=True)


def route_topk(logits: torch.Tensor, topk: int, scoring: str = "softmax", bias: torch.Tensor | None = None, n_group: int = 1,
               topk_group: int = 1, renormalize: bool = True, renorm_floor: float = 0.0, scale: float = 1.0,
               score_in_input_dtype: bool = False):
    """Expert routing.  TopKSoftmax (tasks/reference/L1/topk_softmax.py:46-52): softmax in fp32, top-k, division by
    the clamped sum (renorm_floor = 1e-20).  GroupedTopK's eager path (tasks/baseline/L1/grouped_topk.py:117-174):
    scores in the logits' dtype (score_in_input_dtype), biased scores for the selection, a group's score = sum of its
    top-2 biased scores (max of the scores without a bias), the topk_group best groups kept, top-k among them,
    weights = unbiased scores of the chosen experts, / sum, * scale, returned as fp32.  Returns (weights fp32, ids int32)."""
    x = logits if score_in_input_dtype else logits.float()
    scores = torch.softmax(x, dim=-1) if scoring == "softmax" else x.sigmoid()
    t, e = scores.shape
    choice = scores if bias is None else scores + bias.unsqueeze(0)
    if n_group > 1 and topk_group < n_group:
        grouped = choice.view(t, n_group, e // n_group)
        gscore = grouped.topk(2, dim=-1)[0].sum(dim=-1) if bias is not None else grouped.max(dim=-1).values
        gidx = torch.topk(gscore, k=topk_group, dim=-1)[1]
        gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1)
        mask = gmask.unsqueeze(-1).expand(t, n_group, e // n_group).reshape(t, e)
        choice = choice.masked_fill(~mask.bool(), float("-inf"))
    ids = torch.topk(choice, k=topk, dim=-1)[1]
    w = scores.gather(1, ids)
    if renormalize:
        den = w.sum(dim=-1, keepdim=True)
        w = w / (den.clamp_min(renorm_floor) if renorm_floor > 0 else den)
    if scale != 1.0:
        w = w * scale
    return w.to(torch.float32), ids.to(torch.int32)


def qwen3_moe_forward(x, gate_w, w13_q, w13_s, w2_q, w2_s, top_k, renormalize=True, router_logits=None, cast_weights=False):
    """Qwen3MoE.forward_impl (tasks/baseline/L2/qwen3_moe.py:161-188) on one rank: gate linear in the activations'
    dtype, TopKSoftmax, the FP8 experts; no all-reduce with one rank.  cast_weights=True is MixtralMoE.forward_impl
    (tasks/baseline/L2/mixtral_moe.py:64-83): router weights rounded to the activations' dtype (:72).
    router_logits: logits computed elsewhere (a test passes the GPU's own, so that a near tie in the top-k is not
    decided by the two sides' different bf16 GEMMs, which are not what is under test)."""
    logits = torch.nn.functional.linear(x, gate_w) if router_logits is None else router_logits
    tw, ti = route_topk(logits, top_k, "softmax", renormalize=renormalize, renorm_floor=1e-20)
    if cast_weights:
        tw = tw.to(x.dtype).float()
    return moe_layer(x, w13_q, w13_s, w2_q, w2_s, tw, ti)


def swiglu_mlp_fp8(x, gate_up_q, gate_up_s, down_q, down_s):
    """LlamaMLP with FP8 block-scaled linears (tasks/baseline/L2/llama_mlp.py:17-39 over Fp8Linear,
    tasks/baseline/L1/fp8_linear.py:371-450): quantise, GEMM, SiLU(gate)*up + quantise, GEMM."""
    a_q, sa = quant_1x128(x)
    h1 = gemm_nt_dequant(a_q, sa, gate_up_q, gate_up_s)
    q2, s2 = silu_mul_quant_1x128(h1)
    return gemm_nt_dequant(q2, s2, down_q, down_s)


def deepseek_moe_forward(x, gate_w, bias, n_group, topk_group, top_k, scoring, norm_topk_prob, routed_scaling_factor,
                         w13_q, w13_s, w2_q, w2_s, shared=None, router_logits=None):
    """DeepSeekMoE.forward_impl, FP8 path (tasks/baseline/L2/deepseek_moe.py:209-304): router logits in bf16 (:246-251),
    GroupedTopK with the scaling factor left at 1 (:143-147, :252-255), fp32 router weights into the experts (:266-284),
    x routed_scaling_factor after the experts (:293-295), + shared expert (:297-300).  shared = (gate_up_q, gate_up_s,
    down_q, down_s) or None."""
    logits = torch.nn.functional.linear(x, gate_w) if router_logits is None else router_logits
    tw, ti = route_topk(logits, top_k, scoring, bias=bias, n_group=n_group, topk_group=topk_group, renormalize=norm_topk_prob,
                        score_in_input_dtype=True)
    out = moe_layer(x, w13_q, w13_s, w2_q, w2_s, tw, ti) * routed_scaling_factor
    if shared is not None:
        out = out + swiglu_mlp_fp8(x, *shared)
    return out
