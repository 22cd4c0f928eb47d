"""FP8 MoE expert pipeline on one GPU: quant -> permute -> grouped GEMM1 -> fused SiLU*up+quant ->
grouped GEMM2 -> weighted combine.  Mirrors FusedExperts._forward_deep_gemm
(tasks/baseline/L2/fused_experts.py:246-283) step for step, with every step a kernel of this library:
seven launches per layer (GEMM1 applies the activation and its quantisation in its epilogue when the weight
scales are powers of two), no host synchronisation, scratch buffers reused across calls.
"""
from __future__ import annotations

import torch

from . import ops

FP8 = torch.float8_e4m3fn


class MoeScratch:
    """Device buffers of the pipeline for up to `t` tokens of one (topk, E, H, I) layer shape.  Layers run one
    after the other, so one set per shape is shared (kb-nano does the same, fused_experts.py:139-206)."""

    def __init__(self, t: int, topk: int, e: int, h: int, i: int, device: torch.device):
        self.key = (t, topk, e, h, i, str(device))
        self.t_cap, self.topk, self.e, self.h, self.i = t, topk, e, h, i
        m_cap = ops.moe_aligned_rows(t, topk, e)
        self.m_cap = m_cap
        self.a_q = torch.empty(t, h, dtype=FP8, device=device)
        self.a_s = torch.empty(t, h // 128, dtype=torch.float32, device=device)
        self.a_perm = torch.empty(m_cap, h, dtype=FP8, device=device)
        self.a_s_perm = torch.empty(m_cap, h // 128, dtype=torch.float32, device=device)
        self.row_expert = torch.empty(m_cap, dtype=torch.int32, device=device)
        self.dest_row = torch.empty(t, topk, dtype=torch.int32, device=device)
        self.workspace = torch.empty(ops.moe_permute_workspace_bytes(t, topk, e), dtype=torch.uint8, device=device)
        # GEMM1 and GEMM2 outputs share one byte buffer, as they are never alive together
        self.mm = torch.empty(m_cap * max(2 * i, h), dtype=torch.bfloat16, device=device)
        self.a2_q = torch.empty(m_cap, i, dtype=FP8, device=device)
        self.a2_s = torch.empty(i // 128, m_cap, dtype=torch.float32, device=device).t()
        # the same scales in the packed form of the UE8M0 GEMMs, written by the permute and the activation kernel
        self.sf1 = torch.empty(ops.packed_sf_rows_bytes(m_cap, h), dtype=torch.uint8, device=device)
        self.sf2 = torch.empty(ops.packed_sf_rows_bytes(m_cap, i), dtype=torch.uint8, device=device)

    def mm1(self, i: int) -> torch.Tensor:
        return self.mm[: self.m_cap * 2 * i].view(self.m_cap, 2 * i)

    def mm2(self, h: int) -> torch.Tensor:
        return self.mm[: self.m_cap * h].view(self.m_cap, h)

    def for_tokens(self, t: int) -> "MoeScratch":
        """The same memory cut down to `t` <= capacity tokens: every tensor a leading slice of the full one (all layouts
        here are addressed by row, so a prefix of the rows is a valid smaller buffer)."""
        if t == self.t_cap:
            return self
        if t > self.t_cap:
            raise ValueError(f"scratch holds {self.t_cap} tokens, {t} asked for")
        v = object.__new__(MoeScratch)
        v.key = (t,) + self.key[1:]
        v.t_cap, v.topk, v.e, v.h, v.i = t, self.topk, self.e, self.h, self.i
        m = ops.moe_aligned_rows(t, self.topk, self.e)
        v.m_cap = m
        v.a_q, v.a_s = self.a_q[:t], self.a_s[:t]
        v.a_perm, v.a_s_perm, v.row_expert = self.a_perm[:m], self.a_s_perm[:m], self.row_expert[:m]
        v.dest_row = self.dest_row[:t]
        v.workspace = self.workspace
        v.mm = self.mm
        v.a2_q, v.a2_s = self.a2_q[:m], self.a2_s[:m]
        v.sf1, v.sf2 = self.sf1, self.sf2
        return v


_SCRATCH: dict = {}
_RETIRED: list = []      # outgrown sets stay alive: a captured CUDA graph may hold pointers into them


def reserve(t: int, topk: int, e: int, h: int, i: int, device: torch.device) -> MoeScratch:
    """Makes the shared scratch of this layer shape hold at least `t` tokens (the `_ensure_buffers` of this pipeline:
    call it with the largest batch before capturing CUDA graphs)."""
    key = (topk, e, h, i, str(device))
    s = _SCRATCH.get(key)
    if s is None or s.t_cap < t:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the MoE scratch must grow, which a CUDA-graph capture does not allow: call moe.reserve() "
                               "(or the layer, eagerly) with the largest batch first")
        if s is not None:
            _RETIRED.append(s)
        s = MoeScratch(t, topk, e, h, i, device)
        _SCRATCH[key] = s
    return s


def get_scratch(t: int, topk: int, e: int, h: int, i: int, device: torch.device) -> MoeScratch:
    """Scratch for `t` tokens: a view of the shared grow-only set of this layer shape.  A smaller batch never frees
    or moves what a larger one allocated, so pointers baked into captured graphs stay valid."""
    return reserve(t, topk, e, h, i, device).for_tokens(t)


def fused_experts_fp8(hidden_states: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                      topk_ids: torch.Tensor, num_experts: int, w13_scale: torch.Tensor, w2_scale: torch.Tensor,
                      scratch: MoeScratch | None = None, out: torch.Tensor | None = None,
                      use_ue8m0: bool = True, fuse_activation: bool = True) -> torch.Tensor:
    """hidden bf16 [T,H]; w13 fp8 [E,2I,H] + fp32 scales [E,2I/128,H/128]; w2 fp8 [E,H,I] + scales
    [E,H/128,I/128]; topk_weights [T,topk] (fp32 or bf16), topk_ids [T,topk] int -> bf16 [T,H]."""
    t, h = hidden_states.shape
    e, n2, _ = w13.shape
    i = n2 // 2
    topk = topk_ids.shape[1]
    if h % 128 or i % 128:
        raise ValueError(f"hidden size {h} and intermediate size {i} must be multiples of 128")
    dev = hidden_states.device
    sc = scratch if scratch is not None else get_scratch(t, topk, e, h, i, dev)
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    ids = ids if ids.is_contiguous() else ids.contiguous()
    w = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
    w = w if w.is_contiguous() else w.contiguous()
    x = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
    if out is None:
        out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)
    ops.per_token_group_quant_fp8(x, sc.a_q, sc.a_s)
    mm1, mm2 = sc.mm1(i), sc.mm2(h)
    # power-of-two weight scales (checked and packed once per tensor) take the UE8M0 block-scaled GEMM
    p13 = ops.packed_weight_scales(w13_scale, n2, h) if use_ue8m0 else None
    p2 = ops.packed_weight_scales(w2_scale, h, i) if use_ue8m0 else None
    if p13 is not None and p2 is not None:
        # the permute and the activation kernel emit the packed activation scales themselves
        ops.moe_permute(sc.a_q, sc.a_s, ids, num_experts, sc.a_perm, sc.a_s_perm, sc.row_expert, sc.dest_row, sc.workspace, sc.sf1)
        if fuse_activation:
            # GEMM1 applies SiLU(gate)*up and the 1x128 quantisation in its epilogue: no bf16 [M, 2I] round trip
            ops.m_grouped_gemm1_silu_quant_contiguous_ue8m0(sc.a_perm, sc.sf1, w13, p13, sc.a2_q, sc.a2_s, sc.row_expert, sc.sf2)
        else:
            ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(sc.a_perm, sc.sf1, w13, p13, mm1, sc.row_expert)
            ops.silu_mul_quant_fp8_list(mm1, sc.a2_q, sc.a2_s, sc.dest_row.view(-1), packed_sf=sc.sf2)
        ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(sc.a2_q, sc.sf2, w2, p2, mm2, sc.row_expert)
    else:
        ops.moe_permute(sc.a_q, sc.a_s, ids, num_experts, sc.a_perm, sc.a_s_perm, sc.row_expert, sc.dest_row, sc.workspace)
        ops.m_grouped_fp8_gemm_nt_contiguous(sc.a_perm, sc.a_s_perm, w13, w13_scale, mm1, sc.row_expert)
        ops.silu_mul_quant_fp8_list(mm1, sc.a2_q, sc.a2_s, sc.dest_row.view(-1))
        ops.m_grouped_fp8_gemm_nt_contiguous(sc.a2_q, sc.a2_s, w2, w2_scale, mm2, sc.row_expert)
    ops.moe_unpermute_combine(mm2, sc.dest_row, w, out)
    return out


LAUNCHES_PER_LAYER = 7   # quant, rank, offsets, scatter, GEMM1 (+activation), GEMM2, combine
