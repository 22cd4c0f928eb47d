"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/moe_grouped_gemm.py`` (class ``MoeGroupedGemm``,
forward at :294-382), the sorted-token grouped GEMM that kb-nano's Triton MoE path calls twice per
layer (``tasks/baseline/L2/fused_experts.py:285-347``, ``tasks/baseline/L2/vllm_fused_experts.py``).

Contract kept from the Triton kernel (:86-189): row ``t`` of ``C`` (``t = sorted_token_ids[i]``, valid
when ``t < A.size(0) * top_k``) is ``dequant(A[t // top_k]) @ dequant(B[e])^T`` with ``e`` the expert of
the ``BLOCK_SIZE_M`` block that position ``i`` falls in, optionally times ``topk_weights.flat[t]``,
written to ``C`` in place; with ``sorted_token_ids=None`` block ``i`` holds the single row ``t = i``.

How it is computed here: the (row -> expert) map is read back out of the sorted lists (a few torch ops
on int32 metadata, as kb-nano's own permute does), the rows are regrouped into 128-aligned expert
segments by ``kbn_moe_permute``, multiplied by this library's grouped FP8 GEMM (UE8M0 tensor-core path
when every weight scale is a power of two, fp32-scale path otherwise) and written back to ``C[t]`` by
``kbn_moe_unpermute_combine`` with one slot per row.  FP8 block-scaled inputs only.
"""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops  # noqa: E402

_FP8 = torch.float8_e4m3fn


def _get_default_config(M: int, E: int = 0, N: int = 0, block_shape: list[int] | None = None) -> dict:
    """Same keys as the baseline's tile configuration (:240-253).  Only BLOCK_SIZE_M matters here: it
    is the block size the caller's ``moe_align`` output is laid out in."""
    if block_shape is not None and len(block_shape) == 2:
        return {"BLOCK_SIZE_M": 64, "BLOCK_SIZE_N": block_shape[0], "BLOCK_SIZE_K": block_shape[1], "GROUP_SIZE_M": 32}
    if M <= 32:
        return {"BLOCK_SIZE_M": 16, "BLOCK_SIZE_N": 128, "BLOCK_SIZE_K": 128, "GROUP_SIZE_M": 1}
    return {"BLOCK_SIZE_M": 64, "BLOCK_SIZE_N": 128, "BLOCK_SIZE_K": 128, "GROUP_SIZE_M": 8}


class MoeGroupedGemm(nn.Module):
    @staticmethod
    def get_config(M: int, N: int = 0, E: int = 0, use_fp8: bool = False, block_shape: list[int] | None = None) -> dict:
        return _get_default_config(M, E, N, block_shape)

    def forward(self, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, topk_weights: torch.Tensor | None,
                sorted_token_ids: torch.Tensor | None, expert_ids: torch.Tensor, num_tokens_post_padded: torch.Tensor,
                mul_routed_weight: bool, top_k: int, config: dict | None = None, a_scale: torch.Tensor | None = None,
                b_scale: torch.Tensor | None = None, use_fp8_w8a8: bool = False, block_shape: list[int] | None = None):
        if not use_fp8_w8a8 or A.dtype != _FP8 or B.dtype != _FP8:
            raise NotImplementedError("kb_nano_b200 implements the FP8 W8A8 grouped GEMM only (use_fp8_w8a8=True)")
        if block_shape is None or list(block_shape) != [128, 128] or a_scale is None or b_scale is None:
            raise NotImplementedError("only 128x128 block-scaled weights with 1x128 activation scales are supported")
        if config is None:
            config = _get_default_config(A.size(0), N=B.size(1))
        bm = int(config["BLOCK_SIZE_M"])
        m, k = A.shape
        e, n, _ = B.shape
        n_pairs = m * top_k
        dev = A.device

        # expert of every row t of C (-1: the row appears in no block), without a host sync
        pair_expert = torch.full((n_pairs + 1,), -1, dtype=torch.int32, device=dev)
        blocks = expert_ids.reshape(-1).to(torch.int32)
        if sorted_token_ids is None:
            cnt = min(blocks.numel(), n_pairs)
            pair_expert[:cnt] = blocks[:cnt]
        else:
            ids = sorted_token_ids.reshape(-1).long()
            pos_expert = blocks.repeat_interleave(bm)[: ids.numel()]
            if pos_expert.numel() < ids.numel():
                ids = ids[: pos_expert.numel()]
            pair_expert.scatter_(0, torch.where(ids < n_pairs, ids, torch.full_like(ids, n_pairs)), pos_expert)
        topk_ids = pair_expert[:n_pairs].view(m, top_k).contiguous()

        a_s = a_scale if a_scale.is_contiguous() else a_scale.contiguous()
        a_q = A if A.is_contiguous() else A.contiguous()
        m_cap = ops.moe_aligned_rows(m, top_k, e)
        a_perm = torch.empty(m_cap, k, dtype=_FP8, device=dev)
        a_s_perm = torch.empty(m_cap, k // 128, dtype=torch.float32, device=dev)
        row_expert = torch.empty(m_cap, dtype=torch.int32, device=dev)
        dest_row = torch.empty(m, top_k, dtype=torch.int32, device=dev)
        workspace = torch.empty(ops.moe_permute_workspace_bytes(m, top_k, e), dtype=torch.uint8, device=dev)
        ops.moe_permute(a_q, a_s, topk_ids, e, a_perm, a_s_perm, row_expert, dest_row, workspace)

        out = torch.empty(m_cap, n, dtype=torch.bfloat16, device=dev)
        packed = ops.packed_weight_scales(b_scale, n, k)
        if packed is not None:
            # activation scales from kb-nano's quantiser are powers of two (tasks/baseline/L1/fp8_linear.py:163-168,237)
            ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(a_perm, ops.pack_sf_rows(a_s_perm, k), B, packed, out, row_expert)
        else:
            ops.m_grouped_fp8_gemm_nt_contiguous(a_perm, a_s_perm, B, b_scale, out, row_expert)

        if mul_routed_weight and topk_weights is not None:
            w = topk_weights.reshape(-1).float()[:n_pairs].contiguous().view(n_pairs, 1)
        else:
            w = torch.ones(n_pairs, 1, dtype=torch.float32, device=dev)
        if C.dtype != torch.bfloat16 or C.shape[0] < n_pairs or C.shape[1] != n or not C.is_contiguous():
            raise ValueError("C must be contiguous bf16 [M*top_k, N]")
        ops.moe_unpermute_combine(out, dest_row.view(n_pairs, 1), w, C[:n_pairs])
