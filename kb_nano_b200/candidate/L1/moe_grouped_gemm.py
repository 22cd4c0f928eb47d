"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/moe_grouped_gemm.py`` (class ``MoeGroupedGemm``,
forward at :294-382), the sorted-token grouped GEMM that kb-nano's Triton MoE path calls twice per
layer (``tasks/baseline/L2/fused_experts.py:285-347``, ``tasks/baseline/L2/vllm_fused_experts.py``).

Contract kept from the Triton kernel (:86-189): row ``t`` of ``C`` (``t = sorted_token_ids[i]``, valid
when ``t < A.size(0) * top_k``) is ``dequant(A[t // top_k]) @ dequant(B[e])^T`` with ``e`` the expert of
the ``BLOCK_SIZE_M`` block that position ``i`` falls in, optionally times ``topk_weights.flat[t]``,
written to ``C`` in place; with ``sorted_token_ids=None`` block ``i`` holds the single row ``t = i``.

How it is computed here: one small kernel reads the (row -> expert) map back out of the sorted lists
(``kbn_moe_pair_experts``), the rows are regrouped into 128-aligned expert segments by ``kbn_moe_permute``,
multiplied by this library's grouped FP8 GEMM (UE8M0 tensor-core path when every weight scale is a power of
two, fp32-scale path otherwise) and written back to ``C[t]`` by ``kbn_moe_unpermute_combine`` with one slot
per row.  The scratch buffers only grow and are kept per device (a captured CUDA graph may hold their
addresses).  FP8 block-scaled inputs only.
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


_SCRATCH: dict = {}      # device -> {name: flat tensor}; buffers only ever grow
_RETIRED: list = []      # outgrown buffers stay alive: a captured CUDA graph may still hold their addresses


def _scratch(dev: torch.device, n_pairs: int, m_cap: int, k: int, n: int, ws_bytes: int) -> dict:
    want = {"pair_expert": (n_pairs, torch.int32), "dest_row": (n_pairs, torch.int32), "row_expert": (m_cap, torch.int32),
            "a_perm": (m_cap * k, _FP8), "a_s_perm": (m_cap * (k // 128), torch.float32), "out": (m_cap * n, torch.bfloat16),
            "workspace": (ws_bytes, torch.uint8), "ones": (n_pairs, torch.float32)}
    sc = _SCRATCH.setdefault((dev.type, dev.index), {})
    for name, (numel, dtype) in want.items():
        cur = sc.get(name)
        if cur is None or cur.numel() < numel:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("MoeGroupedGemm: scratch would have to grow during stream capture; run the largest shape eagerly first")
            if cur is not None:
                _RETIRED.append(cur)
            sc[name] = torch.ones(numel, dtype=dtype, device=dev) if name == "ones" else torch.empty(numel, dtype=dtype, device=dev)
    return sc


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

        if C.dtype != torch.bfloat16 or C.shape[0] < n_pairs or C.shape[1] != n or not C.is_contiguous():
            raise ValueError("C must be contiguous bf16 [M*top_k, N]")
        m_cap = ops.moe_aligned_rows(m, top_k, e)
        sc = _scratch(dev, n_pairs, m_cap, k, n, ops.moe_permute_workspace_bytes(m, top_k, e))

        # expert of every row t of C (-1: the row appears in no block), without a host sync
        blocks = expert_ids.reshape(-1)
        blocks = blocks if blocks.dtype == torch.int32 and blocks.is_contiguous() else blocks.to(torch.int32).contiguous()
        ids = None
        if sorted_token_ids is not None:
            ids = sorted_token_ids.reshape(-1)
            ids = ids if ids.dtype == torch.int32 and ids.is_contiguous() else ids.to(torch.int32).contiguous()
        pair_expert = sc["pair_expert"][:n_pairs]
        ops.moe_pair_experts(ids, blocks, bm, pair_expert)
        topk_ids = pair_expert.view(m, top_k)

        a_s = a_scale if a_scale.is_contiguous() else a_scale.contiguous()
        a_q = A if A.is_contiguous() else A.contiguous()
        a_perm = sc["a_perm"][: m_cap * k].view(m_cap, k)
        a_s_perm = sc["a_s_perm"][: m_cap * (k // 128)].view(m_cap, k // 128)
        row_expert = sc["row_expert"][:m_cap]
        dest_row = sc["dest_row"][:n_pairs].view(m, top_k)
        ops.moe_permute(a_q, a_s, topk_ids, e, a_perm, a_s_perm, row_expert, dest_row, sc["workspace"])

        out = sc["out"][: m_cap * n].view(m_cap, n)
        packed = ops.packed_weight_scales(b_scale, n, k)
        if packed is not None:
            # activation scales from kb-nano's quantiser are powers of two (tasks/baseline/L1/fp8_linear.py:163-168,237)
            ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(a_perm, ops.pack_sf_rows(a_s_perm, k), B, packed, out, row_expert)
        else:
            ops.m_grouped_fp8_gemm_nt_contiguous(a_perm, a_s_perm, B, b_scale, out, row_expert)

        if mul_routed_weight and topk_weights is not None:
            w = topk_weights.reshape(-1).float()[:n_pairs].contiguous().view(n_pairs, 1)
        else:
            w = sc["ones"][:n_pairs].view(n_pairs, 1)
        ops.moe_unpermute_combine(out, dest_row.view(n_pairs, 1), w, C[:n_pairs])
