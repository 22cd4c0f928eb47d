"""Drop-in candidate for kb-nano's ``tasks/baseline/L2/vllm_fused_experts.py`` (class ``VllmFusedExperts``,
forward at :115-237), the FP8 block-scaled expert path DeepSeek's MoE layer uses
(``tasks/baseline/L2/deepseek_moe.py:266-284``).  The baseline runs quant -> moe_align -> Triton grouped GEMM
-> silu_and_mul -> quant -> Triton grouped GEMM (x routed weight) -> moe_sum with freshly allocated scratch;
here the same arguments go through kb_nano_b200's pipeline (quant -> permute -> grouped GEMM with the
activation and its quantisation in the epilogue -> grouped GEMM -> weighted sum in fp32).  The routed weight
is applied in the final sum instead of GEMM2's epilogue, which changes roundings only (the bf16 tolerance of
the reference harness, ``bench/kernels/runner.py:31-37``).  ``vllm_fused_experts`` is not a kernel-swapper
target (``infra/kernel_swapper.py:44-68``: DeepSeek is not in the L4 model list), so a maintainer binds this
class by hand: ``deepseek_moe.VllmFusedExperts = VllmFusedExperts`` before the model is built."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import moe  # noqa: E402


class VllmFusedExperts(nn.Module):
    def __init__(self):
        super().__init__()

    def forward(self, hidden_states: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                topk_ids: torch.Tensor, num_experts: int, w13_scale: torch.Tensor, w2_scale: torch.Tensor,
                block_shape: list[int]) -> torch.Tensor:
        assert hidden_states.is_contiguous(), "hidden_states must be contiguous"
        assert w13.stride(-1) == 1 and w2.stride(-1) == 1
        assert topk_weights.size() == topk_ids.size()
        if hidden_states.dtype != torch.bfloat16:
            raise NotImplementedError("kb_nano_b200 takes bf16 activations (the dtype kb-nano's FP8 models run in)")
        if w13.dtype != torch.float8_e4m3fn or w2.dtype != torch.float8_e4m3fn:
            raise NotImplementedError("VllmFusedExperts is the FP8 W8A8 block-scaled path: weights must be float8_e4m3fn")
        if list(block_shape) != [128, 128]:
            raise NotImplementedError(f"block_shape {block_shape}: only 128x128 weight blocks are supported")
        # the baseline allocates its result per call; the scratch behind it is shared between calls of one shape
        return moe.fused_experts_fp8(hidden_states, w13, w2, topk_weights, topk_ids, num_experts, w13_scale, w2_scale)
