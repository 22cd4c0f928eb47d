"""Drop-in candidate for kb-nano's ``tasks/baseline/L2/fused_experts.py`` (class ``FusedExperts``,
forward at :208-244).  FP8 W8A8 block-scaled experts run through kb_nano_b200's pipeline (the
DeepGEMM-layout sequence of :246-283); like the baseline it returns a new bf16 [T, H] tensor and
leaves every input untouched.  ``w13_scale_dg`` / ``w2_scale_dg`` (DeepGEMM-transformed copies of the
scales) are accepted and ignored: the kernels read the fp32 ``[E, N/128, K/128]`` scales directly,
power of two or not."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import moe  # noqa: E402


class FusedExperts(nn.Module):
    def __init__(self):
        super().__init__()

    def forward(self, hidden_states: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                topk_ids: torch.Tensor, num_experts: int, w13_scale: torch.Tensor | None = None,
                w2_scale: torch.Tensor | None = None, w13_scale_dg: torch.Tensor | None = None,
                w2_scale_dg: torch.Tensor | None = None, use_fp8_w8a8: bool = False,
                block_shape: list[int] | None = None) -> torch.Tensor:
        if not use_fp8_w8a8 or w13.dtype != torch.float8_e4m3fn:
            raise NotImplementedError("kb_nano_b200 implements the FP8 W8A8 expert path only (use_fp8_w8a8=True)")
        if block_shape is not None and list(block_shape) != [128, 128]:
            raise NotImplementedError(f"block_shape {block_shape}: only 128x128 weight blocks are supported")
        if w13_scale is None or w2_scale is None:
            raise ValueError("w13_scale and w2_scale are required for FP8 experts")
        return moe.fused_experts_fp8(hidden_states, w13, w2, topk_weights, topk_ids, num_experts, w13_scale, w2_scale)
