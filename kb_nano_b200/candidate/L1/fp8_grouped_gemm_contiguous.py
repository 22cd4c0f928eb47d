"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/fp8_grouped_gemm_contiguous.py`` (class
``Fp8GroupedGemmContiguous`` at :136-170): in-place grouped FP8 GEMM over expert-contiguous rows,
``expert_ids`` int32 per row with -1 marking padding.  Also exports the function form
``m_grouped_fp8_gemm_nt_contiguous((a, sa), (b, sb), out, expert_ids)`` that
tasks/baseline/L2/fused_experts.py:16-23 imports from tasks/baseline/L1/moe_grouped_gemm.py:71-83."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops, torch_ops  # noqa: E402,F401

_ALIGNMENT = 128   # rows of one expert start on a multiple of this (one MMA row block)


def m_grouped_fp8_gemm_nt_contiguous(a_and_scale, b_and_scale, output, expert_ids):
    a, sa = a_and_scale
    b, sb = b_and_scale
    if torch.compiler.is_compiling():
        torch.ops.kbn_b200.m_grouped_gemm_nt_contiguous(a, sa, b, sb, output, expert_ids)
    else:
        ops.m_grouped_fp8_gemm_nt_contiguous(a, sa, b, sb, output, expert_ids)


class Fp8GroupedGemmContiguous(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self._alignment: int = _ALIGNMENT

    def alignment(self) -> int:
        return self._alignment

    def forward(self, a_fp8: torch.Tensor, a_scale: torch.Tensor, b_fp8: torch.Tensor, b_scale: torch.Tensor,
                c_bf16: torch.Tensor, expert_ids: torch.Tensor) -> None:
        m_grouped_fp8_gemm_nt_contiguous((a_fp8, a_scale), (b_fp8, b_scale), c_bf16, expert_ids)
