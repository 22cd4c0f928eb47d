"""The C-ABI kernels as opaque torch.library custom ops (namespace ``kbn_b200``).

kb-nano wraps its FP8 kernels the same way (``torch.ops.kb_nano_fp8.*``,
tasks/baseline/L1/fp8_linear.py:85-178; ``torch.ops.kb_nano_fp8_moe.*``,
tasks/baseline/L1/fp8_grouped_gemm_contiguous.py:100-133) so that torch.compile treats them as
single in-place nodes and never traces into them.  Outputs are caller-allocated and mutated.
"""
from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("kbn_b200::per_token_group_quant_fp8", mutates_args=("output_fp8", "output_scale"))
def per_token_group_quant_fp8(input: torch.Tensor, output_fp8: torch.Tensor, output_scale: torch.Tensor,
                              use_ue8m0: bool = True, eps: float = 1e-10) -> None:
    ops.per_token_group_quant_fp8(input, output_fp8, output_scale, use_ue8m0, eps)


@torch.library.custom_op("kbn_b200::silu_mul_quant_fp8", mutates_args=("output_fp8", "output_scale"))
def silu_mul_quant_fp8(input: torch.Tensor, output_fp8: torch.Tensor, output_scale: torch.Tensor,
                       use_ue8m0: bool = True, eps: float = 1e-10) -> None:
    ops.silu_mul_quant_fp8(input, output_fp8, output_scale, use_ue8m0, eps)


@torch.library.custom_op("kbn_b200::fp8_gemm_nt", mutates_args=("output",))
def fp8_gemm_nt(a_fp8: torch.Tensor, a_scale: torch.Tensor, b_fp8: torch.Tensor, b_scale: torch.Tensor,
                output: torch.Tensor) -> None:
    ops.fp8_gemm_nt_auto(a_fp8, a_scale, b_fp8, b_scale, output)


@torch.library.custom_op("kbn_b200::m_grouped_gemm_nt_contiguous", mutates_args=("c_bf16",))
def m_grouped_gemm_nt_contiguous(a_fp8: torch.Tensor, a_scale: torch.Tensor, b_fp8: torch.Tensor,
                                 b_scale: torch.Tensor, c_bf16: torch.Tensor, expert_ids: torch.Tensor) -> None:
    ops.m_grouped_fp8_gemm_nt_contiguous(a_fp8, a_scale, b_fp8, b_scale, c_bf16, expert_ids)


@torch.library.custom_op("kbn_b200::m_grouped_gemm_nt_masked", mutates_args=("c_bf16",))
def m_grouped_gemm_nt_masked(a_fp8: torch.Tensor, a_scale: torch.Tensor, b_fp8: torch.Tensor,
                             b_scale: torch.Tensor, c_bf16: torch.Tensor, masked_m: torch.Tensor) -> None:
    ops.m_grouped_fp8_gemm_nt_masked(a_fp8, a_scale, b_fp8, b_scale, c_bf16, masked_m)
