"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/rmsnorm_quant.py`` (classes ``RMSNormFP8Quant`` :63-97
and ``FusedAddRMSNormFP8Quant`` :100-132): same arguments, outputs fp8 ``[tokens, hidden]`` and fp32 scales
``[tokens, hidden/128]`` in column-major layout; the add form modifies ``input`` and ``residual`` in place."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops  # noqa: E402

_FP8_GROUP_SIZE = 128


def _outputs(input: torch.Tensor):
    hidden_size = input.size(-1)
    num_tokens = input.numel() // hidden_size
    num_groups = (hidden_size + _FP8_GROUP_SIZE - 1) // _FP8_GROUP_SIZE
    output_fp8 = torch.empty(num_tokens, hidden_size, dtype=torch.float8_e4m3fn, device=input.device)
    output_scales = torch.empty(num_groups, num_tokens, dtype=torch.float32, device=input.device).transpose(0, 1)
    return output_fp8, output_scales, num_tokens, hidden_size


class RMSNormFP8Quant(nn.Module):
    def forward(self, input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
        output_fp8, output_scales, t, h = _outputs(input)
        x2 = input.reshape(t, h)
        ops.rmsnorm_quant_fp8(x2 if x2.is_contiguous() else x2.contiguous(), weight, output_fp8, output_scales, eps)
        return output_fp8, output_scales


class FusedAddRMSNormFP8Quant(nn.Module):
    def forward(self, input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Modifies *input* and *residual* in-place."""
        output_fp8, output_scales, t, h = _outputs(input)
        if not input.is_contiguous() or not residual.is_contiguous():
            raise ValueError("input and residual must be contiguous (they are updated in place)")
        ops.rmsnorm_quant_fp8(input.view(t, h), weight, output_fp8, output_scales, eps, residual=residual.view(t, h))
        return output_fp8, output_scales, residual
