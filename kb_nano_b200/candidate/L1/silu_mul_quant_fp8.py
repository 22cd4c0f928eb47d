"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/silu_mul_quant_fp8.py`` (class
``SiluMulQuantFp8``, forward at :87-143): same arguments, same asserts, same outputs --
fp8 [M, N//2] row-major and fp32 scales [M, (N//2)//128] with strides (1, M)."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops, torch_ops  # noqa: E402,F401

_GROUP_SIZE = 128


class SiluMulQuantFp8(nn.Module):
    def forward(self, input: torch.Tensor, output: torch.Tensor | None = None, use_ue8m0: bool = True,
                eps: float = 1e-10) -> tuple[torch.Tensor, torch.Tensor]:
        assert input.ndim == 2
        M, N = input.size()
        N_2 = N // 2
        assert M % _GROUP_SIZE == 0, f"M={M} must be divisible by {_GROUP_SIZE}"
        assert N_2 % _GROUP_SIZE == 0, f"N//2={N_2} must be divisible by {_GROUP_SIZE}"
        if output is None:
            output = torch.empty((M, N_2), dtype=torch.float8_e4m3fn, device=input.device)
        output_scales = torch.empty((N_2 // _GROUP_SIZE, M), dtype=torch.float32, device=input.device).transpose(0, 1)
        if not input.is_contiguous():
            input = input.contiguous()
        if torch.compiler.is_compiling():
            torch.ops.kbn_b200.silu_mul_quant_fp8(input, output, output_scales, use_ue8m0, eps)
        else:
            ops.silu_mul_quant_fp8(input, output, output_scales, use_ue8m0, eps)
        return output, output_scales
