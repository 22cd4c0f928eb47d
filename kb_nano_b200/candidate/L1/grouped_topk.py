"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/grouped_topk.py`` (class ``GroupedTopK``, forward at
:75-174): DeepSeek-style routing -- sigmoid or softmax scores, an optional selection bias
(``e_score_correction_bias``: biased scores choose, unbiased scores weigh; group score = sum of the group's two
best biased scores, or its best score without a bias), group-limited top-k, renormalisation without an epsilon
and the routed scaling factor -- in one kernel of kb_nano_b200.  Weights come back as float32 and ids as int32,
in descending order of the selection value (the baseline's order is unspecified unless VLLM_BATCH_INVARIANT=1)."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops  # noqa: E402


class GroupedTopK(nn.Module):
    def __init__(self, scoring_func: str = "sigmoid", renormalize: bool = True, routed_scaling_factor: float = 1.0) -> None:
        super().__init__()
        if scoring_func not in ("sigmoid", "softmax"):
            raise ValueError(f"Unsupported scoring function: {scoring_func}")
        self.scoring_func = scoring_func
        self.renormalize = renormalize
        self.routed_scaling_factor = routed_scaling_factor

    def forward(self, gating_output: torch.Tensor, e_score_correction_bias: torch.Tensor | None, num_expert_group: int,
                topk_group: int, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
        logits = gating_output if gating_output.dtype in (torch.float32, torch.bfloat16) else gating_output.float()
        logits = logits if logits.stride(-1) == 1 else logits.contiguous()
        bias = e_score_correction_bias
        if bias is not None:
            bias = bias.float().contiguous()
        # the baseline scores in the dtype of the gating output
        return ops.moe_route_topk(logits, topk, self.scoring_func, bias=bias, n_group=num_expert_group, topk_group=topk_group,
                                  renormalize=self.renormalize, scale=float(self.routed_scaling_factor),
                                  round_bf16=logits.dtype == torch.bfloat16)
