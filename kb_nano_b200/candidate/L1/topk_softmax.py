"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/topk_softmax.py`` (class ``TopKSoftmax``, forward at
:37-60): softmax over the router logits in fp32, top-k, optional renormalisation by the sum clamped at 1e-20.
One kernel of kb_nano_b200 instead of the baseline's softmax / topk / divide / two copies; like the baseline it
returns views of buffers that persist between calls (CUDA-graph friendly) and float32 weights / int32 ids."""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops  # noqa: E402


class TopKSoftmax(nn.Module):
    def __init__(self):
        super().__init__()
        self._topk_weights = None
        self._topk_ids = None

    def _ensure_buffers(self, M, top_k, device):
        if (self._topk_weights is None or self._topk_weights.size(0) < M or self._topk_weights.size(1) != top_k
                or self._topk_weights.device != device):
            self._topk_weights = torch.empty(M, top_k, dtype=torch.float32, device=device)
            self._topk_ids = torch.empty(M, top_k, dtype=torch.int32, device=device)

    def forward(self, router_logits: torch.Tensor, top_k: int, renormalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
        M = router_logits.size(0)
        self._ensure_buffers(M, top_k, router_logits.device)
        logits = router_logits if router_logits.dtype in (torch.float32, torch.bfloat16) else router_logits.float()
        logits = logits if logits.stride(-1) == 1 else logits.contiguous()
        topk_weights, topk_ids = self._topk_weights[:M], self._topk_ids[:M]
        ops.moe_route_topk(logits, top_k, "softmax", renormalize=renormalize, renorm_floor=1e-20, out_w=topk_weights, out_ids=topk_ids)
        return topk_weights, topk_ids
