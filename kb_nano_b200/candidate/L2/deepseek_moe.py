"""Drop-in candidate for kb-nano's ``tasks/baseline/L2/deepseek_moe.py (class DeepSeekMoE, forward_impl at :209-304)``: the FP8 W8A8 MoE block with the
same constructor arguments, parameter names, weight-loader signatures and forward contract, expert-parallel where
the baseline is tensor-parallel -- each rank owns a block of whole experts, tokens travel by peer stores over NVLink
and no all-reduce follows (``kb_nano_b200/layers.py`` holds the implementation and says what differs).  bf16
experts are refused."""
from __future__ import annotations

import importlib.util
import os

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200.layers import DeepSeekMoE  # noqa: E402,F401

__all__ = ["DeepSeekMoE"]
