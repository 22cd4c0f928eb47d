"""Drop-in candidate for kb-nano's ``tasks/baseline/L1/fp8_linear.py``.

kb-nano's kernel swapper loads ``<candidate dir>/L1/fp8_linear.py`` and replaces the baseline
class named like the file's last nn.Module (``Fp8Linear``; infra/kernel_swapper.py:131-144,
328-355).  Signatures, tensor layouts and in-place/ownership rules follow the baseline
(tasks/baseline/L1/fp8_linear.py:282-297 ``PerTokenGroupQuantFp8``, :335-450 ``Fp8Linear``);
the work is done by kb_nano_b200's sm_100a kernels instead of Triton / vLLM / DeepGEMM.
"""
from __future__ import annotations

import importlib.util
import math
import os

import torch
import torch.nn as nn

_spec = importlib.util.spec_from_file_location(
    "_kbn_candidate_bootstrap", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_bootstrap.py"))
_spec.loader.exec_module(importlib.util.module_from_spec(_spec))

from kb_nano_b200 import ops, torch_ops  # noqa: E402,F401

_GROUP = 128


def _alloc_colmajor_scale(M: int, num_groups: int, device: torch.device) -> torch.Tensor:
    """fp32 [M, num_groups] with strides (1, M): the layout the baseline quantises into
    (tasks/baseline/L1/fp8_linear.py:300-313)."""
    return torch.empty((num_groups, M), device=device, dtype=torch.float32).permute(-1, -2)


def unpack_ue8m0_packed_scales(sf: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """fp32 [ceil(N/128), ceil(K/128)] block scales from the packed layout DeepGEMM's sm_100
    ``transform_sf_into_required_layout`` emits for weights: int32 [N, ceil(K/128/4)], one row per
    output channel, each int32 holding the UE8M0 exponent bytes of four consecutive K-blocks
    (lowest byte first).  Assumed layout (DeepGEMM is not part of the kb-nano tree; kb-nano itself only passes
    the tensor through, tasks/baseline/L1/fp8_linear.py:502-512): any other shape is refused rather than
    guessed at, and the 128 rows of a block must agree."""
    nb, kb = math.ceil(N / _GROUP), math.ceil(K / _GROUP)
    if sf.dtype != torch.int32 or sf.dim() != 2 or tuple(sf.shape) != (N, math.ceil(kb / 4)):
        raise ValueError(f"packed UE8M0 weight scales must be int32 [{N}, {math.ceil(kb / 4)}] for a [{N}, {K}] weight, "
                         f"got {sf.dtype} {tuple(sf.shape)}")
    rows = sf[::_GROUP][:nb].contiguous()
    if not torch.equal(rows.repeat_interleave(_GROUP, dim=0)[:N], sf):
        raise ValueError("packed UE8M0 weight scales: rows of one 128-row block differ; not a 128x128 block-scale layout")
    exps = rows.view(torch.uint8).view(nb, -1)[:, :kb].to(torch.int32)
    return torch.pow(2.0, (exps - 127).float())


def postprocess_fp8_weights(weight_fp8: torch.Tensor, scale_inv: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Load-time step of the same name in the baseline (tasks/baseline/L1/fp8_linear.py:453-512): re-quantise
    a checkpoint's block-scaled FP8 weight to power-of-two scales.  Returns (new weight, fp32 scales
    [ceil(N/128), ceil(K/128)]) -- the layout this file's Fp8Linear reads; no DeepGEMM layout transform is
    needed.  The packed form the tensor core reads is built here as well (and kept with the scales), so that no
    later call, eager or captured, has to check the scales again."""
    N, K = weight_fp8.shape
    w = weight_fp8.clone() if weight_fp8.is_contiguous() else weight_fp8.contiguous()
    s = scale_inv[: math.ceil(N / _GROUP), : math.ceil(K / _GROUP)].to(torch.float32).contiguous().clone()
    ops.requant_weights_ue8m0(w, s)
    if N % _GROUP == 0 and K % _GROUP == 0:
        ops.packed_weight_scales(s, N, K)
    return w, s


def postprocess_fp8_weights_batched(weight_fp8: torch.Tensor, scale_inv: torch.Tensor) -> None:
    """In-place form for 3-D MoE weights [E,N,K] (tasks/baseline/L1/fp8_linear.py:515-554)."""
    assert weight_fp8.ndim == 3
    E, N, K = weight_fp8.shape
    s = scale_inv[:, : math.ceil(N / _GROUP), : math.ceil(K / _GROUP)]
    if s.is_contiguous() and s.dtype == torch.float32 and weight_fp8.is_contiguous():
        ops.requant_weights_ue8m0(weight_fp8, s)
        ops.packed_weight_scales(s, N, K)      # packed copy for the tensor core, made at load time
    else:
        w, s2 = weight_fp8.contiguous(), s.to(torch.float32).contiguous()
        ops.requant_weights_ue8m0(w, s2)
        weight_fp8.copy_(w)
        s.copy_(s2)


class _Fp8PrefillBufs:
    __slots__ = ("a", "s", "o")

    def __init__(self, max_tokens: int, K: int, N: int, device: torch.device):
        self.a = torch.empty(max_tokens, K, dtype=torch.float8_e4m3fn, device=device)
        self.s = _alloc_colmajor_scale(max_tokens, math.ceil(K / _GROUP), device)
        self.o = torch.empty(max_tokens, N, dtype=torch.bfloat16, device=device)


class PerTokenGroupQuantFp8(nn.Module):
    """In-place per-token-group FP8 quantisation; ``out_scale`` may have any strides."""

    def forward(self, x: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor) -> None:
        x = x if x.is_contiguous() else x.contiguous()
        if torch.compiler.is_compiling():
            torch.ops.kbn_b200.per_token_group_quant_fp8(x, out_fp8, out_scale)
        else:
            ops.per_token_group_quant_fp8(x, out_fp8, out_scale)


class Fp8Linear(nn.Module):
    """Block-scaled FP8 linear: 1x128 activation quant (column-major UE8M0 scales) + FP8 GEMM."""

    BLOCK_SIZE = _GROUP
    _FLASHINFER_M_THRESHOLD = 32   # kept for interface parity; there is no separate small-M path

    def __init__(self):
        super().__init__()
        self._a_buf: torch.Tensor | None = None
        self._s_buf: torch.Tensor | None = None
        self._o_buf: torch.Tensor | None = None
        self._pf: _Fp8PrefillBufs | None = None
        self._sf_cache: dict = {}

    def _ensure_buffers(self, max_tokens: int, K: int, N: int, device: torch.device):
        num_groups = math.ceil(K / self.BLOCK_SIZE)
        self._a_buf = torch.empty(max_tokens, K, dtype=torch.float8_e4m3fn, device=device)
        self._s_buf = _alloc_colmajor_scale(max_tokens, num_groups, device)
        self._o_buf = torch.empty(max_tokens, N, dtype=torch.bfloat16, device=device)

    def _block_scales(self, weight_scale_inv: torch.Tensor, N: int, K: int) -> torch.Tensor:
        if weight_scale_inv.dtype == torch.float32:
            return weight_scale_inv[: math.ceil(N / _GROUP), : math.ceil(K / _GROUP)]
        if weight_scale_inv.dtype == torch.int32:
            # keyed by address, shape and version; the entry keeps the int32 tensor alive so the address cannot be reused
            key = (weight_scale_inv.data_ptr(), N, K, weight_scale_inv._version)
            if key not in self._sf_cache:
                self._sf_cache[key] = (unpack_ue8m0_packed_scales(weight_scale_inv, N, K), weight_scale_inv)
            return self._sf_cache[key][0]
        raise TypeError(f"unsupported weight_scale_inv dtype {weight_scale_inv.dtype}")

    def forward(self, input_bf16: torch.Tensor, weight_fp8: torch.Tensor, weight_scale_inv: torch.Tensor,
                bias: torch.Tensor | None = None) -> torch.Tensor:
        N, K = weight_fp8.shape
        input_2d = input_bf16.reshape(-1, K)
        if not input_2d.is_contiguous():
            input_2d = input_2d.contiguous()
        M = input_2d.shape[0]
        num_groups = (K + self.BLOCK_SIZE - 1) // self.BLOCK_SIZE
        dev = input_2d.device
        compiling = torch.compiler.is_compiling()
        if not compiling and self._a_buf is not None and M <= self._a_buf.shape[0]:
            q_input, output = self._a_buf[:M], self._o_buf[:M]
        elif not compiling and self._pf is not None and M <= self._pf.a.shape[0]:
            q_input, output = self._pf.a[:M], self._pf.o[:M]
        else:
            q_input = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=dev)
            output = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        input_scale = _alloc_colmajor_scale(M, num_groups, dev)
        w_scale = self._block_scales(weight_scale_inv, N, K)
        # the bias rides in the GEMM's epilogue (added in fp32 before the rounding to bf16, like the reference's
        # F.linear); under torch.compile the opaque ops have no bias argument and the add stays a torch op
        fused_bias = None
        if bias is not None and not compiling and bias.dtype == torch.bfloat16 and bias.is_contiguous():
            fused_bias = bias
        if compiling:
            torch.ops.kbn_b200.per_token_group_quant_fp8(input_2d, q_input, input_scale)
            torch.ops.kbn_b200.fp8_gemm_nt(q_input, input_scale, weight_fp8, w_scale, output)
        else:
            ops.fp8_linear(input_2d, q_input, input_scale, weight_fp8, w_scale, output, fused_bias)
        if bias is not None and fused_bias is None:
            output = output + bias
        return output.view(*input_bf16.shape[:-1], N)
