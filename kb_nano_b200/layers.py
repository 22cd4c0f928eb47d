"""MoE layers a model can reach: router -> FP8 experts -> scaling -> shared expert, expert-parallel.

Host-side mirror of kb-nano's three L2 MoE blocks for their FP8 W8A8 path --

  Qwen3MoE      tasks/baseline/L2/qwen3_moe.py:24-193     (gate -> TopKSoftmax -> FusedExperts -> all-reduce)
  MixtralMoE    tasks/baseline/L2/mixtral_moe.py:15-88    (the same with renormalize=True and weights cast to the
                                                            activations' dtype)
  DeepSeekMoE   tasks/baseline/L2/deepseek_moe.py:39-304  (shared expert on a side stream, bf16 router logits,
                                                            GroupedTopK with e_score_correction_bias, VllmFusedExperts,
                                                            x routed_scaling_factor after the experts, + shared, all-reduce)

-- with the same constructor arguments, parameter names, weight-loader signatures and forward() contract, and one
structural difference: where kb-nano shards every expert's intermediate dimension over the ranks (tensor parallel)
and all-reduces the layer output (tasks/baseline/L1/allreduce.py:37-48), these layers give each rank a contiguous
block of whole experts and exchange tokens instead (`ep.EpMoe`: peer stores over NVLink).  The layer output is
then complete on the rank that owns the tokens and no all-reduce follows.  With one rank the experts run through
the single-GPU pipeline (`moe.fused_experts_fp8`).  The weight loaders therefore keep an expert's full 2I / I
rows and skip experts of other ranks; the shared expert of DeepSeekMoE is replicated.

Everything on the hot path is a kernel of this library (routing, quantisation, grouped GEMMs, activation,
exchange, weighted sum); the router's small bf16 GEMM is torch's (a plain library GEMM outside the FP8 path).
bf16 expert weights are refused: the FP8 path is what this package implements.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ep as _ep
from . import moe as _moe
from . import ops as _ops

FP8 = torch.float8_e4m3fn
_BLOCK = 128


def _world(group=None) -> tuple[int, int]:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def _scale_shape(out_dim: int, in_dim: int) -> tuple[int, int]:
    return (math.ceil(out_dim / _BLOCK), math.ceil(in_dim / _BLOCK))


class _MoeBlock(nn.Module):
    """What the three layers share: the FP8 weights of this rank's block of experts under kb-nano's parameter
    names (registered on the layer itself, so checkpoint names map as they do for the baseline classes), their
    loaders, the call that runs the experts (single-GPU pipeline or expert-parallel exchange), the custom-op switch
    kb-nano's engine flips (`_use_custom_op`, `_layer_name`) and forward() around forward_impl()."""

    def _init_experts(self, num_experts: int, hidden: int, inter: int, top_k: int, scale_names: tuple[str, str], group=None,
                      ep_max_tokens: int = 256, ep_max_m: int = 256):
        self.num_experts, self.hidden_size, self.moe_intermediate, self.top_k = num_experts, hidden, inter, top_k
        self.ep_rank, self.ep_size = _world(group)
        self.tp_size = self.ep_size              # kb-nano's attribute name for the number of ranks the layer spans
        self._group = group
        self.expert_lo, self.expert_hi = _ep.expert_range(self.ep_rank, self.ep_size, num_experts)
        e_l = self.expert_hi - self.expert_lo
        self._scale_names = scale_names
        self.w13 = nn.Parameter(torch.empty(e_l, 2 * inter, hidden, dtype=FP8), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(e_l, hidden, inter, dtype=FP8), requires_grad=False)
        setattr(self, scale_names[0], nn.Parameter(torch.ones(e_l, *_scale_shape(2 * inter, hidden), dtype=torch.float32), requires_grad=False))
        setattr(self, scale_names[1], nn.Parameter(torch.ones(e_l, *_scale_shape(hidden, inter), dtype=torch.float32), requires_grad=False))
        self.w13.weight_loader = self._w13_weight_loader
        self.w2.weight_loader = self._w2_weight_loader
        getattr(self, scale_names[0]).weight_loader = self._w13_scale_loader
        getattr(self, scale_names[1]).weight_loader = self._w2_scale_loader
        self.ep_max_tokens, self.ep_max_m = ep_max_tokens, ep_max_m
        self._ep_layer: _ep.EpMoe | None = None
        self._use_custom_op = False
        self._layer_name = ""

    # loaders: kb-nano's signatures (qwen3_moe.py:131-159, deepseek_moe.py:182-202); a checkpoint tensor holds one
    # expert's full w1 / w3 / w2 (or its block scales); experts of other ranks are skipped, nothing is narrowed
    def _local(self, expert_id: int) -> int | None:
        return expert_id - self.expert_lo if self.expert_lo <= expert_id < self.expert_hi else None

    def _w13_weight_loader(self, param, loaded_weight, expert_id: int, is_w1: bool):
        le = self._local(expert_id)
        if le is None:
            return
        n = self.moe_intermediate
        off = 0 if is_w1 else n
        param.data[le, off:off + n, :].copy_(loaded_weight)

    def _w2_weight_loader(self, param, loaded_weight, expert_id: int):
        le = self._local(expert_id)
        if le is not None:
            param.data[le].copy_(loaded_weight)

    def _w13_scale_loader(self, param, loaded_weight, expert_id: int, is_w1: bool):
        le = self._local(expert_id)
        if le is None:
            return
        rows = math.ceil(self.moe_intermediate / _BLOCK)
        off = 0 if is_w1 else rows
        param.data[le, off:off + rows, :].copy_(loaded_weight)

    def _w2_scale_loader(self, param, loaded_weight, expert_id: int):
        le = self._local(expert_id)
        if le is not None:
            param.data[le].copy_(loaded_weight)

    def configure_ep(self, max_tokens: int, max_m: int | None = None) -> None:
        """Sizes the expert-parallel context (tokens per rank and call, rows an expert may receive per call).  A
        collective step when the world is larger than one: every rank calls it, before any CUDA-graph capture."""
        self.ep_max_tokens = max_tokens
        if max_m is not None:
            self.ep_max_m = max_m
        if self._ep_layer is not None:
            self._ep_layer.close()
            self._ep_layer = None

    def _ep(self, x: torch.Tensor) -> "_ep.EpMoe":
        t = x.shape[0]
        if t > self.ep_max_tokens:
            raise ValueError(f"{t} tokens in one call, the expert-parallel context holds {self.ep_max_tokens}: call configure_ep() "
                             "on every rank with the largest batch first")
        if self._ep_layer is None:
            self._ep_layer = _ep.EpMoe(self.ep_rank, self.ep_size, self.num_experts, self.hidden_size, self.moe_intermediate,
                                       max_tokens=self.ep_max_tokens, topk=self.top_k, max_m=self.ep_max_m, group=self._group,
                                       device=x.device)
        return self._ep_layer

    def _route_and_run(self, x: torch.Tensor, router_logits: torch.Tensor, **route) -> torch.Tensor:
        """Router logits -> experts.  One rank: the routing kernel, then the single-GPU pipeline.  Several ranks: the
        expert-parallel layer routes inside its dispatch kernel."""
        if self.ep_size == 1:
            tw, ti = _ops.moe_route_topk(router_logits, self.top_k, **route)
            return self._run_experts(x, tw, ti)
        w13_s, w2_s = getattr(self, self._scale_names[0]), getattr(self, self._scale_names[1])
        lg = router_logits if router_logits.stride(-1) == 1 else router_logits.contiguous()
        return self._ep(x).forward_routed(x, lg, self.w13, w13_s, self.w2, w2_s, **route)

    def _run_experts(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        w13_s, w2_s = getattr(self, self._scale_names[0]), getattr(self, self._scale_names[1])
        if self.ep_size == 1:
            return _moe.fused_experts_fp8(x, self.w13, self.w2, topk_weights, topk_ids, self.num_experts, w13_s, w2_s)
        return self._ep(x).forward(x, topk_ids, topk_weights, self.w13, w13_s, self.w2, w2_s)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self._use_custom_op:
            return torch.ops.kb_nano.moe_forward(hidden_states, self._layer_name)
        return self.forward_impl(hidden_states)

    @staticmethod
    def _require_fp8(quant_config, who: str):
        if quant_config is None:
            raise NotImplementedError(f"{who}: kb_nano_b200 implements the FP8 W8A8 block-scaled experts only (pass quant_config)")
        block = list(quant_config.get("weight_block_size", [128, 128]))
        if block != [128, 128]:
            raise NotImplementedError(f"{who}: weight_block_size {block}: only 128x128 weight blocks are supported")


class Qwen3MoE(_MoeBlock):
    """tasks/baseline/L2/qwen3_moe.py:24-193.  Parameters: gate.weight [E, H] bf16 (replicated), w13 / w13_scale /
    w2 / w2_scale of this rank's experts."""

    def __init__(self, config, quant_config: dict | None = None, group=None):
        super().__init__()
        self._require_fp8(quant_config, "Qwen3MoE")
        self.num_experts = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.hidden_size = config.hidden_size
        self.renormalize = getattr(config, "norm_topk_prob", True)
        self.use_fp8 = True
        self.block_shape = [128, 128]
        self.gate = nn.Linear(config.hidden_size, config.num_experts, bias=False, dtype=torch.bfloat16)
        self._init_experts(config.num_experts, config.hidden_size, config.moe_intermediate_size, config.num_experts_per_tok,
                           ("w13_scale", "w2_scale"), group)

    def forward_impl(self, hidden_states: torch.Tensor) -> torch.Tensor:
        orig_shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        x = x if x.is_contiguous() else x.contiguous()
        router_logits = self.gate(x)
        # TopKSoftmax (tasks/baseline/L1/topk_softmax.py:37-60): fp32 softmax, top-k, division by the sum clamped at 1e-20
        out = self._route_and_run(x, router_logits, scoring="softmax", renormalize=self.renormalize, renorm_floor=1e-20)
        return out.view(orig_shape)


class MixtralMoE(_MoeBlock):
    """tasks/baseline/L2/mixtral_moe.py:15-88 with FP8 block-scaled expert weights (the baseline class holds bf16
    experts; `quant_config` is this class's addition and required).  Router weights are rounded to the activations'
    dtype before they weigh the expert outputs, as the baseline does (:72)."""

    def __init__(self, config, quant_config: dict | None = None, group=None):
        super().__init__()
        self._require_fp8(quant_config, "MixtralMoE")
        self.num_experts = config.num_local_experts
        self.top_k = config.num_experts_per_tok
        self.hidden_size = config.hidden_size
        self.gate = nn.Linear(config.hidden_size, config.num_local_experts, bias=False, dtype=torch.bfloat16)
        self._init_experts(config.num_local_experts, config.hidden_size, config.intermediate_size, config.num_experts_per_tok,
                           ("w13_scale", "w2_scale"), group)

    def forward_impl(self, hidden_states: torch.Tensor) -> torch.Tensor:
        orig_shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        x = x if x.is_contiguous() else x.contiguous()
        router_logits = self.gate(x)
        tw, ti = _ops.moe_route_topk(router_logits, self.top_k, "softmax", renormalize=True, renorm_floor=1e-20)
        tw = tw.to(x.dtype).float()              # the baseline's topk_weights.to(hidden_states.dtype)
        out = self._run_experts(x, tw, ti)
        return out.view(orig_shape)


class _SharedExpertFp8(nn.Module):
    """The shared expert: a SwiGLU MLP with FP8 block-scaled weights (kb-nano: LlamaMLP with reduce_results=False,
    tasks/baseline/L2/llama_mlp.py:17-39), replicated on every rank.  Two FP8 linears around the fused
    SiLU*up + quantisation kernel: four launches."""

    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden, inter
        self.gate_up_weight = nn.Parameter(torch.empty(2 * inter, hidden, dtype=FP8), requires_grad=False)
        self.gate_up_scale = nn.Parameter(torch.ones(*_scale_shape(2 * inter, hidden), dtype=torch.float32), requires_grad=False)
        self.down_weight = nn.Parameter(torch.empty(hidden, inter, dtype=FP8), requires_grad=False)
        self.down_scale = nn.Parameter(torch.ones(*_scale_shape(hidden, inter), dtype=torch.float32), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t, h, i = x.shape[0], self.hidden_size, self.intermediate_size
        dev = x.device
        a_q = torch.empty(t, h, dtype=FP8, device=dev)
        a_s = torch.empty(h // _BLOCK, t, device=dev).t()
        gu = torch.empty(t, 2 * i, dtype=torch.bfloat16, device=dev)
        _ops.fp8_linear(x, a_q, a_s, self.gate_up_weight, self.gate_up_scale, gu)
        q2 = torch.empty(t, i, dtype=FP8, device=dev)
        s2 = torch.empty(i // _BLOCK, t, device=dev).t()
        _ops.silu_mul_quant_fp8(gu, q2, s2)
        out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)
        _ops.fp8_gemm_nt_auto(q2, s2, self.down_weight, self.down_scale, out)
        return out


class DeepSeekMoE(_MoeBlock):
    """tasks/baseline/L2/deepseek_moe.py:39-304, FP8 path.  Parameters: gate_weight [E, H], e_score_correction_bias
    [E] (topk_method 'noaux_tc' only), w13 / w2 / w13_weight_scale_inv / w2_weight_scale_inv of this rank's experts,
    shared_expert.*.  The shared expert runs on a side stream while the routed experts run (`VLLM_DISABLE_SHARED_
    EXPERTS_STREAM` != 0 puts it on the main stream, as in the baseline, :165-172)."""

    def __init__(self, config, quant_config: dict | None = None, group=None):
        super().__init__()
        self._require_fp8(quant_config, "DeepSeekMoE")
        import os
        self.num_experts = config.n_routed_experts
        self.top_k = config.num_experts_per_tok
        self.hidden_size = config.hidden_size
        self.routed_scaling_factor = getattr(config, "routed_scaling_factor", 1.0)
        self.use_fp8 = True
        self.n_group = getattr(config, "n_group", 1)
        self.topk_group = getattr(config, "topk_group", 1)
        self.scoring_func = getattr(config, "scoring_func", "softmax")
        self.norm_topk_prob = getattr(config, "norm_topk_prob", True)
        self.topk_method = getattr(config, "topk_method", "noaux_tc")
        self.gate_weight = nn.Parameter(torch.empty(config.n_routed_experts, config.hidden_size, dtype=torch.bfloat16), requires_grad=False)
        self.gate_weight.weight_loader = lambda p, w: p.data.copy_(w)
        if self.topk_method == "noaux_tc":
            self.e_score_correction_bias = nn.Parameter(torch.zeros(config.n_routed_experts, dtype=torch.float32), requires_grad=False)
            self.e_score_correction_bias.weight_loader = lambda p, w: p.data.copy_(w)
        else:
            self.register_parameter("e_score_correction_bias", None)
        n_shared = getattr(config, "n_shared_experts", 1)
        self.shared_expert = (_SharedExpertFp8(config.hidden_size, config.moe_intermediate_size * n_shared)
                              if n_shared is not None and n_shared > 0 else None)
        self._init_experts(config.n_routed_experts, config.hidden_size, config.moe_intermediate_size, config.num_experts_per_tok,
                           ("w13_weight_scale_inv", "w2_weight_scale_inv"), group)
        self._disable_shared_stream = os.environ.get("VLLM_DISABLE_SHARED_EXPERTS_STREAM", "0") != "0"
        self._shared_stream: torch.cuda.Stream | None = None

    def forward_impl(self, hidden_states: torch.Tensor) -> torch.Tensor:
        orig_shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        x = x if x.is_contiguous() else x.contiguous()
        shared_out = None
        side = self.shared_expert is not None and not self._disable_shared_stream
        if side:
            if self._shared_stream is None:
                self._shared_stream = torch.cuda.Stream(x.device)
            self._shared_stream.wait_stream(torch.cuda.current_stream(x.device))
            with torch.cuda.stream(self._shared_stream):
                shared_out = self.shared_expert(x)
        elif self.shared_expert is not None:
            shared_out = self.shared_expert(x)
        # bf16 router logits for the FP8 expert path (deepseek_moe.py:246-251), GroupedTopK with the factor left at 1
        # (:143-147), fp32 router weights straight into the experts (:266-284)
        router_logits = F.linear(x, self.gate_weight)
        bias = self.e_score_correction_bias
        out = self._route_and_run(x, router_logits, scoring=self.scoring_func, bias=bias.float().contiguous() if bias is not None else None,
                                  n_group=self.n_group, topk_group=self.topk_group, renormalize=self.norm_topk_prob,
                                  round_bf16=router_logits.dtype == torch.bfloat16)
        out = out * self.routed_scaling_factor               # after the experts (:293-295)
        if shared_out is not None:
            if side:
                main = torch.cuda.current_stream(x.device)
                main.wait_stream(self._shared_stream)
                shared_out.record_stream(main)
            out = out + shared_out
        return out.view(orig_shape)
