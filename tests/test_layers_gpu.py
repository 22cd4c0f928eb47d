"""The model-reachable MoE layers (router -> FP8 experts -> scaling -> shared expert) on one GPU against the oracle's
restatement of kb-nano's forward_impl of the same class.  The router's bf16 GEMM is torch's on both sides; the
oracle is handed the GPU's logits so that a near tie in the top-k is not decided by two different bf16 GEMMs."""
import importlib.util
import os
import sys
from types import SimpleNamespace

import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close

pytestmark = pytest.mark.gpu
QUANT = {"weight_block_size": [128, 128]}


def _load(name, cls):
    from kb_nano_b200 import candidate_dir
    spec = importlib.util.spec_from_file_location(f"_candidate_impl_L2_{name}", os.path.join(candidate_dir(), "L2", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return getattr(mod, cls)


def _fill(layer, e, h, i, seed, scale_names):
    """Weights through the layer's own loaders, one expert and one projection at a time, as a checkpoint arrives."""
    from kb_nano_b200 import inputs
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=seed, std=0.05)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=seed + 1, std=0.05)
    s13, s2 = getattr(layer, scale_names[0]), getattr(layer, scale_names[1])
    for ex in range(e):
        layer.w13.weight_loader(layer.w13, w13_q[ex, :i], ex, True)
        layer.w13.weight_loader(layer.w13, w13_q[ex, i:], ex, False)
        s13.weight_loader(s13, w13_s[ex, : i // 128], ex, True)
        s13.weight_loader(s13, w13_s[ex, i // 128:], ex, False)
        layer.w2.weight_loader(layer.w2, w2_q[ex], ex)
        s2.weight_loader(s2, w2_s[ex], ex)
    return w13_q, w13_s, w2_q, w2_s


@pytest.mark.parametrize("name,cls", [("qwen3_moe", "Qwen3MoE"), ("mixtral_moe", "MixtralMoE")])
def test_softmax_routed_layers(cuda_dev, name, cls):
    from kb_nano_b200 import inputs
    t, h, i, e, topk = 80, 512, 256, 8, 2
    if cls == "Qwen3MoE":
        cfg = SimpleNamespace(num_experts=e, num_experts_per_tok=topk, hidden_size=h, moe_intermediate_size=i, norm_topk_prob=True)
    else:
        cfg = SimpleNamespace(num_local_experts=e, num_experts_per_tok=topk, hidden_size=h, intermediate_size=i)
    layer = _load(name, cls)(cfg, QUANT)
    with pytest.raises(NotImplementedError):
        _load(name, cls)(cfg, None)                       # bf16 experts are outside this package
    w = _fill(layer, e, h, i, 11, ("w13_scale", "w2_scale"))
    gate_w = (torch.randn(e, h, generator=torch.Generator().manual_seed(4)) * 0.05).to(torch.bfloat16)
    layer.gate.weight.data.copy_(gate_w)
    layer = layer.to(cuda_dev)
    assert {n for n, _ in layer.named_parameters()} == {"gate.weight", "w13", "w2", "w13_scale", "w2_scale"}
    x = inputs.activations(t, h, seed=5)
    xd = x.to(cuda_dev).view(4, 20, h)                    # the layer flattens leading dimensions and restores them
    out = layer(xd)
    assert out.shape == xd.shape
    logits = torch.nn.functional.linear(xd.view(-1, h), layer.gate.weight).cpu()
    ref = to.qwen3_moe_forward(x, gate_w, *w, top_k=topk, renormalize=True, router_logits=logits, cast_weights=cls == "MixtralMoE")
    assert_gemm_close(out.view(-1, h).cpu(), ref, cls)


@pytest.mark.parametrize("shared_stream", [True, False])
def test_deepseek_moe_layer(cuda_dev, shared_stream, monkeypatch):
    from kb_nano_b200 import inputs
    monkeypatch.setenv("VLLM_DISABLE_SHARED_EXPERTS_STREAM", "0" if shared_stream else "1")
    t, h, i, e, topk = 64, 512, 256, 16, 4
    cfg = SimpleNamespace(n_routed_experts=e, num_experts_per_tok=topk, hidden_size=h, moe_intermediate_size=i, routed_scaling_factor=2.5,
                          n_group=4, topk_group=2, scoring_func="sigmoid", norm_topk_prob=True, topk_method="noaux_tc", n_shared_experts=1)
    layer = _load("deepseek_moe", "DeepSeekMoE")(cfg, QUANT)
    w = _fill(layer, e, h, i, 21, ("w13_weight_scale_inv", "w2_weight_scale_inv"))
    g = torch.Generator().manual_seed(6)
    gate_w = (torch.randn(e, h, generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(e, generator=g) * 0.1
    layer.gate_weight.weight_loader(layer.gate_weight, gate_w)
    layer.e_score_correction_bias.weight_loader(layer.e_score_correction_bias, bias)
    gu_q, gu_s = inputs.weight(2 * i, h, seed=31, std=0.05)
    dn_q, dn_s = inputs.weight(h, i, seed=32, std=0.05)
    se = layer.shared_expert
    se.gate_up_weight.data.copy_(gu_q); se.gate_up_scale.data.copy_(gu_s); se.down_weight.data.copy_(dn_q); se.down_scale.data.copy_(dn_s)
    layer = layer.to(cuda_dev)
    x = inputs.activations(t, h, seed=7)
    xd = x.to(cuda_dev)
    out = layer(xd)
    torch.cuda.synchronize()
    logits = torch.nn.functional.linear(xd, layer.gate_weight).cpu()
    ref = to.deepseek_moe_forward(x, gate_w, bias, 4, 2, topk, "sigmoid", True, 2.5, *w, shared=(gu_q, gu_s, dn_q, dn_s), router_logits=logits)
    assert_gemm_close(out.cpu(), ref, f"DeepSeekMoE, shared expert on a side stream: {shared_stream}")
    # without the shared expert and the scaling the layer is the routed experts alone
    cfg2 = SimpleNamespace(**{**vars(cfg), "n_shared_experts": 0, "routed_scaling_factor": 1.0})
    layer2 = _load("deepseek_moe", "DeepSeekMoE")(cfg2, QUANT)
    _fill(layer2, e, h, i, 21, ("w13_weight_scale_inv", "w2_weight_scale_inv"))
    layer2.gate_weight.data.copy_(gate_w); layer2.e_score_correction_bias.data.copy_(bias)
    out2 = layer2.to(cuda_dev)(xd)
    ref2 = to.deepseek_moe_forward(x, gate_w, bias, 4, 2, topk, "sigmoid", True, 1.0, *w, shared=None, router_logits=logits)
    assert_gemm_close(out2.cpu(), ref2, "DeepSeekMoE, routed experts only")


def test_moe_scratch_only_grows(cuda_dev):
    """A smaller batch after a larger one reuses the larger batch's memory (slices of it) and frees nothing: pointers a
    captured CUDA graph holds stay valid; a captured small-batch graph gives the same result after a larger eager call."""
    from kb_nano_b200 import inputs, moe
    h, i, e, topk = 256, 128, 4, 2
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=1, std=0.05)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=2, std=0.05)
    d = cuda_dev
    wd = [w.to(d) for w in (w13_q, w13_s, w2_q, w2_s)]
    big = moe.get_scratch(1024, topk, e, h, i, d)
    small = moe.get_scratch(8, topk, e, h, i, d)
    assert small.a_perm.data_ptr() == big.a_perm.data_ptr() and small.m_cap < big.m_cap
    x = inputs.activations(8, h, seed=3).to(d)
    tw, ti = inputs.route_softmax_topk(inputs.router_logits(8, e, seed=3), topk)
    tw, ti = tw.to(d), ti.to(d)
    out = torch.empty(8, h, dtype=torch.bfloat16, device=d)
    moe.fused_experts_fp8(x, wd[0], wd[2], tw, ti, e, wd[1], wd[3], out=out)
    want = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        moe.fused_experts_fp8(x, wd[0], wd[2], tw, ti, e, wd[1], wd[3], out=out)
    xb = inputs.activations(3000, h, seed=4).to(d)                       # larger than anything before: the scratch grows
    twb, tib = inputs.route_softmax_topk(inputs.router_logits(3000, e, seed=4), topk)
    moe.fused_experts_fp8(xb, wd[0], wd[2], twb.to(d), tib.to(d), e, wd[1], wd[3])
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
