"""Size-independent properties of the MoE layers at the full sizes of BASELINE.json's configurations, where the CPU
oracle is too slow to run: exact linearity in the router weights, agreement of the fused and unfused activation,
agreement of the expert-parallel layer with the single-GPU pipeline, and a sampled-token check against the oracle."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close

pytestmark = pytest.mark.gpu


class _Experts:
    """Index-by-expert view that copies only the experts the oracle touches to the host."""

    def __init__(self, dev_tensor):
        self.t, self.cache = dev_tensor, {}

    def __getitem__(self, e):
        if e not in self.cache:
            self.cache[e] = self.t[e].cpu()
        return self.cache[e]


def _need(dev, gib):
    free, _ = torch.cuda.mem_get_info(dev)
    if free < gib * (1 << 30):
        pytest.skip(f"needs {gib} GiB of free device memory")


def test_config2_layer_properties(cuda_dev):
    """configs[2]: 4096 tokens, 256 experts, top-8, hidden 7168, intermediate 2048 (contiguous layout)."""
    from kb_nano_b200 import inputs, moe, ops
    _need(cuda_dev, 40)
    d = cuda_dev
    t, h, i, e, topk = 4096, 7168, 2048, 256, 8
    x = inputs.activations(t, h, seed=0, device=d)
    tw, ti = inputs.route_sigmoid_topk(inputs.router_logits(t, e, seed=0, device=d), topk)
    tw, ti = tw.contiguous(), ti.contiguous()
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=1, device=d)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=2, device=d)
    out = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s).clone()
    assert ops.gemm_status(d) == 0 and bool(torch.isfinite(out.float()).all())
    # router weights times a power of two: every product and partial sum scales exactly, so do the bf16 results
    out2 = moe.fused_experts_fp8(x, w13_q, w2_q, tw * 2.0, ti, e, w13_s, w2_s).clone()
    assert torch.equal((out.float() * 2.0).to(torch.bfloat16).view(torch.int16), out2.view(torch.int16))
    # activation inside GEMM1's epilogue or as a kernel of its own: same bits
    out3 = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s, fuse_activation=False).clone()
    assert torch.equal(out.view(torch.int16), out3.view(torch.int16))
    # the same tokens in another order give the same rows
    perm = torch.randperm(t, device=d, generator=torch.Generator(device=d).manual_seed(1))
    out4 = moe.fused_experts_fp8(x[perm].contiguous(), w13_q, w2_q, tw[perm].contiguous(), ti[perm].contiguous(), e, w13_s, w2_s)
    assert torch.equal(out[perm].view(torch.int16), out4.view(torch.int16))
    # a sample of tokens against the CPU oracle (only the experts those tokens use are dequantised)
    pick = torch.tensor([0, 1, 777, 4095])
    used = sorted(set(ti[pick.to(d)].reshape(-1).tolist()))
    ref = to.moe_layer(x[pick.to(d)].cpu(), _Experts(w13_q), _Experts(w13_s), _Experts(w2_q), _Experts(w2_s), tw[pick.to(d)].cpu(),
                       ti[pick.to(d)].cpu(), experts=used)
    assert_gemm_close(out[pick.to(d)].cpu(), ref, "configs[2], sampled tokens")


def test_config3_expert_parallel_equals_single_gpu(cuda_dev):
    """configs[3] on one rank: 128 tokens, masked layout with 256 local experts, against the contiguous pipeline."""
    from kb_nano_b200 import ep, inputs, moe, ops
    _need(cuda_dev, 40)
    d = cuda_dev
    t, h, i, e, topk = 128, 7168, 2048, 256, 8
    x = inputs.activations(t, h, seed=0, device=d)
    tw, ti = inputs.route_sigmoid_topk(inputs.router_logits(t, e, seed=0, device=d), topk)
    tw, ti = tw.contiguous(), ti.contiguous()
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=1, device=d)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=2, device=d)
    layer = ep.EpMoe(0, 1, e, h, i, max_tokens=t, topk=topk, max_m=256, device=d)
    out = layer.forward(x, ti, tw, w13_q, w13_s, w2_q, w2_s).clone()
    layer.check()
    layer.close()
    single = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s)
    assert ops.gemm_status(d) == 0
    assert torch.equal(out.view(torch.int16), single.view(torch.int16))


def test_config4_layer_properties(cuda_dev):
    """configs[4]: 16384 tokens, 8 experts, top-2 softmax, hidden 4096, intermediate 14336."""
    from kb_nano_b200 import inputs, moe, ops
    _need(cuda_dev, 24)
    d = cuda_dev
    t, h, i, e, topk = 16384, 4096, 14336, 8, 2
    x = inputs.activations(t, h, seed=0, device=d)
    tw, ti = inputs.route_softmax_topk(inputs.router_logits(t, e, seed=0, device=d), topk)
    tw, ti = tw.contiguous(), ti.contiguous()
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=1, device=d)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=2, device=d)
    out = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s).clone()
    assert ops.gemm_status(d) == 0 and bool(torch.isfinite(out.float()).all())
    out2 = moe.fused_experts_fp8(x, w13_q, w2_q, tw * 0.5, ti, e, w13_s, w2_s).clone()
    assert torch.equal((out.float() * 0.5).to(torch.bfloat16).view(torch.int16), out2.view(torch.int16))
    out3 = moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s, fuse_activation=False)
    assert torch.equal(out.view(torch.int16), out3.view(torch.int16))
    pick = torch.tensor([3, 16383])
    ref = to.moe_layer(x[pick.to(d)].cpu(), _Experts(w13_q), _Experts(w13_s), _Experts(w2_q), _Experts(w2_s), tw[pick.to(d)].cpu(),
                       ti[pick.to(d)].cpu(), experts=sorted(set(ti[pick.to(d)].reshape(-1).tolist())))
    assert_gemm_close(out[pick.to(d)].cpu(), ref, "configs[4], sampled tokens")
