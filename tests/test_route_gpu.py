"""GPU parity of the routing kernel against kb-nano's TopKSoftmax (reference-generated fixture) and against the
oracle's restatement of GroupedTopK.  Expert ids must agree wherever the selection values are not tied to within
rounding; weights within 2e-6 relative (fp32 exp on the GPU and on the host differ in the last place)."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import golden

pytestmark = pytest.mark.gpu


def check(w, ids, w_ref, ids_ref, what, rtol=2e-6):
    w, ids, w_ref, ids_ref = w.cpu(), ids.cpu(), w_ref.cpu(), ids_ref.cpu()
    same = ids == ids_ref
    # a differing id is acceptable only for a (near-)tie: the weights at that position agree
    assert bool(torch.allclose(w[~same], w_ref[~same], rtol=1e-5, atol=1e-7)), f"{what}: ids differ beyond ties"
    assert float((~same).float().mean()) < 0.01, f"{what}: too many differing ids"
    assert bool(torch.allclose(w, w_ref, rtol=rtol, atol=1e-8)), f"{what}: weights, max diff {float((w - w_ref).abs().max())}"


def test_topk_softmax_golden(cuda_dev):
    from kb_nano_b200 import ops
    g = golden("routing")
    for name, k in (("8", 2), ("256", 8)):
        lg = torch.from_numpy(g["logits" + name]).to(cuda_dev)
        w, ids = ops.moe_route_topk(lg, k, "softmax", renormalize=True, renorm_floor=1e-20)
        check(w, ids, torch.from_numpy(g["w" + name]), torch.from_numpy(g["ids" + name]), f"TopKSoftmax golden E={name}")
    lg = torch.from_numpy(g["logits256"]).to(cuda_dev)
    w, ids = ops.moe_route_topk(lg, 8, "softmax", renormalize=False)
    check(w, ids, torch.from_numpy(g["w256_raw"]), torch.from_numpy(g["ids256_raw"]), "TopKSoftmax golden, raw weights")


def test_topk_softmax_candidate(cuda_dev):
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_topk_softmax", os.path.join(candidate_dir(), "L1", "topk_softmax.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    g = golden("routing")
    router = mod.TopKSoftmax()
    lg = torch.from_numpy(g["logits8"]).to(cuda_dev)
    w, ids = router(lg, 2, True)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    check(w, ids, torch.from_numpy(g["w8"]), torch.from_numpy(g["ids8"]), "TopKSoftmax candidate")
    w2, ids2 = router(lg.to(torch.bfloat16), 2, True)                  # bf16 logits are converted to fp32 first, as in the baseline
    rw, ri = to.route_topk(lg.to(torch.bfloat16).cpu(), 2, "softmax", renorm_floor=1e-20)
    check(w2, ids2, rw, ri, "TopKSoftmax candidate, bf16 logits")


@pytest.mark.parametrize("t,e,k,scoring,n_group,topk_group,use_bias,renorm,scale",
                         [(4096, 256, 8, "sigmoid", 1, 1, False, True, 1.0),       # BASELINE configs[2] routing
                          (16384, 8, 2, "softmax", 1, 1, False, True, 1.0),        # BASELINE configs[4] routing
                          (300, 256, 8, "sigmoid", 8, 4, True, True, 2.5),         # DeepSeek-V3: groups, bias, scaling
                          (77, 64, 6, "softmax", 8, 3, False, False, 1.0),         # groups smaller than a warp, max as group score
                          (5, 160, 6, "sigmoid", 5, 2, True, True, 1.0),
                          (1, 1000, 32, "softmax", 1, 1, False, True, 1.0)])
def test_route_vs_oracle(cuda_dev, t, e, k, scoring, n_group, topk_group, use_bias, renorm, scale):
    from kb_nano_b200 import inputs, ops
    lg = inputs.router_logits(t, e, seed=t + e)
    bias = 0.1 * torch.randn(e, generator=torch.Generator().manual_seed(e)) if use_bias else None
    rw, ri = to.route_topk(lg, k, scoring, bias, n_group, topk_group, renorm, 0.0, scale)
    w, ids = ops.moe_route_topk(lg.to(cuda_dev), k, scoring, bias=bias.to(cuda_dev) if use_bias else None, n_group=n_group,
                                topk_group=topk_group, renormalize=renorm, scale=scale)
    check(w, ids, rw, ri, f"route {scoring} E={e} k={k} groups={n_group}/{topk_group}")
    assert bool((ids.cpu() >= 0).all()) and bool((ids.cpu() < e).all())
    assert bool((torch.sort(ids.cpu(), dim=1).values.diff(dim=1) != 0).all()) if k > 1 else True     # no expert twice


def test_grouped_topk_candidate_bf16(cuda_dev):
    """The GroupedTopK drop-in class with bf16 gating output: scores and weights are rounded to bf16 step by step."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_grouped_topk", os.path.join(candidate_dir(), "L1", "grouped_topk.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    lg = inputs.router_logits(200, 256, seed=11).to(torch.bfloat16)
    bias = 0.05 * torch.randn(256, generator=torch.Generator().manual_seed(3))
    rw, ri = to.route_topk(lg, 8, "sigmoid", bias, 8, 4, True, 0.0, 2.5, score_in_input_dtype=True)
    w, ids = mod.GroupedTopK("sigmoid", True, 2.5)(lg.to(cuda_dev), bias.to(cuda_dev), 8, 4, 8)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    # bf16 scores tie often: compare the chosen sets through their weights, which are bf16-exact
    w, ids = w.cpu(), ids.cpu()
    same = ids == ri
    assert float(same.float().mean()) > 0.9
    assert bool(torch.allclose(torch.sort(w, dim=1).values, torch.sort(rw, dim=1).values, rtol=2e-2, atol=1e-6))
    with pytest.raises(ValueError):
        mod.GroupedTopK("tanh")


def test_grouped_topk_against_the_baselines_eager_branch(cuda_dev):
    """The routing kernel and the GroupedTopK drop-in against the fixture recorded from the baseline file's own eager
    branch (tasks/baseline/L1/grouped_topk.py:117-174): fp32 gating outputs with and without the selection bias."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, ops
    from tests.util import bf16_from_bits
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_grouped_topk_g", os.path.join(candidate_dir(), "L1", "grouped_topk.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    g = golden("grouped_topk")
    d = cuda_dev
    w, ids = mod.GroupedTopK("sigmoid", True, 2.5)(torch.from_numpy(g["a_logits"]).to(d), torch.from_numpy(g["a_bias"]).to(d), 8, 4, 8)
    check(w, ids, torch.from_numpy(g["a_w"]), torch.from_numpy(g["a_ids"]), "GroupedTopK fixture, sigmoid + bias + groups")
    w, ids = mod.GroupedTopK("softmax", False, 1.0)(torch.from_numpy(g["b_logits"]).to(d), None, 4, 2, 6)
    check(w, ids, torch.from_numpy(g["b_w"]), torch.from_numpy(g["b_ids"]), "GroupedTopK fixture, softmax, no bias")
    # bf16 gating output: scores tie often in bf16, so the chosen sets are compared through their sorted weights
    w, ids = mod.GroupedTopK("sigmoid", True, 1.0)(bf16_from_bits(g["c_logits"]).to(d), torch.from_numpy(g["c_bias"]).to(d), 4, 2, 8)
    rw, ri = torch.from_numpy(g["c_w"]), torch.from_numpy(g["c_ids"])
    assert float((ids.cpu() == ri).float().mean()) > 0.9
    assert bool(torch.allclose(torch.sort(w.cpu(), dim=1).values, torch.sort(rw, dim=1).values, rtol=2e-2, atol=1e-6))
