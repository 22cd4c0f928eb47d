"""Pins both editions of the CPU oracle (C and torch) to fixtures produced by kb-nano's own Python
reference (tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import torch

from oracle import c_oracle as co
from oracle import torch_oracle as to
from tests.util import (assert_gemm_close, assert_quant_equal, bf16_from_bits, bits16, fp8_from_bits, golden)


def test_quant_1x128_matches_reference():
    g = golden("quant_1x128")
    q, s = co.quant_1x128(g["x"])
    assert_quant_equal(q, s, g["q"], g["s"], "C oracle")
    qt, st = to.quant_1x128(bf16_from_bits(g["x"]))
    assert_quant_equal(qt, st, g["q"], g["s"], "torch oracle")
    # column-major scale layout holds the same values
    q2, s2 = co.quant_1x128(g["x"], colmajor=True)
    assert s2.strides == (4, 4 * g["x"].shape[0])
    assert_quant_equal(q2, np.ascontiguousarray(s2), g["q"], g["s"], "C oracle, col-major")


def test_quant_ragged_k_matches_reference():
    g = golden("quant_1x128")
    q, s = co.quant_1x128(g["x_ragged"])
    assert_quant_equal(q, s, g["q_ragged"], g["s_ragged"], "C oracle ragged K")
    qt, st = to.quant_1x128(bf16_from_bits(g["x_ragged"]))
    assert_quant_equal(qt, st, g["q_ragged"], g["s_ragged"], "torch oracle ragged K")


def test_scale_is_power_of_two_and_zero_group_scale():
    g = golden("quant_1x128")
    s = g["s"]
    assert ((s.view(np.uint32) & 0x7FFFFF) == 0).all()
    assert (s[0] == 2.0 ** -42).all()          # all-zero row: 2^ceil(log2(1e-10/448))
    assert s[1, 0] == 2.0 ** -7                 # absmax 3.5 -> exactly 2^-7
    assert s[9, 0] == 2.0 ** -6 and s[10, 0] == 2.0 ** -7   # just above / below a 1.75 mantissa


def test_silu_table_matches_reference_for_every_gate():
    ref = golden("silu_table")["table"]
    gates = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    finite = torch.isfinite(gates).numpy()
    tab = co.silu_bf16_table()
    assert int(((tab != ref) & finite).sum()) == 0
    t2 = bits16(to.silu_mul_bf16(torch.stack([gates, torch.ones_like(gates)], 1))).ravel()
    assert int(((t2 != ref) & finite).sum()) == 0


def test_silu_mul_quant_matches_reference():
    g = golden("silu_mul_quant")
    q, s = co.silu_mul_quant_1x128(g["x"])
    assert_quant_equal(q, np.ascontiguousarray(s), g["q"], g["s"], "C oracle")
    qt, st = to.silu_mul_quant_1x128(bf16_from_bits(g["x"]))
    assert_quant_equal(qt, st, g["q"], g["s"], "torch oracle")
    assert (bits16(to.silu_mul_bf16(bf16_from_bits(g["x"]))) == g["y"]).all()


def test_block_quant_matches_reference():
    g = golden("block_quant")
    for e in range(g["w"].shape[0]):
        q, s = co.block_quant_128x128(g["w"][e])
        assert_quant_equal(q, s, g["q"][e], g["s"][e], f"C oracle expert {e}")
    qt, st = to.block_quant_128x128(bf16_from_bits(g["w"]))
    assert_quant_equal(qt, st, g["q"], g["s"], "torch oracle")
    q, s = co.block_quant_128x128(g["w_ragged"])
    assert_quant_equal(q, s, g["q_ragged"], g["s_ragged"], "C oracle ragged")
    # the harness's own activation quantiser agrees with the L1 reference one
    a = golden("quant_1x128")
    assert (g["act_q"] == a["q"]).all() and (g["act_s"] == a["s"]).all()


def test_package_input_quantiser_matches_reference():
    from kb_nano_b200 import inputs
    g = golden("block_quant")
    q, s = inputs.block_quant_128x128(bf16_from_bits(g["w"]))
    assert_quant_equal(q, s, g["q"], g["s"], "kb_nano_b200.inputs.block_quant_128x128")


def test_dense_gemm_matches_reference():
    g = golden("fp8_linear")
    ref = bf16_from_bits(g["c"])
    c = co.gemm_nt_dequant(g["a_q"], g["a_s"], g["w_q"], g["w_s"])
    assert_gemm_close(bf16_from_bits(c), ref, "C oracle")
    ct = to.gemm_nt_dequant(fp8_from_bits(g["a_q"]), torch.from_numpy(g["a_s"]), fp8_from_bits(g["w_q"]), torch.from_numpy(g["w_s"]))
    assert (bits16(ct) == g["c"]).mean() > 0.999      # same torch ops: identical up to matmul blocking
    assert_gemm_close(ct, ref, "torch oracle")
    # whole layer from bf16 input: quant + gemm
    out = to.fp8_linear(bf16_from_bits(g["a"]), fp8_from_bits(g["w_q"]), torch.from_numpy(g["w_s"]))
    assert_gemm_close(out, ref, "torch oracle fp8_linear")


def test_grouped_gemm_matches_reference():
    g = golden("grouped_gemm")
    topk_ids = g["topk_ids"]
    t, k = topk_ids.shape
    # reference output row r = (token r//k, slot r%k); same rows through the per-row-expert form
    a_rows = np.repeat(g["a_q"], k, axis=0)
    s_rows = np.repeat(g["a_s"], k, axis=0)
    row_expert = topk_ids.reshape(-1).astype(np.int32)
    ref = bf16_from_bits(g["c"])
    c = co.grouped_gemm_nt(a_rows, s_rows, g["b_q"], g["b_s"], row_expert)
    assert_gemm_close(bf16_from_bits(c), ref, "C oracle")
    ct = to.grouped_gemm_contig(fp8_from_bits(a_rows), torch.from_numpy(s_rows), fp8_from_bits(g["b_q"]),
                                torch.from_numpy(g["b_s"]), torch.from_numpy(row_expert))
    assert_gemm_close(ct, ref, "torch oracle")
    # -1 rows stay untouched
    re2 = row_expert.copy()
    re2[::5] = -1
    init = np.full(g["c"].shape, 0x7FC0, np.uint16)
    c2 = co.grouped_gemm_nt(a_rows, s_rows, g["b_q"], g["b_s"], re2, c_init=init)
    assert (c2[::5] == 0x7FC0).all() and (c2[1::5] == c[1::5]).all()


def test_masked_layout_oracle_agrees_with_contiguous():
    g = golden("grouped_gemm")
    e = g["b_q"].shape[0]
    topk_ids = g["topk_ids"]
    t, k = topk_ids.shape
    max_m = 32
    a_q = torch.zeros(e, max_m, g["a_q"].shape[1], dtype=torch.uint8)
    a_s = torch.ones(e, max_m, g["a_s"].shape[1])
    masked = torch.zeros(e, dtype=torch.int32)
    where = {}
    for r in range(t * k):
        ex = int(topk_ids.reshape(-1)[r])
        where[r] = (ex, int(masked[ex]))
        a_q[ex, masked[ex]] = torch.from_numpy(g["a_q"][r // k])
        a_s[ex, masked[ex]] = torch.from_numpy(g["a_s"][r // k])
        masked[ex] += 1
    out = to.grouped_gemm_masked(a_q.view(torch.float8_e4m3fn), a_s, fp8_from_bits(g["b_q"]), torch.from_numpy(g["b_s"]), masked)
    ref = bf16_from_bits(g["c"])
    got = torch.stack([out[where[r][0], where[r][1]] for r in range(t * k)])
    assert_gemm_close(got, ref, "masked oracle")


def test_moe_layer_matches_reference():
    g = golden("fused_experts")
    out = to.moe_layer(bf16_from_bits(g["x"]), fp8_from_bits(g["w13_q"]), torch.from_numpy(g["w13_s"]),
                       fp8_from_bits(g["w2_q"]), torch.from_numpy(g["w2_s"]), torch.from_numpy(g["topk_w"]),
                       torch.from_numpy(g["topk_ids"]))
    assert_gemm_close(out, bf16_from_bits(g["out"]), "torch oracle moe_layer")


def test_routing_oracles():
    torch.manual_seed(1)
    logits = torch.randn(32, 16)
    w, ids = to.route_sigmoid_topk(logits, 4)
    assert ids.dtype == torch.int32 and torch.allclose(w.sum(-1), torch.ones(32))
    assert (torch.sigmoid(logits).gather(1, ids.long()) >= torch.sigmoid(logits).topk(4).values[:, -1:]).all()
    w2, ids2 = to.route_softmax_topk(logits, 2)
    assert torch.allclose(w2.sum(-1), torch.ones(32)) and (ids2[:, 0] == logits.argmax(-1)).all()


def test_routing_oracle_matches_reference_fixture():
    """The oracle's routing restatement reproduces kb-nano's TopKSoftmax bit for bit on CPU."""
    g = golden("routing")
    for name, k in (("8", 2), ("256", 8)):
        w, ids = to.route_topk(torch.from_numpy(g["logits" + name]), k, "softmax", renorm_floor=1e-20)
        assert (ids.numpy() == g["ids" + name]).all()
        assert (w.numpy() == g["w" + name]).all()
    w, ids = to.route_topk(torch.from_numpy(g["logits256"]), 8, "softmax", renormalize=False)
    assert (ids.numpy() == g["ids256_raw"]).all() and (w.numpy() == g["w256_raw"]).all()
    # group-limited selection keeps only experts of the best groups
    lg = torch.randn(16, 64, generator=torch.Generator().manual_seed(1))
    w, ids = to.route_topk(lg, 4, "sigmoid", None, 8, 2, True)
    assert all(len(set((ids[r] // 8).tolist())) <= 2 for r in range(16))
    assert torch.allclose(w.sum(dim=1), torch.ones(16))


def test_grouped_topk_oracle_matches_the_baselines_eager_branch():
    """GroupedTopK has no reference/ edition in kb-nano: the fixture holds the output of the baseline file's own
    eager branch (tasks/baseline/L1/grouped_topk.py:117-174, run on CPU by tests/golden/make_golden.py) and the
    oracle's restatement reproduces it bit for bit: ids and fp32 weights, with and without the selection bias,
    fp32 and bf16 gating outputs."""
    g = golden("grouped_topk")
    w, ids = to.route_topk(torch.from_numpy(g["a_logits"]), 8, "sigmoid", bias=torch.from_numpy(g["a_bias"]), n_group=8, topk_group=4,
                           renormalize=True, scale=2.5, score_in_input_dtype=True)
    assert (ids.numpy() == g["a_ids"]).all() and (w.numpy().view(np.uint32) == g["a_w"].view(np.uint32)).all()
    w, ids = to.route_topk(torch.from_numpy(g["b_logits"]), 6, "softmax", n_group=4, topk_group=2, renormalize=False, score_in_input_dtype=True)
    assert (ids.numpy() == g["b_ids"]).all() and (w.numpy().view(np.uint32) == g["b_w"].view(np.uint32)).all()
    w, ids = to.route_topk(bf16_from_bits(g["c_logits"]), 8, "sigmoid", bias=torch.from_numpy(g["c_bias"]), n_group=4, topk_group=2,
                           renormalize=True, score_in_input_dtype=True)
    assert (ids.numpy() == g["c_ids"]).all() and (w.numpy().view(np.uint32) == g["c_w"].view(np.uint32)).all()
