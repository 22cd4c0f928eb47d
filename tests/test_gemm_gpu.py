"""GPU parity, through the C ABI, of the block-scaled FP8 GEMMs against the oracle's
dequantise-then-fp32-matmul: max relative error 1e-2 (|d| <= 1e-2 + 1e-2*|ref|), cosine > 0.9999."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close, bf16_from_bits, fp8_from_bits, golden

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def make_dense(m, n, k, seed, dev, arbitrary_scales=False):
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(m, k, seed=seed)
    a_q, a_s = to.quant_1x128(x)
    w_q, w_s = inputs.weight(((n + 127) // 128) * 128, ((k + 127) // 128) * 128, seed=seed + 1)
    w_q = w_q[:n, :k].contiguous()
    if arbitrary_scales:
        w_s = w_s * (1.0 + 0.37 * torch.rand(w_s.shape, generator=torch.Generator().manual_seed(seed)))
    return a_q, a_s, w_q, w_s


def run_dense(a_q, a_s, w_q, w_s, dev, colmajor=True):
    from kb_nano_b200 import ops
    m, n = a_q.shape[0], w_q.shape[0]
    sa = a_s.to(dev)
    if colmajor:
        sa = sa.t().contiguous().t()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.fp8_gemm_nt(a_q.to(dev), sa, w_q.to(dev), w_s.to(dev), out)
    assert ops.gemm_status(dev) == 0
    return out.cpu()


def test_dense_golden(cuda_dev):
    g = golden("fp8_linear")
    out = run_dense(fp8_from_bits(g["a_q"]), torch.from_numpy(g["a_s"]), fp8_from_bits(g["w_q"]), torch.from_numpy(g["w_s"]), cuda_dev)
    assert_gemm_close(out, bf16_from_bits(g["c"]), "golden fp8_linear")


@pytest.mark.parametrize("m,n,k", [(1, 4096, 7168), (5, 1000, 400), (8, 256, 512), (9, 2304, 4096), (16, 7168, 2048), (13, 24, 144)])
@pytest.mark.parametrize("arbitrary", [False, True])
def test_dense_decode_sizes(cuda_dev, m, n, k, arbitrary):
    """M <= 16 takes the weight-streaming kernel (tokens as the N dimension of mma.sync, any fp32 scales): ragged N
    and K, one to sixteen tokens, row- and column-major activation scales; two runs agree bit for bit."""
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m * 7 + n + k, dev=cuda_dev, arbitrary_scales=arbitrary)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    outs = [run_dense(a_q, a_s, w_q, w_s, cuda_dev, colmajor=cm) for cm in (True, False, True)]
    assert_gemm_close(outs[0], ref, f"decode-size dense {m}x{n}x{k}")
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (1, 256, 512), (127, 384, 1024), (129, 128, 256), (300, 640, 7168), (64, 2304, 4096)])
def test_dense_shapes(cuda_dev, m, n, k):
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m + n + k, dev=cuda_dev)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    for cm in (True, False):
        assert_gemm_close(run_dense(a_q, a_s, w_q, w_s, cuda_dev, colmajor=cm), ref, f"dense {m}x{n}x{k} colmajor={cm}")


def test_dense_ragged_n_and_k(cuda_dev):
    a_q, a_s, w_q, w_s = make_dense(70, 200, 400, seed=5, dev=cuda_dev)     # N%128 != 0, K%128 != 0 (K%16 == 0)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    assert_gemm_close(run_dense(a_q, a_s, w_q, w_s, cuda_dev), ref, "ragged N,K")


def test_dense_arbitrary_fp32_weight_scales(cuda_dev):
    a_q, a_s, w_q, w_s = make_dense(256, 512, 2048, seed=8, dev=cuda_dev, arbitrary_scales=True)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    assert_gemm_close(run_dense(a_q, a_s, w_q, w_s, cuda_dev), ref, "non-power-of-two weight scales")


def test_dense_config1(cuda_dev):
    """Dense-linear configuration: M=512, K=7168, N=4096 through the Fp8Linear drop-in class."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_fp8_linear", os.path.join(candidate_dir(), "L1", "fp8_linear.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    x = inputs.activations(512, 7168, seed=0)
    w_q, w_s = inputs.weight(4096, 7168, seed=1)
    lin = mod.Fp8Linear()
    out = lin(x.to(cuda_dev).view(4, 128, 7168), w_q.to(cuda_dev), w_s.to(cuda_dev))
    assert out.shape == (4, 128, 4096) and out.dtype == torch.bfloat16
    ref = to.fp8_linear(x, w_q, w_s)
    assert_gemm_close(out.cpu().view(512, 4096), ref, "C1 Fp8Linear")
    bias = torch.randn(4096, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    out_b = lin(x.to(cuda_dev), w_q.to(cuda_dev), w_s.to(cuda_dev), bias.to(cuda_dev))
    # the bias is added in the GEMM's epilogue, in fp32 before the one rounding to bf16: the reference's
    # F.linear(x, w, bias) (tasks/reference/L1/fp8_linear.py:103); kb-nano's baseline class rounds first and adds in
    # bf16 (tasks/baseline/L1/fp8_linear.py:446-447), which the same tolerance covers
    assert_gemm_close(out_b.cpu(), to.fp8_linear(x, w_q, w_s, bias), "C1 Fp8Linear + bias")
    # against rounding first: the two differ by the rounding of the bias-free result, i.e. by at most half a bf16 ulp of
    # THAT value, which a tolerance relative to the sum does not cover where result and bias cancel
    plain = out.cpu().view(512, 4096).float()
    d = (out_b.cpu().float() - (plain + bias.float())).abs()
    assert bool((d <= 2.0 ** -7 * torch.maximum(plain.abs(), (plain + bias.float()).abs()) + 1e-6).all())


def make_grouped(e, n, k, counts, seed):
    """Expert-contiguous rows with 128-aligned segments; returns tensors on CPU."""
    from kb_nano_b200 import inputs
    b_q, b_s = inputs.expert_weights(e, n, k, seed=seed)
    starts, total = [], 0
    for c in counts:
        starts.append(total)
        total += ((c + 127) // 128) * 128
    total += 128                                   # one all-padding block at the end
    x = inputs.activations(total, k, seed=seed + 3)
    a_q, a_s = to.quant_1x128(x)
    row_expert = torch.full((total,), -1, dtype=torch.int32)
    for i, c in enumerate(counts):
        row_expert[starts[i]:starts[i] + c] = i
    return a_q, a_s, b_q, b_s, row_expert


@pytest.mark.parametrize("counts", [[128, 256], [1, 0, 127, 129], [300, 5, 0, 0, 77, 128, 1, 640]])
def test_grouped_contiguous(cuda_dev, counts):
    from kb_nano_b200 import ops
    e, n, k = len(counts), 512, 1024
    a_q, a_s, b_q, b_s, row_expert = make_grouped(e, n, k, counts, seed=sum(counts))
    ref = to.grouped_gemm_contig(a_q, a_s, b_q, b_s, row_expert)
    for cm in (False, True):
        sa = a_s.to(cuda_dev)
        if cm:
            sa = sa.t().contiguous().t()
        out = torch.full((a_q.shape[0], n), 7.0, dtype=torch.bfloat16, device=cuda_dev)
        ops.m_grouped_fp8_gemm_nt_contiguous(a_q.to(cuda_dev), sa, b_q.to(cuda_dev), b_s.to(cuda_dev), out, row_expert.to(cuda_dev))
        assert ops.gemm_status(cuda_dev) == 0
        out = out.cpu()
        valid = row_expert >= 0
        assert_gemm_close(out[valid], ref[valid], f"contiguous {counts} colmajor={cm}")
        assert bool((out[~valid] == 7.0).all()), "padding rows must not be written"


def test_grouped_contiguous_golden(cuda_dev):
    """The reference MoeGroupedGemm result, rows regrouped into the expert-contiguous layout."""
    from kb_nano_b200 import ops
    g = golden("grouped_gemm")
    ids = torch.from_numpy(g["topk_ids"]).reshape(-1)
    tk = g["topk_ids"].shape[1]
    e = g["b_q"].shape[0]
    order = torch.argsort(ids, stable=True)
    rows, row_expert, src = [], [], []
    for ex in range(e):
        sel = order[ids[order] == ex]
        pad = (-len(sel)) % 128
        rows += sel.tolist() + [0] * pad
        row_expert += [ex] * len(sel) + [-1] * pad
        src += sel.tolist() + [-1] * pad
    rows = torch.tensor(rows)
    a_q = fp8_from_bits(g["a_q"])[rows // tk].contiguous()
    a_s = torch.from_numpy(g["a_s"])[rows // tk].contiguous()
    out = torch.zeros(len(rows), g["b_q"].shape[1], dtype=torch.bfloat16, device=cuda_dev)
    ops.m_grouped_fp8_gemm_nt_contiguous(a_q.to(cuda_dev), a_s.to(cuda_dev), fp8_from_bits(g["b_q"]).to(cuda_dev),
                                         torch.from_numpy(g["b_s"]).to(cuda_dev), out, torch.tensor(row_expert, dtype=torch.int32, device=cuda_dev))
    out = out.cpu()
    src = torch.tensor(src)
    got = torch.zeros_like(bf16_from_bits(g["c"]))
    got[src[src >= 0]] = out[src >= 0]
    assert_gemm_close(got, bf16_from_bits(g["c"]), "golden grouped gemm")


@pytest.mark.parametrize("masked", [[0, 1, 128, 129, 256, 77], [256] * 4, [0] * 3, [5, 200]])
def test_grouped_masked(cuda_dev, masked):
    from kb_nano_b200 import inputs, ops
    e, max_m, n, k = len(masked), 256, 384, 512
    b_q, b_s = inputs.expert_weights(e, n, k, seed=len(masked))
    x = inputs.activations(e * max_m, k, seed=17)
    a_q, a_s = to.quant_1x128(x)
    a_q, a_s = a_q.view(e, max_m, k), a_s.view(e, max_m, k // 128)
    mm = torch.tensor(masked, dtype=torch.int32)
    ref = to.grouped_gemm_masked(a_q, a_s, b_q, b_s, mm)
    out = torch.full((e, max_m, n), 7.0, dtype=torch.bfloat16, device=cuda_dev)
    ops.m_grouped_fp8_gemm_nt_masked(a_q.to(cuda_dev), a_s.to(cuda_dev), b_q.to(cuda_dev), b_s.to(cuda_dev), out, mm.to(cuda_dev))
    assert ops.gemm_status(cuda_dev) == 0
    out = out.cpu()
    for i, c in enumerate(masked):
        if c:
            assert_gemm_close(out[i, :c], ref[i, :c], f"masked expert {i} rows {c}")
        assert bool((out[i, c:] == 7.0).all()), "rows beyond masked_m must not be written"


def test_gemm_linearity_at_full_size(cuda_dev):
    """Size-independent property on the dense configuration's shape: doubling every activation scale
    doubles the output exactly (powers of two commute with every rounding step)."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(512, 7168, seed=0, device=cuda_dev)
    w_q, w_s = inputs.weight(4096, 7168, seed=1, device=cuda_dev)
    a_q = torch.empty(512, 7168, dtype=FP8, device=cuda_dev)
    a_s = torch.empty(56, 512, device=cuda_dev).t()
    ops.per_token_group_quant_fp8(x, a_q, a_s)
    o1 = torch.empty(512, 4096, dtype=torch.bfloat16, device=cuda_dev)
    o2 = torch.empty_like(o1)
    ops.fp8_gemm_nt(a_q, a_s, w_q, w_s, o1)
    ops.fp8_gemm_nt(a_q, (a_s * 2.0).t().contiguous().t(), w_q, w_s, o2)
    assert ops.gemm_status(cuda_dev) == 0
    assert bool((o2.float() == 2.0 * o1.float()).all())
    # and repeated launches are bit-identical (fixed summation order)
    o3 = torch.empty_like(o1)
    ops.fp8_gemm_nt(a_q, a_s, w_q, w_s, o3)
    assert bool((o3.view(torch.int16) == o1.view(torch.int16)).all())


@pytest.mark.parametrize("m,n,k,arbitrary,what", [
    (512, 512, 1024, False, "block-scaled kernel, 256-wide tiles"),
    (64, 4096, 7168, False, "cluster split-K kernel"),
    (200, 392, 400, False, "block-scaled kernel, ragged N and K"),
    (256, 512, 2048, True, "fp32-scale kernel"),
    (5, 1000, 400, True, "weight-streaming kernel, M <= 16"),
])
def test_dense_bias_in_the_epilogue(cuda_dev, m, n, k, arbitrary, what):
    """bias rides in the GEMM: added to the fp32 accumulator before the one rounding to bf16, which is the reference's
    F.linear(x, w, bias) (tasks/reference/L1/fp8_linear.py:103) -- checked for every dense kernel, through
    ops.fp8_gemm_nt_auto (power-of-two scales take the block-scaled kernels) and the Fp8Linear drop-in."""
    from kb_nano_b200 import ops
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m + n, dev=cuda_dev, arbitrary_scales=arbitrary)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s, bias)
    d = cuda_dev
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=d)
    ops.fp8_gemm_nt_auto(a_q.to(d), a_s.to(d), w_q.to(d), w_s.to(d), out, bias.to(d))
    assert ops.gemm_status(d) == 0
    assert_gemm_close(out.cpu(), ref, what)
    # without a bias the same call gives the plain product: the bias is not sticky
    out0 = torch.empty_like(out)
    ops.fp8_gemm_nt_auto(a_q.to(d), a_s.to(d), w_q.to(d), w_s.to(d), out0)
    assert_gemm_close(out0.cpu(), to.gemm_nt_dequant(a_q, a_s, w_q, w_s), what + ", no bias")
    with pytest.raises(ValueError):
        ops.fp8_gemm_nt_auto(a_q.to(d), a_s.to(d), w_q.to(d), w_s.to(d), out, bias.float().to(d))


def test_fp8_linear_candidate_bias(cuda_dev):
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_fp8_linear_b", os.path.join(candidate_dir(), "L1", "fp8_linear.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    m, n, k = 96, 512, 1024
    x = inputs.activations(m, k, seed=2)
    w_q, w_s = inputs.weight(n, k, seed=3)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(5))).to(torch.bfloat16)
    d = cuda_dev
    lin = mod.Fp8Linear()
    got = lin(x.to(d), w_q.to(d), w_s.to(d), bias.to(d))
    assert_gemm_close(got.cpu(), to.fp8_linear(x, w_q, w_s, bias), "Fp8Linear with bias")
    got32 = lin(x.to(d), w_q.to(d), w_s.to(d), bias.float().to(d))      # a bias the kernel does not take: added by torch, as the baseline does
    assert got32.dtype == torch.float32 or got32.dtype == torch.bfloat16
