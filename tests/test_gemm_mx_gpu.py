"""GPU parity of the UE8M0 block-scaled GEMM path (scales packed and applied by the tensor core) against
the same oracle and tolerance as the fp32-scale kernels, and against the fp32-scale kernels themselves."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_gemm_close, bf16_from_bits, fp8_from_bits, golden
from tests.test_gemm_gpu import make_dense, make_grouped

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def run_dense_mx(a_q, a_s, w_q, w_s, dev):
    from kb_nano_b200 import ops
    m, k = a_q.shape
    n = w_q.shape[0]
    sfb = ops.packed_weight_scales(w_s.to(dev), n, k)
    assert sfb is not None
    sfa = ops.pack_sf_rows(a_s.to(dev), k)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.fp8_gemm_nt_ue8m0(a_q.to(dev), sfa, w_q.to(dev), sfb, out)
    assert ops.gemm_status(dev) == 0
    return out.cpu()


def test_mx_dense_golden(cuda_dev):
    g = golden("fp8_linear")
    out = run_dense_mx(fp8_from_bits(g["a_q"]), torch.from_numpy(g["a_s"]), fp8_from_bits(g["w_q"]), torch.from_numpy(g["w_s"]), cuda_dev)
    assert_gemm_close(out, bf16_from_bits(g["c"]), "golden fp8_linear (ue8m0 path)")


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (1, 256, 512), (127, 384, 1024), (129, 128, 256), (300, 640, 7168), (64, 2304, 4096), (70, 200, 400)])
def test_mx_dense_shapes(cuda_dev, m, n, k):
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m + n + k, dev=cuda_dev)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    assert_gemm_close(run_dense_mx(a_q, a_s, w_q, w_s, cuda_dev), ref, f"dense ue8m0 {m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(1, 4096, 7168), (16, 4096, 7168), (33, 7168, 2048), (100, 1000, 1040), (128, 128, 1024), (96, 384, 2048),
                                   (200, 512, 4096)])
def test_mx_dense_few_tiles_split_k(cuda_dev, m, n, k):
    """Decode-sized problems: K is split over a thread-block cluster and the partial tiles are summed through
    distributed shared memory (splits of 8, 8, 4, 2, 4, 8, 8 CTAs here; ragged N and K in the fourth case).
    Two runs must agree bit for bit (the partials are added in a fixed order)."""
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m + n + k, dev=cuda_dev)
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    out1 = run_dense_mx(a_q, a_s, w_q, w_s, cuda_dev)
    assert_gemm_close(out1, ref, f"dense ue8m0 split-K {m}x{n}x{k}")
    out2 = run_dense_mx(a_q, a_s, w_q, w_s, cuda_dev)
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))


@pytest.mark.parametrize("m,n,k,bias", [(512, 4096, 7168, False), (512, 2048, 2048, True), (300, 3000, 2048, True), (256, 4096, 1024, False),
                                        (384, 2304, 4096, True), (129, 4096, 1024, False)])
def test_mx_dense_cta_pairs(cuda_dev, m, n, k, bias):
    """A few hundred rows and too few 256 x 256 tiles for every SM: two CTAs share a tile (one tensor-core instruction
    over both SMs) and 2 or 4 pairs of a cluster split K (2 slices in the first and third case, 4 in the second and
    fourth; ragged rows and columns, a second row block of one row in the last case).  The partials are added in slice order: two runs agree bit for bit."""
    from kb_nano_b200 import ops
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=m + n + k, dev=cuda_dev)
    b = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16) if bias else None
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s, b)
    sfb = ops.packed_weight_scales(w_s.to(cuda_dev), n, k)
    sfa = ops.pack_sf_rows(a_s.to(cuda_dev), k)
    outs = []
    for _ in range(2):
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        ops.fp8_gemm_nt_ue8m0(a_q.to(cuda_dev), sfa, w_q.to(cuda_dev), sfb, out, b.to(cuda_dev) if bias else None)
        assert ops.gemm_status(cuda_dev) == 0
        outs.append(out.cpu())
    assert_gemm_close(outs[0], ref, f"dense ue8m0 CTA pairs {m}x{n}x{k}")
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_mx_scales_with_wide_exponent_range(cuda_dev):
    """Each K-block and each row with a different power-of-two scale: catches any mix-up of the packed order."""
    m, n, k = 256, 512, 1024
    a_q, a_s, w_q, w_s = make_dense(m, n, k, seed=77, dev=cuda_dev)
    gen = torch.Generator().manual_seed(5)
    a_s = torch.pow(2.0, torch.randint(-12, 4, a_s.shape, generator=gen).float())
    w_s = torch.pow(2.0, torch.randint(-9, 3, w_s.shape, generator=gen).float())
    ref = to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    got = run_dense_mx(a_q, a_s, w_q, w_s, cuda_dev)
    g, r = got.float(), ref.float()
    # values span many octaves: compare relative to each row's own magnitude
    scale = r.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    assert float(((g - r).abs() / scale).max()) < 1e-2
    assert float(torch.nn.functional.cosine_similarity(g.flatten().double(), r.flatten().double(), dim=0)) > 0.9999


def test_non_pow2_weight_scales_are_detected(cuda_dev):
    from kb_nano_b200 import ops
    w_s = torch.tensor([[0.5, 0.25], [0.75, 1.0]], device=cuda_dev)
    assert ops.packed_weight_scales(w_s, 256, 256) is None
    assert ops.packed_weight_scales(torch.tensor([[0.5, 0.25], [2.0, 1.0]], device=cuda_dev), 256, 256) is not None


@pytest.mark.parametrize("counts", [[128, 256], [1, 0, 127, 129], [300, 5, 0, 0, 77, 128, 1, 640]])
def test_mx_grouped_contiguous(cuda_dev, counts):
    from kb_nano_b200 import ops
    e, n, k = len(counts), 512, 1024
    a_q, a_s, b_q, b_s, row_expert = make_grouped(e, n, k, counts, seed=sum(counts))
    ref = to.grouped_gemm_contig(a_q, a_s, b_q, b_s, row_expert)
    d = cuda_dev
    out = torch.full((a_q.shape[0], n), 7.0, dtype=torch.bfloat16, device=d)
    ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(a_q.to(d), ops.pack_sf_rows(a_s.to(d), k), b_q.to(d), ops.packed_weight_scales(b_s.to(d), n, k),
                                               out, row_expert.to(d))
    assert ops.gemm_status(d) == 0
    out = out.cpu()
    valid = row_expert >= 0
    assert_gemm_close(out[valid], ref[valid], f"contiguous ue8m0 {counts}")
    assert bool((out[~valid] == 7.0).all())


# 64 experts x 4 column tiles: every CTA walks several tiles whose row blocks alternate between at most 64 and more than
# 64 live rows (the kernel cuts its shared-memory ring differently for the two), with fewer K blocks than ring slots
MIXED = [3, 100, 70, 64, 65, 256, 0, 31, 129, 16, 200, 1, 128, 33, 90, 7] * 4


@pytest.mark.parametrize("masked,n", [([0, 1, 128, 129, 256, 77], 384), ([256] * 4, 384), ([0] * 3, 384), ([5, 200], 384), (MIXED, 1024)])
def test_mx_grouped_masked(cuda_dev, masked, n):
    from kb_nano_b200 import inputs, ops
    e, max_m, k = len(masked), 256, 512
    b_q, b_s = inputs.expert_weights(e, n, k, seed=len(masked))
    a_q, a_s = to.quant_1x128(inputs.activations(e * max_m, k, seed=17))
    a_q, a_s = a_q.view(e, max_m, k), a_s.view(e, max_m, k // 128)
    mm = torch.tensor(masked, dtype=torch.int32)
    ref = to.grouped_gemm_masked(a_q, a_s, b_q, b_s, mm)
    d = cuda_dev
    out = torch.full((e, max_m, n), 7.0, dtype=torch.bfloat16, device=d)
    ops.m_grouped_fp8_gemm_nt_masked_ue8m0(a_q.to(d), ops.pack_sf_rows(a_s.to(d), k), b_q.to(d), ops.packed_weight_scales(b_s.to(d), n, k), out, mm.to(d))
    assert ops.gemm_status(d) == 0
    out = out.cpu()
    for i, c in enumerate(masked):
        if c:
            assert_gemm_close(out[i, :c], ref[i, :c], f"masked ue8m0 expert {i}")
        assert bool((out[i, c:] == 7.0).all())


@pytest.mark.parametrize("counts,i_sz,k", [([128, 256], 256, 512), ([1, 0, 127, 129], 384, 1024), ([300, 5, 0, 0, 77, 128, 1, 640], 128, 256)])
def test_gemm1_with_fused_activation_contiguous(cuda_dev, counts, i_sz, k):
    """GEMM1 with SiLU(gate)*up + quantisation in its epilogue gives the bits of the bf16 GEMM followed by the
    stand-alone activation kernel (bytes, fp32 scales, packed scales); padding rows stay untouched."""
    from kb_nano_b200 import ops
    e, d = len(counts), cuda_dev
    a_q, a_s, b_q, b_s, row_expert = make_grouped(e, 2 * i_sz, k, counts, seed=sum(counts) + i_sz)
    m = a_q.shape[0]
    a_q, row_expert, b_q = a_q.to(d), row_expert.to(d), b_q.to(d)
    sfa, sfb = ops.pack_sf_rows(a_s.to(d), k), ops.packed_weight_scales(b_s.to(d), 2 * i_sz, k)
    mm1 = torch.zeros(m, 2 * i_sz, dtype=torch.bfloat16, device=d)
    ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(a_q, sfa, b_q, sfb, mm1, row_expert)
    q_ref = torch.full((m, i_sz), 0x55, dtype=torch.uint8, device=d).view(FP8)
    s_ref = torch.full((i_sz // 128, m), 7.0, device=d).t()
    ops.silu_mul_quant_fp8_rows(mm1, q_ref, s_ref, row_expert)
    q = torch.full((m, i_sz), 0x55, dtype=torch.uint8, device=d).view(FP8)
    s = torch.full((i_sz // 128, m), 7.0, device=d).t()
    sf = torch.zeros(ops.packed_sf_rows_bytes(m, i_sz), dtype=torch.uint8, device=d)
    ops.m_grouped_gemm1_silu_quant_contiguous_ue8m0(a_q, sfa, b_q, sfb, q, s, row_expert, sf)
    assert ops.gemm_status(d) == 0
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    s_valid = torch.where(s == 7.0, torch.zeros_like(s), s)
    assert torch.equal(sf, ops.pack_sf_rows(s_valid, i_sz))
    valid = (row_expert >= 0).cpu()
    assert bool((q.view(torch.uint8).cpu()[valid] != 0x55).any()) and bool((s.cpu()[~valid] == 7.0).all())


@pytest.mark.parametrize("masked,i_sz", [([0, 1, 128, 129, 256, 77], 256), ([256] * 3, 256), ([5, 200], 256), (MIXED, 512)])
def test_gemm1_with_fused_activation_masked(cuda_dev, masked, i_sz):
    from kb_nano_b200 import inputs, ops
    e, max_m, k, d = len(masked), 256, 512, cuda_dev
    b_q, b_s = inputs.expert_weights(e, 2 * i_sz, k, seed=len(masked) + 9)
    a_q, a_s = to.quant_1x128(inputs.activations(e * max_m, k, seed=23))
    a_q, mm = a_q.view(e, max_m, k).to(d), torch.tensor(masked, dtype=torch.int32, device=d)
    b_q = b_q.to(d)
    sfa, sfb = ops.pack_sf_rows(a_s.to(d), k), ops.packed_weight_scales(b_s.to(d), 2 * i_sz, k)
    mm1 = torch.zeros(e, max_m, 2 * i_sz, dtype=torch.bfloat16, device=d)
    ops.m_grouped_fp8_gemm_nt_masked_ue8m0(a_q, sfa, b_q, sfb, mm1, mm)
    q_ref = torch.full((e, max_m, i_sz), 0x55, dtype=torch.uint8, device=d).view(FP8)
    s_ref = torch.full((e, max_m, i_sz // 128), 7.0, device=d)
    ops.silu_mul_quant_fp8_masked(mm1, q_ref, s_ref, mm)
    q = torch.full((e, max_m, i_sz), 0x55, dtype=torch.uint8, device=d).view(FP8)
    s = torch.full((e, max_m, i_sz // 128), 7.0, device=d)
    sf = torch.zeros(ops.packed_sf_rows_bytes(e * max_m, i_sz), dtype=torch.uint8, device=d)
    ops.m_grouped_gemm1_silu_quant_masked_ue8m0(a_q, sfa, b_q, sfb, q, s, mm, sf)
    assert ops.gemm_status(d) == 0
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    s_valid = torch.where(s == 7.0, torch.zeros_like(s), s)
    assert torch.equal(sf, ops.pack_sf_rows(s_valid.view(e * max_m, -1), i_sz))


def test_mx_matches_fp32_scale_kernel_on_config1(cuda_dev):
    from kb_nano_b200 import inputs, ops
    d = cuda_dev
    x = inputs.activations(512, 7168, seed=0, device=d)
    w_q, w_s = inputs.weight(4096, 7168, seed=1, device=d)
    a_q = torch.empty(512, 7168, dtype=FP8, device=d)
    a_s = torch.empty(56, 512, device=d).t()
    ops.per_token_group_quant_fp8(x, a_q, a_s)
    o1 = torch.empty(512, 4096, dtype=torch.bfloat16, device=d)
    o2 = torch.empty_like(o1)
    ops.fp8_gemm_nt(a_q, a_s, w_q, w_s, o1)
    ops.fp8_gemm_nt_ue8m0(a_q, ops.pack_sf_rows(a_s, 7168), w_q, ops.packed_weight_scales(w_s, 4096, 7168), o2)
    assert ops.gemm_status(d) == 0
    assert_gemm_close(o2.cpu(), o1.cpu(), "ue8m0 path vs fp32-scale path")
    ref = to.gemm_nt_dequant(a_q.cpu(), a_s.cpu(), w_q.cpu(), w_s.cpu())
    assert_gemm_close(o2.cpu(), ref, "ue8m0 path vs oracle, C1")


@pytest.mark.parametrize("shape", [(256, 384), (3, 256, 256), (200, 328)])
def test_weight_requant_to_power_of_two_scales(cuda_dev, shape):
    """Checkpoint-style weights (plain fp32 block scales) re-quantised on the GPU to UE8M0 scales: bytes and
    scales identical to the oracle's dequantise -> per-block cast, and the result takes the UE8M0 GEMM path."""
    from kb_nano_b200 import ops
    gen = torch.Generator().manual_seed(sum(shape))
    w = (0.02 * torch.randn(*shape, generator=gen)).to(torch.bfloat16)
    w_q, w_s = to.block_quant_128x128(w, ue8m0=False)            # arbitrary fp32 scales, as a checkpoint holds them
    ref_q, ref_s = to.requant_weights_ue8m0(w_q, w_s, eps=1e-4)
    d = cuda_dev
    gq, gs = w_q.to(d).contiguous(), w_s.to(d).contiguous()
    assert ops.packed_weight_scales(gs, shape[-2], shape[-1]) is None          # not powers of two yet
    ops.requant_weights_ue8m0(gq, gs, eps=1e-4)
    assert bool((gq.cpu().view(torch.uint8) == ref_q.view(torch.uint8)).all()), "re-quantised bytes differ"
    assert bool((gs.cpu() == ref_s).all()), "re-quantised scales differ"
    assert ops.packed_weight_scales(gs, shape[-2], shape[-1]) is not None


def test_postprocess_then_fp8_linear(cuda_dev):
    """The load-time helper of the Fp8Linear drop-in, then the layer itself, against the oracle."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_fp8_linear_pp", os.path.join(candidate_dir(), "L1", "fp8_linear.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    w = (0.02 * torch.randn(512, 1024, generator=torch.Generator().manual_seed(4))).to(torch.bfloat16)
    w_q, w_s = to.block_quant_128x128(w, ue8m0=False)
    d = cuda_dev
    nw, ns = mod.postprocess_fp8_weights(w_q.to(d), w_s.to(d))
    assert bool(((ns.view(torch.int32) & 0x7FFFFF) == 0).all())
    x = inputs.activations(96, 1024, seed=6)
    out = mod.Fp8Linear()(x.to(d), nw, ns)
    ref_q, ref_s = to.requant_weights_ue8m0(w_q, w_s)
    assert_gemm_close(out.cpu(), to.fp8_linear(x, ref_q, ref_s), "Fp8Linear after postprocess_fp8_weights")
    w3_q, w3_s = torch.stack([w_q, w_q]).to(d), torch.stack([w_s, w_s]).to(d)
    mod.postprocess_fp8_weights_batched(w3_q, w3_s)
    assert bool((w3_q[1].view(torch.uint8) == nw.view(torch.uint8)).all()) and bool((w3_s[0] == ns).all())


@pytest.mark.parametrize("m", [5, 200, 512])
def test_fp8_linear_two_launches(cuda_dev, m):
    """ops.fp8_linear (quantiser emitting packed scales + block-scaled GEMM, or the weight-streaming kernel for few
    rows) against the oracle; the library counts two kernel launches."""
    from kb_nano_b200 import _lib, inputs, ops
    n, k, d = 1024, 2048, cuda_dev
    x = inputs.activations(m, k, seed=m, device=d)
    w_q, w_s = inputs.weight(n, k, seed=m + 1, device=d)
    a_q = torch.empty(m, k, dtype=FP8, device=d)
    a_s = torch.empty(k // 128, m, device=d).t()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=d)
    ops.fp8_linear(x, a_q, a_s, w_q, w_s, out)             # first call packs the weight scales
    l0 = _lib.launch_count()
    ops.fp8_linear(x, a_q, a_s, w_q, w_s, out)
    assert _lib.launch_count() - l0 == 2
    assert ops.gemm_status(d) == 0
    rq, rs = to.quant_1x128(x.cpu())
    assert torch.equal(a_q.cpu().view(torch.uint8), rq.view(torch.uint8))
    assert_gemm_close(out.cpu(), to.gemm_nt_dequant(rq, rs, w_q.cpu(), w_s.cpu()), f"fp8_linear M={m}")
