"""Second oracle: kb-nano's own Triton kernels for this path, run on the GPU beside the CUDA kernels.

The files come from the kb-nano tree through `oracle/make_ref.py` (oracle/_ref/, git-ignored, made where a kb-nano
tree is present and carried to the GPU machine with the repository).  Bit-for-bit for the two quantisers --
tasks/baseline/L1/silu_mul_quant_fp8.py:23-76 (the kernel the models run between the MoE projections; the CPU
fixtures pin torch's `exp`, this pins Triton's `tl.exp`) and the `_fp8_group_quant_kernel` of
tasks/baseline/L1/fp8_linear.py:181-215 -- and under the bf16 tolerance for `_fused_moe_kernel`
(tasks/baseline/L1/moe_grouped_gemm.py:86-189).  Skipped, with the reason, where oracle/_ref or a launchable Triton
is missing."""
import importlib
import os

import numpy as np
import pytest
import torch

from tests.util import assert_gemm_close, bf16_from_bits, bits16, bits8, fp8_from_bits, golden

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _ref(name):
    if not os.path.isfile(os.path.join(REF_DIR, name + ".py")):
        pytest.skip("oracle/_ref is absent (made by oracle/make_ref.py where a kb-nano tree is present)")
    try:
        import triton  # noqa: F401
    except Exception as ex:      # pragma: no cover
        pytest.skip(f"Triton is not importable: {ex}")
    return importlib.import_module("oracle._ref." + name)


def _launch(fn):
    """Runs a Triton launch; a Triton that cannot compile for this GPU is a skip, not a failure of this library."""
    try:
        out = fn()
        torch.cuda.synchronize()
        return out
    except AssertionError:
        raise
    except Exception as ex:
        pytest.skip(f"the reference's Triton kernel does not launch here: {type(ex).__name__}: {str(ex)[:200]}")


def _ours_smq(x, dev):
    from kb_nano_b200 import ops
    m, n = x.shape
    q = torch.empty(m, n // 2, dtype=FP8, device=dev)
    s = torch.empty(n // 256, m, device=dev).t()
    ops.silu_mul_quant_fp8(x, q, s)
    return q, s


def _count_diff(q, s, q_ref, s_ref):
    nb = int((bits8(q) != bits8(q_ref)).sum())
    ns = int((s.cpu().contiguous().numpy().view(np.uint32) != s_ref.cpu().contiguous().numpy().view(np.uint32)).sum())
    return nb, ns


def test_silu_mul_quant_every_gate_against_the_triton_kernel(cuda_dev):
    """Every finite bf16 gate (magnitudes above 1e30 aside: an infinite product has no defined quantisation) times a
    spread of ups through kb-nano's Triton kernel and through both of this library's kernels (the small-input one
    and the persistent one with the table in shared memory): not one fp8 byte or scale bit may differ."""
    mod = _ref("silu_mul_quant_fp8")
    rng = np.random.default_rng(7)
    gates = np.arange(65536, dtype=np.uint16)
    gf = bf16_from_bits(gates).float().numpy()
    gates = np.where(np.isfinite(gf) & (np.abs(gf) < 1e30), gates, np.uint16(0x3F80))
    for rows, what in ((128, "small-input kernel"), (512, "shared-memory-table kernel")):
        g = np.tile(gates.reshape(8, 8192), (rows // 8, 1))
        rng.shuffle(g, axis=1)
        ups = bits16(torch.from_numpy(rng.standard_normal(g.shape).astype(np.float32) * 2).to(torch.bfloat16))
        x = bf16_from_bits(np.concatenate([g, ups], axis=1)).to(cuda_dev)
        q_ref, s_ref = _launch(lambda: mod.SiluMulQuantFp8()(x))
        q, s = _ours_smq(x, cuda_dev)
        nb, ns = _count_diff(q, s, q_ref, s_ref)
        assert nb == 0 and ns == 0, f"{what}: {nb} fp8 bytes and {ns} scales differ from the Triton kernel"
        assert s.stride() == s_ref.stride()


def test_silu_mul_quant_config2_against_the_triton_kernel(cuda_dev):
    """BASELINE configs[1] at full size: bf16 [16384, 2x2048] with 0.1% of the entries x50."""
    from kb_nano_b200 import inputs
    mod = _ref("silu_mul_quant_fp8")
    x = inputs.activations(16384, 4096, seed=0, device=cuda_dev, outlier_frac=1e-3, outlier_scale=50.0)
    q_ref, s_ref = _launch(lambda: mod.SiluMulQuantFp8()(x))
    q, s = _ours_smq(x, cuda_dev)
    nb, ns = _count_diff(q, s, q_ref, s_ref)
    assert nb == 0 and ns == 0, f"{nb} fp8 bytes and {ns} scales differ from the Triton kernel"


def test_quant_1x128_against_the_triton_kernel(cuda_dev):
    """The edge-case fixture (zeros, eps-sized values, every exponent, outliers) and a large random input through
    `_fp8_group_quant_kernel`, launched as tasks/baseline/L1/fp8_linear.py:269-279 launches it."""
    from kb_nano_b200 import inputs, ops
    mod = _ref("fp8_group_quant")
    g = golden("quant_1x128")
    cases = [bf16_from_bits(g["x"]).to(cuda_dev), inputs.activations(4096, 7168, seed=3, device=cuda_dev, outlier_frac=1e-3)]
    for x in cases:
        x = x.contiguous()
        m, k = x.shape
        if k % 128:
            continue
        q_ref = torch.empty(m, k, dtype=FP8, device=cuda_dev)
        s_ref = torch.empty(k // 128, m, device=cuda_dev).t()
        _launch(lambda: mod._fp8_group_quant_kernel[(m * (k // 128),)](
            x, q_ref, s_ref, x.stride(0), q_ref.stride(0), s_ref.stride(0), s_ref.stride(1), k,
            fp8_max=float(torch.finfo(FP8).max), GROUP_SIZE=128, USE_UE8M0=True))
        q = torch.empty_like(q_ref)
        s = torch.empty(k // 128, m, device=cuda_dev).t()
        ops.per_token_group_quant_fp8(x, q, s)
        nb, ns = _count_diff(q, s, q_ref, s_ref)
        assert nb == 0 and ns == 0, f"[{m},{k}]: {nb} fp8 bytes and {ns} scales differ from the Triton kernel"


def test_grouped_gemm_against_the_triton_kernel(cuda_dev):
    """kb-nano's `_fused_moe_kernel` (through its MoeGroupedGemm module) and this library's drop-in for it on the
    grouped-GEMM fixture's inputs: both within the bf16 tolerance of the fixture, and of each other."""
    import importlib.util
    import sys
    from kb_nano_b200 import candidate_dir
    mod = _ref("moe_grouped_gemm")
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_moe_grouped_gemm_t", os.path.join(candidate_dir(), "L1", "moe_grouped_gemm.py"))
    ours = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = ours
    spec.loader.exec_module(ours)
    g = golden("grouped_gemm")
    d = cuda_dev
    a_q, a_s = fp8_from_bits(g["a_q"]).to(d), torch.from_numpy(g["a_s"]).to(d)
    b_q, b_s = fp8_from_bits(g["b_q"]).to(d), torch.from_numpy(g["b_s"]).to(d)
    tw = torch.from_numpy(g["topk_w"]).to(d)
    sorted_ids, blk = torch.from_numpy(g["sorted_ids"]).to(d), torch.from_numpy(g["blk_experts"]).to(d)
    t, topk = g["topk_ids"].shape
    ntpp = torch.tensor([sorted_ids.numel()], dtype=torch.int32, device=d)
    cfg = {"BLOCK_SIZE_M": 16, "BLOCK_SIZE_N": 64, "BLOCK_SIZE_K": 128, "GROUP_SIZE_M": 1}
    c_ref = torch.zeros(t * topk, b_q.shape[1], dtype=torch.bfloat16, device=d)
    _launch(lambda: mod.MoeGroupedGemm()(a_q, b_q, c_ref, tw, sorted_ids, blk, ntpp, False, topk, config=cfg, a_scale=a_s, b_scale=b_s,
                                        use_fp8_w8a8=True, block_shape=[128, 128]))
    c = torch.zeros_like(c_ref)
    ours.MoeGroupedGemm()(a_q, b_q, c, tw, sorted_ids, blk, ntpp, False, topk, config=cfg, a_scale=a_s, b_scale=b_s,
                          use_fp8_w8a8=True, block_shape=[128, 128])
    assert_gemm_close(c_ref.cpu(), bf16_from_bits(g["c"]), "Triton _fused_moe_kernel vs fixture")
    assert_gemm_close(c.cpu(), c_ref.cpu(), "drop-in vs Triton _fused_moe_kernel")
