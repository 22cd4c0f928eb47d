"""GPU parity, through the C ABI, of the two memory-bound kernels against the CPU oracle:
fp8 bytes and fp32 scale bits must be identical."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from oracle import torch_oracle as to
from tests.util import assert_quant_equal, bf16_from_bits, bits16, golden

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def run_quant(x_cpu, dev, colmajor=False, ue8m0=True, eps=1e-10, through="ops"):
    from kb_nano_b200 import ops
    x = x_cpu.to(dev)
    m, k = x.shape
    g = (k + 127) // 128
    q = torch.empty(m, k, dtype=FP8, device=dev)
    s = torch.empty(g, m, device=dev).t() if colmajor else torch.empty(m, g, device=dev)
    ops.per_token_group_quant_fp8(x, q, s, ue8m0, eps)
    torch.cuda.synchronize()
    return q.cpu(), s.cpu()


def test_quant_golden(cuda_dev):
    g = golden("quant_1x128")
    for cm in (False, True):
        q, s = run_quant(bf16_from_bits(g["x"]), cuda_dev, colmajor=cm)
        assert_quant_equal(q, s, g["q"], g["s"], f"golden colmajor={cm}")


def test_quant_ragged_k_generic_path(cuda_dev):
    g = golden("quant_1x128")
    q, s = run_quant(bf16_from_bits(g["x_ragged"]), cuda_dev)      # K=200: 16-byte path with a short group
    assert_quant_equal(q, s, g["q_ragged"], g["s_ragged"], "ragged K=200")
    x = bf16_from_bits(g["x_ragged"])[:, :197].contiguous()         # K=197: element-wise kernel
    q, s = run_quant(x, cuda_dev)
    qr, sr = co.quant_1x128(bits16(x))
    assert_quant_equal(q, s, qr, sr, "ragged K=197")


@pytest.mark.parametrize("m", [1, 127, 128, 129])
def test_quant_row_counts(cuda_dev, m):
    from kb_nano_b200 import inputs
    x = inputs.activations(m, 7168, seed=m)
    q, s = run_quant(x, cuda_dev, colmajor=True)
    qr, sr = co.quant_1x128(bits16(x))
    assert_quant_equal(q, s, qr, sr, f"M={m}")


def test_quant_every_bf16_absmax(cuda_dev):
    """One group per positive finite bf16 value as its absmax: pins the exponent rule everywhere."""
    bits = np.arange(1, 0x7F80, dtype=np.uint16)
    x = np.zeros((bits.size, 128), np.uint16)
    x[:, 3] = bits
    x[:, 77] = bits | 0x8000                # same magnitude, negative
    x[:, 100] = (bits >> 1)                 # something smaller alongside
    xt = bf16_from_bits(x)
    q, s = run_quant(xt, cuda_dev)
    qr, sr = co.quant_1x128(x)
    assert_quant_equal(q, s, qr, sr, "all absmax")
    qt, st = to.quant_1x128(xt)
    assert_quant_equal(q, s, qt, st, "all absmax vs torch oracle")


def test_quant_config1_activation(cuda_dev):
    """A of the dense-linear configuration: [512, 7168] ~ N(0,1), column-major scales."""
    from kb_nano_b200 import inputs
    x = inputs.activations(512, 7168, seed=0)
    q, s = run_quant(x, cuda_dev, colmajor=True)
    qr, sr = co.quant_1x128(bits16(x))
    assert_quant_equal(q, s, qr, sr, "C1 activations")
    assert (np.ascontiguousarray(s.numpy()).view(np.uint32) & 0x7FFFFF == 0).all()


def test_quant_plain_scales(cuda_dev):
    from kb_nano_b200 import inputs
    x = inputs.activations(64, 1024, seed=3, outlier_frac=1e-3)
    q, s = run_quant(x, cuda_dev, ue8m0=False)
    qr, sr = co.quant_1x128(bits16(x), ue8m0=False)
    assert_quant_equal(q, s, qr, sr, "ue8m0=False")


def test_quant_strided_rows_and_noncontiguous_scale_views(cuda_dev):
    from kb_nano_b200 import inputs, ops
    big = inputs.activations(40, 1024, seed=5).to(cuda_dev)
    x = big[:, 256:768]                      # row stride 1024, K = 512
    q_big = torch.zeros(40, 1024, dtype=torch.uint8, device=cuda_dev).view(FP8)
    q = q_big[:, 128:640]
    s = torch.empty(40, 4, device=cuda_dev)
    ops.per_token_group_quant_fp8(x, q, s)
    qr, sr = co.quant_1x128(bits16(x.cpu().contiguous()))
    assert_quant_equal(q.cpu().contiguous(), s.cpu(), qr, sr, "strided")
    # bytes outside the view are untouched
    assert int(q_big.view(torch.uint8)[:, :128].sum()) == 0 and int(q_big.view(torch.uint8)[:, 640:].sum()) == 0


def test_quant_empty(cuda_dev):
    from kb_nano_b200 import ops
    x = torch.empty(0, 256, dtype=torch.bfloat16, device=cuda_dev)
    ops.per_token_group_quant_fp8(x, torch.empty(0, 256, dtype=FP8, device=cuda_dev), torch.empty(0, 2, device=cuda_dev))


def test_quant_idempotent_scale_of_requantised_output(cuda_dev):
    """Size-independent property at a large size: dequantised output re-quantises to the same bytes."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(4096, 7168, seed=11, device=cuda_dev)
    q = torch.empty(4096, 7168, dtype=FP8, device=cuda_dev)
    s = torch.empty(4096, 56, device=cuda_dev)
    ops.per_token_group_quant_fp8(x, q, s)
    deq = (q.float().view(4096, 56, 128) * s[:, :, None]).view(4096, 7168).to(torch.bfloat16)
    q2 = torch.empty_like(q)
    s2 = torch.empty_like(s)
    ops.per_token_group_quant_fp8(deq, q2, s2)
    # e4m3 values times a power of two are exact in bf16, so the second pass reproduces the bytes
    # wherever the group's largest quantised magnitude still maps to the same scale
    same_scale = (s2 == s)
    assert same_scale.float().mean() > 0.5
    eq = (q2.view(torch.uint8) == q.view(torch.uint8)).view(4096, 56, 128).all(-1)
    assert bool(eq[same_scale].all())
    # and a sampled slab is bit-exact against the oracle
    rows = torch.arange(0, 4096, 97)
    qr, sr = co.quant_1x128(bits16(x[rows].cpu()))
    assert_quant_equal(q[rows].cpu(), s[rows].cpu(), qr, sr, "sampled rows of [4096,7168]")


# ---- fused SiLU*up + quant -----------------------------------------------------------------------

def run_smq(x_cpu, dev, ue8m0=True, eps=1e-10):
    from kb_nano_b200 import ops
    x = x_cpu.to(dev)
    m, n = x.shape
    q = torch.empty(m, n // 2, dtype=FP8, device=dev)
    s = torch.empty(n // 2 // 128, m, device=dev).t()
    ops.silu_mul_quant_fp8(x, q, s, ue8m0, eps)
    torch.cuda.synchronize()
    return q.cpu(), s.cpu()


def test_silu_exhaustive_over_all_gates(cuda_dev):
    """silu(g) -> bf16 on the device equals the oracle for every finite bf16 gate."""
    from kb_nano_b200 import ops
    dev_tab = bits16(ops.silu_bf16_table(cuda_dev).cpu())
    ref = co.silu_bf16_table()
    gates = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    finite = torch.isfinite(gates).numpy()
    bad = np.nonzero((dev_tab != ref) & finite)[0]
    assert bad.size == 0, f"{bad.size} gates differ, first {bad[:8]}"
    assert int(((dev_tab != golden('silu_table')['table']) & finite).sum()) == 0


def test_silu_exhaustive_gate_times_several_ups(cuda_dev):
    """Every finite gate against a spread of up values, through the full kernel."""
    gates = np.arange(65536, dtype=np.uint16)
    gates = gates[np.isfinite(bf16_from_bits(gates).float().numpy())]
    n = (gates.size // 128) * 128
    gates = gates[:n].reshape(-1, 128)
    rng = np.random.default_rng(0)
    ups_f = rng.standard_normal(gates.shape).astype(np.float32) * 3
    # keep silu(g)*up finite in bf16: an infinite product has no defined quantisation
    huge = np.abs(bf16_from_bits(gates).float().numpy()) > 1e30
    ups_f = np.where(huge, np.clip(ups_f, -1.0, 1.0), ups_f)
    ups = bits16(torch.from_numpy(ups_f).to(torch.bfloat16))
    x = np.concatenate([gates, ups], axis=1)
    q, s = run_smq(bf16_from_bits(x), cuda_dev)
    qr, sr = co.silu_mul_quant_1x128(x)
    assert_quant_equal(q, s, qr, np.ascontiguousarray(sr), "all gates x random ups")


def test_silu_every_gate_through_the_shared_memory_table_kernel(cuda_dev):
    """Inputs of 32768 groups or more run on the persistent kernel that keeps the exact table in shared
    memory; every finite gate appears in this one, with random ups, checked bit for bit."""
    rng = np.random.default_rng(1)
    gates = np.arange(65536, dtype=np.uint16)
    gf = bf16_from_bits(gates).float().numpy()
    gates = np.where(np.isfinite(gf) & (np.abs(gf) < 1e30), gates, np.uint16(0x3F80))
    g = np.tile(gates.reshape(8, 8192), (64, 1))                     # [512, 8192]: 512 * 64 = 32768 groups
    rng.shuffle(g, axis=1)
    ups = bits16(torch.from_numpy(rng.standard_normal(g.shape).astype(np.float32) * 2).to(torch.bfloat16))
    x = np.concatenate([g, ups], axis=1)
    q, s = run_smq(bf16_from_bits(x), cuda_dev)
    qr, sr = co.silu_mul_quant_1x128(x)
    assert_quant_equal(q, s, qr, np.ascontiguousarray(sr), "shared-memory-table kernel, all gates")


def test_silu_mul_quant_golden(cuda_dev):
    g = golden("silu_mul_quant")
    q, s = run_smq(bf16_from_bits(g["x"]), cuda_dev)
    assert_quant_equal(q, s, g["q"], g["s"], "golden")
    assert s.stride() == (1, 128)


def test_silu_mul_quant_config2_sample(cuda_dev):
    """The fused-activation configuration: [16384, 2x2048] with 0.1% entries x50; rows sampled for the oracle."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(16384, 4096, seed=0, device=cuda_dev, outlier_frac=1e-3, outlier_scale=50.0)
    q = torch.empty(16384, 2048, dtype=FP8, device=cuda_dev)
    s = torch.empty(16, 16384, device=cuda_dev).t()
    ops.silu_mul_quant_fp8(x, q, s)
    rows = torch.arange(0, 16384, 16)
    qr, sr = co.silu_mul_quant_1x128(bits16(x[rows].cpu()))
    assert_quant_equal(q[rows].cpu(), s[rows].cpu(), qr, np.ascontiguousarray(sr), "C2 sampled rows")
    # whole-tensor properties: power-of-two scales, |q| <= 448, every group reaches >= 224 unless it is eps-clamped
    sb = s.contiguous().view(torch.int32)
    assert bool(((sb & 0x7FFFFF) == 0).all())
    qa = q.float().abs().view(16384, 16, 128).amax(-1)
    assert bool((qa <= 448).all()) and bool(((qa >= 224) | (s <= 2.0 ** -42)).all())


def test_silu_mul_quant_plain_scales_and_eps(cuda_dev):
    from kb_nano_b200 import inputs
    x = inputs.activations(128, 512, seed=9)
    q, s = run_smq(x, cuda_dev, ue8m0=False, eps=1e-6)
    qr, sr = co.silu_mul_quant_1x128(bits16(x), eps=1e-6, ue8m0=False)
    assert_quant_equal(q, s, qr, np.ascontiguousarray(sr), "ue8m0=False eps=1e-6")


def test_candidate_modules_match_oracle(cuda_dev):
    """The kb-nano drop-in classes, loaded by file path as kb-nano's kernel swapper does."""
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    def load(name):
        spec = importlib.util.spec_from_file_location(f"_candidate_impl_L1_{name}", os.path.join(candidate_dir(), "L1", name + ".py"))
        mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
        return mod
    x = inputs.activations(256, 1024, seed=2).to(cuda_dev)
    out, scales = load("silu_mul_quant_fp8").SiluMulQuantFp8()(x)
    qr, sr = co.silu_mul_quant_1x128(bits16(x.cpu()))
    assert scales.shape == (256, 4) and scales.stride() == (1, 256)
    assert_quant_equal(out.cpu(), scales.cpu(), qr, np.ascontiguousarray(sr), "SiluMulQuantFp8")
    with pytest.raises(AssertionError):
        load("silu_mul_quant_fp8").SiluMulQuantFp8()(x[:100])
    m = load("fp8_linear")
    q = torch.empty(256, 1024, dtype=FP8, device=cuda_dev)
    s = torch.empty(256, 8, device=cuda_dev)
    assert m.PerTokenGroupQuantFp8()(x, q, s) is None
    qr, sr = co.quant_1x128(bits16(x.cpu()))
    assert_quant_equal(q.cpu(), s.cpu(), qr, sr, "PerTokenGroupQuantFp8")


def test_silu_mul_quant_row_skipping_variants(cuda_dev):
    """Expert-contiguous (-1 rows skipped) and masked (rows >= masked_m skipped) forms: processed rows are
    bit-exact, skipped rows are left untouched."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(512, 1024, seed=21)
    qr, sr = co.silu_mul_quant_1x128(bits16(x))
    row_expert = torch.full((512,), -1, dtype=torch.int32)
    row_expert[:100] = 0
    row_expert[128:300] = 2
    row_expert[384:385] = 3
    q = torch.full((512, 512), 0x55, dtype=torch.uint8, device=cuda_dev).view(FP8)
    s = torch.full((4, 512), 7.0, device=cuda_dev).t()
    ops.silu_mul_quant_fp8_rows(x.to(cuda_dev), q, s, row_expert.to(cuda_dev))
    v = (row_expert >= 0).numpy()
    assert_quant_equal(q.cpu().view(torch.uint8).numpy()[v], s.cpu().numpy()[v], qr[v], np.ascontiguousarray(sr)[v], "rows variant")
    assert (q.cpu().view(torch.uint8).numpy()[~v] == 0x55).all() and (s.cpu().numpy()[~v] == 7.0).all()
    # masked: 4 experts x 128 rows
    masked = torch.tensor([0, 128, 5, 77], dtype=torch.int32)
    q3 = torch.full((4, 128, 512), 0x55, dtype=torch.uint8, device=cuda_dev).view(FP8)
    s3 = torch.full((4, 128, 4), 7.0, device=cuda_dev)
    ops.silu_mul_quant_fp8_masked(x.to(cuda_dev).view(4, 128, 1024), q3, s3, masked.to(cuda_dev))
    q3 = q3.cpu().view(torch.uint8).numpy().reshape(512, 512)
    s3 = s3.cpu().numpy().reshape(512, 4)
    v = np.concatenate([np.arange(128) < int(c) for c in masked])
    assert_quant_equal(q3[v], s3[v], qr[v], np.ascontiguousarray(sr)[v], "masked variant")
    assert (q3[~v] == 0x55).all() and (s3[~v] == 7.0).all()


@pytest.mark.parametrize("m,n2", [(512, 512), (4096, 2048)])
def test_silu_mul_quant_row_list(cuda_dev, m, n2):
    """Only the listed rows are processed (small inputs: flat kernel; 32768 groups or more: the persistent one)."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(m, 2 * n2, seed=m)
    gen = torch.Generator().manual_seed(n2)
    rows = torch.randperm(m, generator=gen)[: m // 2].to(torch.int32)
    rows[::7] = -1                                           # skipped entries
    q = torch.full((m, n2), 0x55, dtype=torch.uint8, device=cuda_dev).view(FP8)
    s = torch.full((n2 // 128, m), 7.0, device=cuda_dev).t()
    pad = torch.cat([rows, torch.full((m * 8,), -1, dtype=torch.int32)]) if m == 4096 else rows   # long list -> persistent kernel
    sf = torch.zeros(ops.packed_sf_rows_bytes(m, n2), dtype=torch.uint8, device=cuda_dev)
    ops.silu_mul_quant_fp8_list(x.to(cuda_dev), q, s, pad.to(cuda_dev), packed_sf=sf)
    # the packed copy of the scales equals packing the fp32 scales of the processed rows afterwards
    s_done = torch.where(s == 7.0, torch.zeros_like(s), s)
    assert torch.equal(sf.cpu(), ops.pack_sf_rows(s_done, n2).cpu())
    qr, sr = co.silu_mul_quant_1x128(bits16(x))
    done = np.zeros(m, bool)
    done[rows[rows >= 0].numpy()] = True
    assert_quant_equal(q.cpu().view(torch.uint8).numpy()[done], s.cpu().numpy()[done], qr[done], np.ascontiguousarray(sr)[done], "row list")
    assert (q.cpu().view(torch.uint8).numpy()[~done] == 0x55).all() and (s.cpu().numpy()[~done] == 7.0).all()


@pytest.mark.parametrize("m,k", [(1, 128), (200, 7168), (129, 1040), (512, 4096)])
def test_quant_emits_packed_scales(cuda_dev, m, k):
    """kbn_quant_1x128_sf: same bytes and scales as the plain call, and the packed copy of the scales equals packing
    them afterwards (rows of the last 128-row block past M are not written)."""
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(m, k, seed=m + k, device=cuda_dev)
    g = (k + 127) // 128
    q0 = torch.empty(m, k, dtype=FP8, device=cuda_dev)
    s0 = torch.empty(g, m, device=cuda_dev).t()
    ops.per_token_group_quant_fp8(x, q0, s0)
    q1 = torch.empty(m, k, dtype=FP8, device=cuda_dev)
    s1 = torch.empty(g, m, device=cuda_dev).t()
    ref = ops.pack_sf_rows(s0, k)
    sf = ref.clone()                       # pre-filled with the reference so that the unwritten padding rows compare equal
    sf.view(torch.int32)[:] ^= 0x01010101
    pad_rows = (-m) % 128
    ops.per_token_group_quant_fp8(x, q1, s1, packed_sf=sf)
    assert torch.equal(q0.view(torch.uint8), q1.view(torch.uint8)) and torch.equal(s0, s1)
    words, refw = sf.view(torch.int32).view(-1, g, 32, 4), ref.view(torch.int32).view(-1, g, 32, 4)
    rows = torch.arange(128, device=cuda_dev)
    valid = torch.ones(words.shape[0], 128, dtype=torch.bool, device=cuda_dev)
    if pad_rows:
        valid[-1, 128 - pad_rows:] = False
    vmask = valid[:, rows % 32 + 32 * (rows // 32)].view(-1, 1, 4, 32).transpose(2, 3).expand_as(words)   # word (l, i) <-> row 32 i + l
    assert torch.equal(words[vmask], refw[vmask])
    assert bool((words[~vmask] == (refw[~vmask] ^ 0x01010101)).all())
