"""Fused (add +) RMSNorm + 1x128 FP8 quant against the oracle's restatement of kb-nano's CUDA kernel.
A floating-point kernel (the sum of squares is order-dependent), so the comparison uses kb-nano's own rule
for (fp8, scale) pairs: |dequant(got) - dequant(ref)| <= 0.5*scale + 0.125*|ref| (bench/kernels/runner.py:265-291),
plus: scales identical and bytes identical on all but a sliver of groups/elements."""
import pytest
import torch

from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def pair_close(q, s, qr, sr, what):
    s, sr = s.cpu().contiguous(), sr.contiguous()
    deq = q.cpu().float() * s.repeat_interleave(128, dim=-1)[:, : q.shape[1]]
    ref = qr.float() * sr.repeat_interleave(128, dim=-1)[:, : q.shape[1]]
    tol = 0.5 * sr.repeat_interleave(128, dim=-1)[:, : q.shape[1]] + 0.125 * ref.abs()
    assert bool(((deq - ref).abs() <= tol).all()), f"{what}: outside the fp8 pair tolerance"
    same_scale = float((s == sr).float().mean())
    same_bytes = float((q.cpu().view(torch.uint8) == qr.view(torch.uint8)).float().mean())
    assert same_scale > 0.999 and same_bytes > 0.995, f"{what}: scales equal {same_scale:.5f}, bytes equal {same_bytes:.5f}"


@pytest.mark.parametrize("m,h", [(1, 128), (7, 1024), (130, 7168), (16, 4096), (5, 200 * 8)])
def test_rmsnorm_quant(cuda_dev, m, h):
    from kb_nano_b200 import inputs, ops
    x = inputs.activations(m, h, seed=m + h, outlier_frac=1e-3)
    w = (1.0 + 0.1 * torch.randn(h, generator=torch.Generator().manual_seed(h))).to(torch.bfloat16)
    q = torch.empty(m, h, dtype=FP8, device=cuda_dev)
    s = torch.empty((h + 127) // 128, m, device=cuda_dev).t()
    ops.rmsnorm_quant_fp8(x.to(cuda_dev), w.to(cuda_dev), q, s, 1e-6)
    qr, sr = to.rmsnorm_quant(x, w, 1e-6)
    pair_close(q, s, qr, sr, f"rmsnorm_quant {m}x{h}")


def test_fused_add_rmsnorm_quant_candidate(cuda_dev):
    import importlib.util, os, sys
    from kb_nano_b200 import candidate_dir, inputs
    spec = importlib.util.spec_from_file_location("_candidate_impl_L1_rmsnorm_quant", os.path.join(candidate_dir(), "L1", "rmsnorm_quant.py"))
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)
    m, h = 96, 7168
    x = inputs.activations(m, h, seed=1)
    r = inputs.activations(m, h, seed=2)
    w = (1.0 + 0.1 * torch.randn(h, generator=torch.Generator().manual_seed(3))).to(torch.bfloat16)
    xd, rd = x.to(cuda_dev).view(2, 48, h).clone(), r.to(cuda_dev).view(2, 48, h).clone()
    q, s, r_out = mod.FusedAddRMSNormFP8Quant()(xd, rd, w.to(cuda_dev), 1e-6)
    qr, sr, r_ref, x_ref = to.rmsnorm_quant(x, w, 1e-6, residual=r)
    assert r_out.data_ptr() == rd.data_ptr() and s.stride() == (1, m)
    assert bool((rd.view(m, h).cpu().view(torch.int16) == r_ref.view(torch.int16)).all()), "residual <- bf16(residual + x) must be exact"
    pair_close(q, s, qr, sr, "fused add rmsnorm quant")
    # normalised row written back to input: bf16 of the same fp32 value, at most one bf16 ulp apart
    got, ref = xd.view(m, h).cpu().float(), x_ref.float()
    assert float(((got - ref).abs() / ref.abs().clamp_min(1e-3)).max()) <= 2.0 ** -7
    q2, s2 = mod.RMSNormFP8Quant()(x.to(cuda_dev).view(2, 48, h), w.to(cuda_dev), 1e-6)
    qr2, sr2 = to.rmsnorm_quant(x, w, 1e-6)
    assert q2.shape == (m, h) and s2.shape == (m, h // 128)
    pair_close(q2, s2, qr2, sr2, "RMSNormFP8Quant")
