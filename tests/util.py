"""Helpers shared by the tests: bit views, golden loading, tolerance rules."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def fp8_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e4m3fn)


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def scale_exponents(s) -> np.ndarray:
    """Biased exponent field of fp32 scales (bits >> 23); power-of-two scales have a zero mantissa."""
    a = s.detach().cpu().contiguous().numpy() if isinstance(s, torch.Tensor) else np.ascontiguousarray(s)
    return a.view(np.uint32) >> 23


def assert_quant_equal(q_got, s_got, q_ref, s_ref, what=""):
    """Bit-exact: fp8 bytes and fp32 scale bits."""
    qg = bits8(q_got) if isinstance(q_got, torch.Tensor) else q_got
    qr = bits8(q_ref) if isinstance(q_ref, torch.Tensor) else q_ref
    sg = (s_got.detach().cpu().contiguous().numpy() if isinstance(s_got, torch.Tensor) else np.ascontiguousarray(s_got)).view(np.uint32)
    sr = (s_ref.detach().cpu().contiguous().numpy() if isinstance(s_ref, torch.Tensor) else np.ascontiguousarray(s_ref)).view(np.uint32)
    nb = int((qg != qr).sum())
    ns = int((sg != sr).sum())
    assert nb == 0 and ns == 0, f"{what}: {nb} fp8 bytes and {ns} scales differ"


# GEMM / MoE outputs: the bound the task states -- max relative error 1e-2 and cosine > 0.9999 --
# evaluated the way kb-nano's harness does for bf16 (bench/kernels/runner.py:31-37,296-312):
# |got-ref| <= atol + rtol*|ref| with atol = rtol = 1e-2, plus a global ||d||inf/||ref||inf check.
RTOL = 1e-2
ATOL = 1e-2
COS_MIN = 0.9999


def gemm_errors(got: torch.Tensor, ref: torch.Tensor) -> dict:
    g = got.detach().float().cpu().flatten()
    r = ref.detach().float().cpu().flatten()
    d = (g - r).abs()
    return {
        "ratio": float((d / (ATOL + RTOL * r.abs())).max()) if d.numel() else 0.0,
        "rel_inf": float(d.max() / r.abs().max().clamp_min(1e-30)) if d.numel() else 0.0,
        "cos": float(torch.nn.functional.cosine_similarity(g.double(), r.double(), dim=0)) if d.numel() else 1.0,
        "finite": bool(torch.isfinite(g).all()),
    }


def assert_gemm_close(got: torch.Tensor, ref: torch.Tensor, what=""):
    e = gemm_errors(got, ref)
    assert e["finite"], f"{what}: non-finite output"
    assert e["ratio"] <= 1.0 and e["rel_inf"] <= RTOL and e["cos"] > COS_MIN, f"{what}: {e}"
