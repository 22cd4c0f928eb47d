"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Values are drawn in fp32 from one torch.Generator and then cast (a bf16 ``randn`` on CPU truncates
its tail), on whatever device is asked for.  CPU and CUDA generators give different streams, so a
parity check generates once and copies the same bits to the other side.

Weight quantisation here (128x128 blocks, UE8M0 scales) is input preparation written with torch
ops; it is what bench/kernels/scenario_registry.py:185-221 does for the harness's coherent FP8
inputs and is not part of the timed path.
"""
from __future__ import annotations

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def activations(m: int, k: int, seed: int = 0, device="cpu", outlier_frac: float = 0.0,
                outlier_scale: float = 50.0) -> torch.Tensor:
    """bf16 [m,k] ~ N(0,1); a fraction `outlier_frac` of entries multiplied by `outlier_scale`."""
    g = _gen(seed, device)
    x = torch.randn(m, k, generator=g, device=device, dtype=torch.float32)
    if outlier_frac > 0.0:
        mask = torch.rand(m, k, generator=g, device=device) < outlier_frac
        x = torch.where(mask, x * outlier_scale, x)
    return x.to(torch.bfloat16)


def block_quant_128x128(w: torch.Tensor, eps: float = 1e-10):
    """w [..., R, C] (R, C multiples of 128) -> (e4m3 same shape, fp32 UE8M0 scales [..., R/128, C/128])."""
    *lead, r, c = w.shape
    v = w.float().reshape(-1, r // 128, 128, c // 128, 128)
    s = v.abs().amax(dim=(2, 4)).clamp_min(eps) / FP8_MAX
    s = torch.pow(2.0, torch.ceil(torch.log2(s)))
    q = torch.clamp(v / s[:, :, None, :, None], -FP8_MAX, FP8_MAX).to(FP8)
    return q.reshape(*lead, r, c), s.reshape(*lead, r // 128, c // 128)


def weight(n: int, k: int, seed: int = 0, device="cpu", std: float = 0.02):
    """One [n,k] weight ~ N(0, std) as bf16, block-quantised: (e4m3 [n,k], fp32 [n/128,k/128])."""
    g = _gen(seed, device)
    w = (std * torch.randn(n, k, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)
    return block_quant_128x128(w)


def expert_weights(e: int, n: int, k: int, seed: int = 0, device="cpu", std: float = 0.02, first: int = 0):
    """[e,n,k] expert weights generated and quantised one expert at a time (expert `first + i` uses
    sub-seed seed*1000003 + first + i, so a rank that owns a block of experts generates exactly the
    weights the whole set would have), keeping only one expert's bf16 master alive at once."""
    q = torch.empty(e, n, k, dtype=FP8, device=device)
    s = torch.empty(e, n // 128, k // 128, dtype=torch.float32, device=device)
    for i in range(e):
        q[i], s[i] = weight(n, k, seed * 1000003 + first + i, device, std)
    return q, s


def route_sigmoid_topk(logits: torch.Tensor, k: int):
    """DeepSeek-V3 style: sigmoid scores, top-k, renormalised weights (fp32), int32 ids."""
    w, ids = torch.topk(torch.sigmoid(logits.float()), k, dim=-1)
    return w / w.sum(dim=-1, keepdim=True), ids.to(torch.int32)


def route_softmax_topk(logits: torch.Tensor, k: int):
    """Mixtral style: softmax, top-k, renormalised weights (fp32), int32 ids."""
    w, ids = torch.topk(torch.softmax(logits.float(), dim=-1), k, dim=-1)
    return w / w.sum(dim=-1, keepdim=True), ids.to(torch.int32)


def router_logits(t: int, e: int, seed: int = 0, device="cpu") -> torch.Tensor:
    return torch.randn(t, e, generator=_gen(seed + 7919, device), device=device, dtype=torch.float32)
