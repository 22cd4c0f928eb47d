"""Tensor-level entry points: validate torch tensors, pass raw pointers to the C ABI.

PyTorch is used for device memory and streams only; every function enqueues hand-written
sm_100a kernels on the current stream of the tensors' device and returns without syncing.
"""
from __future__ import annotations

import collections
import ctypes

import torch

from . import _lib

FP8 = torch.float8_e4m3fn
GROUP = 128


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("kb_nano_b200 ops need CUDA tensors (there is no CPU path)")
        if t.device != dev:
            raise ValueError("all tensors must be on the same device")
    return dev


class _on:
    """Make the tensors' device current for the duration of a call (no-op when it already is)."""

    def __init__(self, dev: torch.device):
        self.guard = None if dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *a):
        if self.guard is not None:
            self.guard.__exit__(*a)


def _scale_strides(scale: torch.Tensor, rows: int, groups: int) -> tuple[int, int]:
    if scale.dtype != torch.float32 or scale.dim() != 2 or tuple(scale.shape) != (rows, groups):
        raise ValueError(f"scale must be float32 [{rows}, {groups}], got {scale.dtype} {tuple(scale.shape)}")
    return scale.stride(0), scale.stride(1)


def per_token_group_quant_fp8(x: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor,
                              use_ue8m0: bool = True, eps: float = 1e-10, packed_sf: torch.Tensor | None = None) -> None:
    """In-place 1x128 quantisation: x bf16 [M,K] -> out_fp8 [M,K], out_scale fp32 [M,ceil(K/128)] (any strides).
    packed_sf (uint8, packed_sf_rows_bytes(M, K) bytes; UE8M0 only) also receives the scales in the packed form the
    *_ue8m0 GEMMs read."""
    dev = _cuda(x, out_fp8, out_scale)
    if x.dim() != 2 or x.dtype != torch.bfloat16:
        raise ValueError(f"x must be bf16 [M,K], got {x.dtype} {tuple(x.shape)}")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != tuple(x.shape):
        raise ValueError("out_fp8 must be float8_e4m3fn with x's shape")
    if x.stride(1) != 1 or out_fp8.stride(1) != 1:
        raise ValueError("x and out_fp8 must be contiguous along K")
    m, k = x.shape
    s_row, s_grp = _scale_strides(out_scale, m, (k + GROUP - 1) // GROUP)
    if packed_sf is not None:
        if not use_ue8m0:
            raise ValueError("packed scales need UE8M0 scales")
        _check_packed(packed_sf, m, k, dev)
        with _on(dev):
            _lib.check(_lib.load().kbn_quant_1x128_sf(x.data_ptr(), m, k, x.stride(0) if m > 1 else k, out_fp8.data_ptr(),
                                                      out_fp8.stride(0) if m > 1 else k, out_scale.data_ptr(), s_row, s_grp,
                                                      eps, packed_sf.data_ptr(), _stream(x)))
        return
    with _on(dev):
        _lib.check(_lib.load().kbn_quant_1x128(x.data_ptr(), m, k, x.stride(0) if m > 1 else k, out_fp8.data_ptr(),
                                               out_fp8.stride(0) if m > 1 else k, out_scale.data_ptr(), s_row, s_grp,
                                               eps, int(use_ue8m0), _stream(x)))


def silu_mul_quant_fp8(inp: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor,
                       use_ue8m0: bool = True, eps: float = 1e-10) -> None:
    """inp bf16 [M, 2*N2] (gate|up) -> out_fp8 [M,N2], out_scale fp32 [M,N2/128] (any strides)."""
    dev = _cuda(inp, out_fp8, out_scale)
    if inp.dim() != 2 or inp.dtype != torch.bfloat16 or inp.stride(1) != 1:
        raise ValueError("inp must be bf16 [M, 2*N2], contiguous along the last dim")
    m, n = inp.shape
    n2 = n // 2
    if n % 2 or n2 % GROUP:
        raise ValueError(f"N//2={n2} must be a multiple of {GROUP}")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (m, n2) or out_fp8.stride(1) != 1:
        raise ValueError("out_fp8 must be float8_e4m3fn [M, N2], contiguous along the last dim")
    s_row, s_grp = _scale_strides(out_scale, m, n2 // GROUP)
    with _on(dev):
        _lib.check(_lib.load().kbn_silu_mul_quant_1x128(inp.data_ptr(), m, n2, inp.stride(0) if m > 1 else n,
                                                        out_fp8.data_ptr(), out_fp8.stride(0) if m > 1 else n2,
                                                        out_scale.data_ptr(), s_row, s_grp, eps, int(use_ue8m0),
                                                        _stream(inp)))


def silu_mul_quant_fp8_rows(inp: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor, row_expert: torch.Tensor,
                            use_ue8m0: bool = True, eps: float = 1e-10) -> None:
    """As silu_mul_quant_fp8, but only rows with row_expert[m] >= 0 are read and written (the padding
    rows of the expert-contiguous layout are skipped)."""
    dev = _cuda(inp, out_fp8, out_scale, row_expert)
    m, n = inp.shape
    n2 = n // 2
    if inp.dtype != torch.bfloat16 or inp.stride(1) != 1 or n % 2 or n2 % GROUP:
        raise ValueError("inp must be bf16 [M, 2*N2] with N2 a multiple of 128, contiguous along the last dim")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (m, n2) or out_fp8.stride(1) != 1:
        raise ValueError("out_fp8 must be float8_e4m3fn [M, N2], contiguous along the last dim")
    if row_expert.dtype != torch.int32 or row_expert.numel() != m or not row_expert.is_contiguous():
        raise ValueError("row_expert must be contiguous int32 [M]")
    s_row, s_grp = _scale_strides(out_scale, m, n2 // GROUP)
    with _on(dev):
        _lib.check(_lib.load().kbn_silu_mul_quant_1x128_rows(inp.data_ptr(), m, n2, inp.stride(0) if m > 1 else n,
                                                             out_fp8.data_ptr(), out_fp8.stride(0) if m > 1 else n2,
                                                             out_scale.data_ptr(), s_row, s_grp, eps, int(use_ue8m0),
                                                             row_expert.data_ptr(), _stream(inp)))


def silu_mul_quant_fp8_list(inp: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor, row_list: torch.Tensor,
                            use_ue8m0: bool = True, eps: float = 1e-10, packed_sf: torch.Tensor | None = None) -> None:
    """As silu_mul_quant_fp8, but only the rows listed in row_list (int32, entries < 0 skipped) are processed.
    packed_sf (uint8, packed_sf_rows_bytes(M, N2) bytes) also receives the listed rows' scales in the packed
    form the *_ue8m0 GEMMs read."""
    dev = _cuda(inp, out_fp8, out_scale, row_list)
    m, n = inp.shape
    n2 = n // 2
    if inp.dtype != torch.bfloat16 or inp.stride(1) != 1 or n % 2 or n2 % GROUP:
        raise ValueError("inp must be bf16 [M, 2*N2] with N2 a multiple of 128, contiguous along the last dim")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (m, n2) or out_fp8.stride(1) != 1:
        raise ValueError("out_fp8 must be float8_e4m3fn [M, N2], contiguous along the last dim")
    if row_list.dtype != torch.int32 or not row_list.is_contiguous():
        raise ValueError("row_list must be contiguous int32")
    s_row, s_grp = _scale_strides(out_scale, m, n2 // GROUP)
    sf_ptr = None
    if packed_sf is not None:
        _check_packed(packed_sf, m, n2, dev)
        sf_ptr = packed_sf.data_ptr()
    with _on(dev):
        _lib.check(_lib.load().kbn_silu_mul_quant_1x128_list(inp.data_ptr(), n2, inp.stride(0) if m > 1 else n, out_fp8.data_ptr(),
                                                             out_fp8.stride(0) if m > 1 else n2, out_scale.data_ptr(), s_row, s_grp,
                                                             eps, int(use_ue8m0), row_list.data_ptr(), row_list.numel(), sf_ptr,
                                                             _stream(inp)))


def silu_mul_quant_fp8_masked(inp: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor, masked_m: torch.Tensor) -> None:
    """Masked layout: inp bf16 [E,max_m,2*N2] -> out_fp8 [E,max_m,N2], out_scale fp32 [E,max_m,N2/128]
    (all contiguous); only rows m < masked_m[e] are processed."""
    dev = _cuda(inp, out_fp8, out_scale, masked_m)
    e, max_m, n = inp.shape
    n2 = n // 2
    if inp.dtype != torch.bfloat16 or not inp.is_contiguous() or n2 % GROUP:
        raise ValueError("inp must be contiguous bf16 [E, max_m, 2*N2] with N2 a multiple of 128")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (e, max_m, n2) or not out_fp8.is_contiguous():
        raise ValueError("out_fp8 must be contiguous float8_e4m3fn [E, max_m, N2]")
    if out_scale.dtype != torch.float32 or tuple(out_scale.shape) != (e, max_m, n2 // GROUP) or not out_scale.is_contiguous():
        raise ValueError("out_scale must be contiguous float32 [E, max_m, N2/128]")
    if masked_m.dtype != torch.int32 or masked_m.numel() != e or not masked_m.is_contiguous():
        raise ValueError("masked_m must be contiguous int32 [E]")
    with _on(dev):
        _lib.check(_lib.load().kbn_silu_mul_quant_1x128_masked(inp.data_ptr(), e, max_m, n2, out_fp8.data_ptr(),
                                                               out_scale.data_ptr(), masked_m.data_ptr(), _stream(inp)))


def silu_bf16_table(device: torch.device | str = "cuda") -> torch.Tensor:
    """bf16 [65536]: silu(g) rounded to bf16 for every gate bit pattern g, as the fused kernel computes it."""
    out = torch.empty(65536, dtype=torch.int16, device=device)
    with _on(out.device):
        _lib.check(_lib.load().kbn_silu_bf16_table(out.data_ptr(), _stream(out)))
    return out.view(torch.bfloat16)


def _check_ab(a: torch.Tensor, b: torch.Tensor, k: int) -> None:
    if a.dtype != FP8 or b.dtype != FP8:
        raise ValueError("A and B must be float8_e4m3fn")
    if not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("A and B must be contiguous (K-major)")
    if a.shape[-1] != k or b.shape[-1] != k:
        raise ValueError("A and B disagree on K")


def _check_sb(sb: torch.Tensor, lead: tuple, n: int, k: int) -> torch.Tensor:
    want = (*lead, (n + 127) // 128, (k + 127) // 128)
    if sb.dtype != torch.float32 or tuple(sb.shape) != want:
        raise ValueError(f"weight scale must be float32 {want}, got {sb.dtype} {tuple(sb.shape)}")
    return sb if sb.is_contiguous() else sb.contiguous()


def _bias_ptr(bias: torch.Tensor | None, n: int, dev) -> int | None:
    if bias is None:
        return None
    if bias.dtype != torch.bfloat16 or bias.numel() != n or not bias.is_contiguous() or bias.device != dev:
        raise ValueError(f"bias must be contiguous bf16 [{n}] on {dev}")
    return bias.data_ptr()


def fp8_gemm_nt(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, out: torch.Tensor,
                bias: torch.Tensor | None = None) -> None:
    """out bf16 [M,N] = (a_q, a_s [M,K/128]) @ (b_q [N,K], b_s [N/128,K/128])^T (+ bias, in fp32, before the rounding),
    written in place."""
    dev = _cuda(a_q, a_s, b_q, b_s, out)
    m, k = a_q.shape
    n = b_q.shape[0]
    _check_ab(a_q, b_q, k)
    sa_row, sa_grp = _scale_strides(a_s, m, (k + 127) // 128)
    b_s = _check_sb(b_s, (), n, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be bf16 [M,N], contiguous along N")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_gemm_nt(a_q.data_ptr(), a_s.data_ptr(), sa_row, sa_grp, b_q.data_ptr(),
                                               b_s.data_ptr(), _bias_ptr(bias, n, dev), out.data_ptr(), out.stride(0) if m > 1 else n,
                                               m, n, k, _stream(out)))


def m_grouped_fp8_gemm_nt_contiguous(a_q, a_s, b_q, b_s, out, expert_ids) -> None:
    """Rows of a_q [M_sum,K] use expert expert_ids[row] of b_q [E,N,K]; rows with id < 0 are not written."""
    dev = _cuda(a_q, a_s, b_q, b_s, out, expert_ids)
    m, k = a_q.shape
    e, n, _ = b_q.shape
    _check_ab(a_q, b_q, k)
    sa_row, sa_grp = _scale_strides(a_s, m, (k + 127) // 128)
    b_s = _check_sb(b_s, (e,), n, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be bf16 [M_sum,N], contiguous along N")
    if expert_ids.dtype != torch.int32 or expert_ids.numel() != m or not expert_ids.is_contiguous():
        raise ValueError("expert_ids must be contiguous int32 [M_sum]")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_contig(a_q.data_ptr(), a_s.data_ptr(), sa_row, sa_grp,
                                                           b_q.data_ptr(), b_s.data_ptr(), out.data_ptr(),
                                                           out.stride(0) if m > 1 else n, expert_ids.data_ptr(),
                                                           m, n, k, e, _stream(out)))


def m_grouped_fp8_gemm_nt_masked(a_q, a_s, b_q, b_s, out, masked_m) -> None:
    """a_q [E,max_m,K], a_s [E,max_m,K/128], b_q [E,N,K], out bf16 [E,max_m,N]; rows >= masked_m[e] untouched."""
    dev = _cuda(a_q, a_s, b_q, b_s, out, masked_m)
    e, max_m, k = a_q.shape
    n = b_q.shape[1]
    _check_ab(a_q, b_q, k)
    if b_q.shape[0] != e:
        raise ValueError("A and B disagree on the number of experts")
    if a_s.dtype != torch.float32 or tuple(a_s.shape) != (e, max_m, (k + 127) // 128):
        raise ValueError("a_s must be float32 [E, max_m, ceil(K/128)]")
    b_s = _check_sb(b_s, (e,), n, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (e, max_m, n) or not out.is_contiguous():
        raise ValueError("out must be contiguous bf16 [E,max_m,N]")
    if masked_m.dtype != torch.int32 or masked_m.numel() != e or not masked_m.is_contiguous():
        raise ValueError("masked_m must be contiguous int32 [E]")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_masked(a_q.data_ptr(), a_s.data_ptr(), a_s.stride(0), a_s.stride(1),
                                                           a_s.stride(2), b_q.data_ptr(), b_s.data_ptr(), out.data_ptr(),
                                                           masked_m.data_ptr(), e, max_m, n, k, _stream(out)))


def gemm_status(device: torch.device | str = "cuda") -> int:
    """0 unless a bounded wait inside a GEMM kernel has ever run out in this process (synchronises)."""
    dev = torch.device(device)
    out = ctypes.c_int32(0)
    with _on(dev if dev.index is not None else torch.device("cuda", torch.cuda.current_device())):
        _lib.check(_lib.load().kbn_gemm_status(ctypes.byref(out), torch.cuda.current_stream().cuda_stream))
    return int(out.value)


def gemm_clear_status(device: torch.device | str = "cuda") -> None:
    """Sets the GEMM status word back to 0 (ordered on the device's current stream)."""
    dev = torch.device(device)
    dev = dev if dev.index is not None else torch.device("cuda", torch.cuda.current_device())
    with _on(dev):
        _lib.check(_lib.load().kbn_gemm_clear_status(torch.cuda.current_stream(dev).cuda_stream))


def moe_pair_experts(sorted_token_ids: torch.Tensor | None, expert_ids: torch.Tensor, block_m: int, pair_expert: torch.Tensor) -> None:
    """pair_expert int32 [n_pairs] <- expert of every (token, slot) pair, from the sorted, block-padded pair list of
    kb-nano's Triton MoE path (position i of sorted_token_ids lies in block i // block_m, whose expert is
    expert_ids[i // block_m]; entries >= n_pairs are padding); -1 for pairs that appear in no block.  Without a list
    block i holds the single pair i."""
    dev = _cuda(expert_ids, pair_expert) if sorted_token_ids is None else _cuda(sorted_token_ids, expert_ids, pair_expert)
    for name, x in (("sorted_token_ids", sorted_token_ids), ("expert_ids", expert_ids), ("pair_expert", pair_expert)):
        if x is not None and (x.dtype != torch.int32 or not x.is_contiguous()):
            raise ValueError(f"{name} must be contiguous int32")
    with _on(dev):
        _lib.check(_lib.load().kbn_moe_pair_experts(
            sorted_token_ids.data_ptr() if sorted_token_ids is not None else None,
            sorted_token_ids.numel() if sorted_token_ids is not None else 0, expert_ids.data_ptr(), expert_ids.numel(), int(block_m),
            pair_expert.numel(), pair_expert.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))


def moe_aligned_rows(t: int, topk: int, e: int) -> int:
    return int(_lib.load().kbn_moe_aligned_rows(t, topk, e))


def moe_permute(a_q: torch.Tensor, a_s: torch.Tensor, topk_ids: torch.Tensor, num_experts: int,
                a_perm: torch.Tensor, a_s_perm: torch.Tensor, row_expert: torch.Tensor, dest_row: torch.Tensor,
                workspace: torch.Tensor, packed_sf: torch.Tensor | None = None) -> None:
    """Group quantised rows by expert into 128-aligned segments (all outputs caller-allocated).  packed_sf
    (uint8, packed_sf_rows_bytes(M_cap, K) bytes) also receives the moved rows' scales in the packed form
    the *_ue8m0 GEMMs read."""
    dev = _cuda(a_q, a_s, topk_ids, a_perm, a_s_perm, row_expert, dest_row, workspace)
    t, k = a_q.shape
    topk = topk_ids.shape[1]
    g = k // GROUP
    m_cap = a_perm.shape[0]
    if a_q.dtype != FP8 or a_perm.dtype != FP8 or not a_q.is_contiguous() or not a_perm.is_contiguous() or a_perm.shape[1] != k:
        raise ValueError("a_q / a_perm must be contiguous float8_e4m3fn with the same K")
    if a_s.dtype != torch.float32 or tuple(a_s.shape) != (t, g) or not a_s.is_contiguous():
        raise ValueError("a_s must be contiguous float32 [T, K/128]")
    if a_s_perm.dtype != torch.float32 or tuple(a_s_perm.shape) != (m_cap, g) or not a_s_perm.is_contiguous():
        raise ValueError("a_s_perm must be contiguous float32 [M_cap, K/128]")
    if topk_ids.dtype != torch.int32 or not topk_ids.is_contiguous() or topk_ids.shape[0] != t:
        raise ValueError("topk_ids must be contiguous int32 [T, topk]")
    if row_expert.dtype != torch.int32 or row_expert.numel() != m_cap or not row_expert.is_contiguous():
        raise ValueError("row_expert must be contiguous int32 [M_cap]")
    if dest_row.dtype != torch.int32 or tuple(dest_row.shape) != (t, topk) or not dest_row.is_contiguous():
        raise ValueError("dest_row must be contiguous int32 [T, topk]")
    ws_bytes = workspace.numel() * workspace.element_size()
    sf_ptr = None
    if packed_sf is not None:
        _check_packed(packed_sf, m_cap, k, dev)
        sf_ptr = packed_sf.data_ptr()
    with _on(dev):
        _lib.check(_lib.load().kbn_moe_permute_sf(a_q.data_ptr(), a_s.data_ptr(), topk_ids.data_ptr(), t, topk, k, num_experts,
                                                  a_perm.data_ptr(), a_s_perm.data_ptr(), row_expert.data_ptr(),
                                                  dest_row.data_ptr(), m_cap, workspace.data_ptr(), ws_bytes, sf_ptr, _stream(a_q)))


def moe_route_topk(logits: torch.Tensor, topk: int, scoring: str = "softmax", bias: torch.Tensor | None = None, n_group: int = 1,
                   topk_group: int = 1, renormalize: bool = True, renorm_floor: float = 0.0, scale: float = 1.0,
                   round_bf16: bool = False, out_w: torch.Tensor | None = None, out_ids: torch.Tensor | None = None):
    """Router logits [T, E] (fp32 or bf16) -> (weights fp32 [T, topk], expert ids int32 [T, topk]) in one kernel:
    softmax or sigmoid scores, optional selection bias and group-limited selection, top-k, renormalisation, scaling."""
    if scoring not in ("softmax", "sigmoid"):
        raise ValueError(f"unsupported scoring function {scoring!r}")
    if logits.dim() != 2 or logits.dtype not in (torch.float32, torch.bfloat16) or logits.stride(1) != 1:
        raise ValueError("logits must be fp32 or bf16 [T, E], contiguous along E")
    t, e = logits.shape
    tensors = [logits] + ([bias] if bias is not None else [])
    if out_w is None:
        out_w = torch.empty(t, topk, dtype=torch.float32, device=logits.device)
    if out_ids is None:
        out_ids = torch.empty(t, topk, dtype=torch.int32, device=logits.device)
    dev = _cuda(*tensors, out_w, out_ids)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != e or not bias.is_contiguous()):
        raise ValueError("bias must be contiguous float32 [E]")
    if out_w.dtype != torch.float32 or tuple(out_w.shape) != (t, topk) or not out_w.is_contiguous():
        raise ValueError("out_w must be contiguous float32 [T, topk]")
    if out_ids.dtype != torch.int32 or tuple(out_ids.shape) != (t, topk) or not out_ids.is_contiguous():
        raise ValueError("out_ids must be contiguous int32 [T, topk]")
    with _on(dev):
        _lib.check(_lib.load().kbn_moe_route_topk(logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0) if t > 1 else e,
                                                  t, e, int(scoring == "softmax"), bias.data_ptr() if bias is not None else None,
                                                  n_group, topk_group, topk, int(renormalize), renorm_floor, scale, int(round_bf16),
                                                  out_w.data_ptr(), out_ids.data_ptr(), _stream(logits)))
    return out_w, out_ids


def moe_permute_workspace_bytes(t: int, topk: int, e: int) -> int:
    return int(_lib.load().kbn_moe_permute_workspace_bytes(t, topk, e))


def moe_unpermute_combine(rows: torch.Tensor, dest_row: torch.Tensor, topk_w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = sum_s topk_w[t,s] * rows[dest_row[t,s]]  (bf16 rows, fp32 weights and accumulation)."""
    dev = _cuda(rows, dest_row, topk_w, out)
    t, topk = dest_row.shape
    h = out.shape[1]
    if rows.dtype != torch.bfloat16 or rows.stride(1) != 1 or rows.shape[1] != h:
        raise ValueError("rows must be bf16 [M_cap, H], contiguous along H")
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (t, h) or not out.is_contiguous():
        raise ValueError("out must be contiguous bf16 [T, H]")
    if topk_w.dtype != torch.float32 or tuple(topk_w.shape) != (t, topk) or not topk_w.is_contiguous():
        raise ValueError("topk_w must be contiguous float32 [T, topk]")
    if dest_row.dtype != torch.int32 or not dest_row.is_contiguous():
        raise ValueError("dest_row must be contiguous int32 [T, topk]")
    with _on(dev):
        _lib.check(_lib.load().kbn_moe_unpermute_combine(rows.data_ptr(), rows.stride(0), dest_row.data_ptr(),
                                                         topk_w.data_ptr(), t, topk, h, out.data_ptr(), _stream(out)))


# ---- UE8M0 fast path: packed power-of-two scales, block-scaled tensor-core instruction -------------

def packed_sf_rows_bytes(rows: int, k: int) -> int:
    return int(_lib.load().kbn_packed_sf_rows_bytes(rows, k))


def _check_packed(buf: torch.Tensor, rows: int, k: int, dev) -> None:
    if buf.dtype != torch.uint8 or not buf.is_contiguous() or buf.device != dev or buf.numel() < packed_sf_rows_bytes(rows, k):
        raise ValueError(f"packed scale buffer must be contiguous uint8 on {dev} with at least {packed_sf_rows_bytes(rows, k)} bytes")
    if buf.data_ptr() % 16:
        raise ValueError("packed scale buffer must be 16-byte aligned")


def pack_sf_rows(scale: torch.Tensor, k: int) -> torch.Tensor:
    """fp32 scales [..., rows, ceil(K/128)] (any strides on the last two dims; leading dims contiguous over
    rows) -> packed uint8 buffer for the *_ue8m0 GEMMs."""
    s2 = scale if scale.dim() == 2 else scale.reshape(-1, scale.shape[-1])
    rows = s2.shape[0]
    if s2.dtype != torch.float32 or s2.shape[1] != (k + 127) // 128:
        raise ValueError("scale must be float32 [rows, ceil(K/128)]")
    lib = _lib.load()
    out = torch.empty(int(lib.kbn_packed_sf_rows_bytes(rows, k)), dtype=torch.uint8, device=scale.device)
    with _on(scale.device):
        _lib.check(lib.kbn_pack_sf_rows(s2.data_ptr(), rows, k, s2.stride(0), s2.stride(1), out.data_ptr(), _stream(scale)))
    return out


_WEIGHT_SF_CACHE: "collections.OrderedDict" = collections.OrderedDict()
_WEIGHT_SF_CACHE_MAX = 16384      # far above the number of FP8 weight tensors of any model; least recently used goes first


def packed_weight_scales(b_s: torch.Tensor, n: int, k: int):
    """(packed buffer or None) for fp32 weight scales [E?, N/128, K/128].  None when some scale is not a
    power of two, in which case the fp32-scale kernel must be used.  Checked and packed once per tensor
    (keyed by storage address, shape and version; the entry keeps the tensor alive, so the address cannot be
    reused).  That first call launches two small kernels and synchronises the stream; it cannot happen inside a
    CUDA-graph capture: load-time code (``postprocess_fp8_weights*`` of the drop-in linear layer, or one eager
    warm-up call) makes it happen before."""
    key = (b_s.data_ptr(), tuple(b_s.shape), b_s._version, str(b_s.device))
    hit = _WEIGHT_SF_CACHE.get(key)
    if hit is not None:
        _WEIGHT_SF_CACHE.move_to_end(key)
        return hit[0]
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("packed_weight_scales: these weight scales have not been seen before and checking them needs a "
                           "host synchronisation, which a CUDA-graph capture does not allow; call the layer once eagerly "
                           "(or ops.packed_weight_scales on its scales) before capturing")
    s = b_s if b_s.is_contiguous() else b_s.contiguous()
    e = s.shape[0] if s.dim() == 3 else 1
    lib = _lib.load()
    with _on(s.device):
        cnt = torch.zeros(1, dtype=torch.int32, device=s.device)
        _lib.check(lib.kbn_count_non_pow2_scales(s.data_ptr(), s.numel(), cnt.data_ptr(), _stream(s)))
        packed = None
        if int(cnt.item()) == 0:
            packed = torch.empty(int(lib.kbn_packed_sf_weights_bytes(e, n, k)), dtype=torch.uint8, device=s.device)
            _lib.check(lib.kbn_pack_sf_weights(s.data_ptr(), e, n, k, packed.data_ptr(), _stream(s)))
    while len(_WEIGHT_SF_CACHE) >= _WEIGHT_SF_CACHE_MAX:
        _WEIGHT_SF_CACHE.popitem(last=False)
    _WEIGHT_SF_CACHE[key] = (packed, b_s)
    return packed


def fp8_gemm_nt_ue8m0(a_q, sfa_packed, b_q, sfb_packed, out, bias: torch.Tensor | None = None) -> None:
    dev = _cuda(a_q, sfa_packed, b_q, sfb_packed, out)
    m, k = a_q.shape
    n = b_q.shape[0]
    _check_ab(a_q, b_q, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be bf16 [M,N], contiguous along N")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_gemm_nt_ue8m0(a_q.data_ptr(), sfa_packed.data_ptr(), b_q.data_ptr(), sfb_packed.data_ptr(),
                                                     _bias_ptr(bias, n, dev), out.data_ptr(), out.stride(0) if m > 1 else n, m, n, k,
                                                     _stream(out)))


def m_grouped_fp8_gemm_nt_contiguous_ue8m0(a_q, sfa_packed, b_q, sfb_packed, out, expert_ids) -> None:
    dev = _cuda(a_q, sfa_packed, b_q, sfb_packed, out, expert_ids)
    m, k = a_q.shape
    e, n, _ = b_q.shape
    _check_ab(a_q, b_q, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be bf16 [M_sum,N], contiguous along N")
    if expert_ids.dtype != torch.int32 or expert_ids.numel() != m or not expert_ids.is_contiguous():
        raise ValueError("expert_ids must be contiguous int32 [M_sum]")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_contig_ue8m0(a_q.data_ptr(), sfa_packed.data_ptr(), b_q.data_ptr(),
                                                                 sfb_packed.data_ptr(), out.data_ptr(), out.stride(0) if m > 1 else n,
                                                                 expert_ids.data_ptr(), m, n, k, e, _stream(out)))


def m_grouped_fp8_gemm_nt_masked_ue8m0(a_q, sfa_packed, b_q, sfb_packed, out, masked_m) -> None:
    dev = _cuda(a_q, sfa_packed, b_q, sfb_packed, out, masked_m)
    e, max_m, k = a_q.shape
    n = b_q.shape[1]
    _check_ab(a_q, b_q, k)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (e, max_m, n) or not out.is_contiguous():
        raise ValueError("out must be contiguous bf16 [E,max_m,N]")
    if masked_m.dtype != torch.int32 or masked_m.numel() != e or not masked_m.is_contiguous():
        raise ValueError("masked_m must be contiguous int32 [E]")
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_masked_ue8m0(a_q.data_ptr(), sfa_packed.data_ptr(), b_q.data_ptr(),
                                                                 sfb_packed.data_ptr(), out.data_ptr(), masked_m.data_ptr(),
                                                                 e, max_m, n, k, _stream(out)))


def m_grouped_gemm1_silu_quant_contiguous_ue8m0(a_q, sfa_packed, w13_q, sfb_packed, out_fp8, out_scale, expert_ids,
                                                packed_sf: torch.Tensor | None = None) -> None:
    """GEMM1 of the expert MLP with SiLU(gate)*up + 1x128 quantisation in its epilogue: a_q [M_sum,K] x
    w13_q [E,2I,K] -> out_fp8 [M_sum,I], out_scale fp32 [M_sum,I/128] (any strides) and, optionally, the packed
    copy of the scales.  Same bits as the bf16 GEMM followed by silu_mul_quant_fp8."""
    dev = _cuda(a_q, sfa_packed, w13_q, sfb_packed, out_fp8, out_scale, expert_ids)
    m, k = a_q.shape
    e, n2, _ = w13_q.shape
    i = n2 // 2
    _check_ab(a_q, w13_q, k)
    if n2 % 2 or i % GROUP:
        raise ValueError("w13 must have 2*I rows per expert with I a multiple of 128")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (m, i) or out_fp8.stride(1) != 1:
        raise ValueError("out_fp8 must be float8_e4m3fn [M_sum, I], contiguous along the last dim")
    if expert_ids.dtype != torch.int32 or expert_ids.numel() != m or not expert_ids.is_contiguous():
        raise ValueError("expert_ids must be contiguous int32 [M_sum]")
    s_row, s_grp = _scale_strides(out_scale, m, i // GROUP)
    sf_ptr = None
    if packed_sf is not None:
        _check_packed(packed_sf, m, i, dev)
        sf_ptr = packed_sf.data_ptr()
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_contig_ue8m0_silu(
            a_q.data_ptr(), sfa_packed.data_ptr(), w13_q.data_ptr(), sfb_packed.data_ptr(), out_fp8.data_ptr(),
            out_fp8.stride(0) if m > 1 else i, out_scale.data_ptr(), s_row, s_grp, sf_ptr, expert_ids.data_ptr(), m, i, k, e,
            _stream(out_fp8)))


def m_grouped_gemm1_silu_quant_masked_ue8m0(a_q, sfa_packed, w13_q, sfb_packed, out_fp8, out_scale, masked_m,
                                            packed_sf: torch.Tensor | None = None) -> None:
    """Masked-layout form: a_q [E,max_m,K] x w13_q [E,2I,K] -> out_fp8 [E,max_m,I], out_scale fp32 [E,max_m,I/128]
    (both contiguous); rows m >= masked_m[e] are not written."""
    dev = _cuda(a_q, sfa_packed, w13_q, sfb_packed, out_fp8, out_scale, masked_m)
    e, max_m, k = a_q.shape
    i = w13_q.shape[1] // 2
    _check_ab(a_q, w13_q, k)
    if w13_q.shape[1] % 2 or i % GROUP:
        raise ValueError("w13 must have 2*I rows per expert with I a multiple of 128")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (e, max_m, i) or not out_fp8.is_contiguous():
        raise ValueError("out_fp8 must be contiguous float8_e4m3fn [E,max_m,I]")
    if out_scale.dtype != torch.float32 or tuple(out_scale.shape) != (e, max_m, i // GROUP) or not out_scale.is_contiguous():
        raise ValueError("out_scale must be contiguous float32 [E,max_m,I/128]")
    if masked_m.dtype != torch.int32 or masked_m.numel() != e or not masked_m.is_contiguous():
        raise ValueError("masked_m must be contiguous int32 [E]")
    sf_ptr = None
    if packed_sf is not None:
        _check_packed(packed_sf, e * max_m, i, dev)
        sf_ptr = packed_sf.data_ptr()
    with _on(dev):
        _lib.check(_lib.load().kbn_fp8_grouped_gemm_masked_ue8m0_silu(
            a_q.data_ptr(), sfa_packed.data_ptr(), w13_q.data_ptr(), sfb_packed.data_ptr(), out_fp8.data_ptr(),
            out_scale.data_ptr(), sf_ptr, masked_m.data_ptr(), e, max_m, i, k, _stream(out_fp8)))


_LINEAR_SF: dict = {}
_LINEAR_SF_RETIRED: list = []     # outgrown buffers stay alive: a captured CUDA graph may still write into them


def fp8_linear(x: torch.Tensor, a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, out: torch.Tensor,
               bias: torch.Tensor | None = None) -> None:
    """The FP8 linear layer in two launches: 1x128 quantisation of x into a_q / a_s, then the GEMM against b_q / b_s
    into out.  With power-of-two weight scales and more than 8 rows the quantiser writes the packed scales the
    block-scaled GEMM reads itself (no packing launch); 8 rows or fewer take the weight-streaming kernel."""
    m, k = x.shape
    n = b_q.shape[0]
    packed_w = packed_weight_scales(b_s, n, k) if m > 8 else None
    if packed_w is None or k % 8 or x.stride(0) % 8 or a_q.stride(0) % 8 or x.data_ptr() % 16:
        per_token_group_quant_fp8(x, a_q, a_s)
        fp8_gemm_nt_auto(a_q, a_s, b_q, b_s, out, bias)
        return
    need = packed_sf_rows_bytes(m, k)
    key = (str(x.device), torch.cuda.current_stream(x.device).cuda_stream)
    buf = _LINEAR_SF.get(key)
    if buf is None or buf.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("fp8_linear: the packed-scale buffer must grow, which a CUDA-graph capture does not allow; "
                               "call the layer eagerly with the largest batch first")
        if buf is not None:
            _LINEAR_SF_RETIRED.append(buf)
        buf = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=x.device)     # one per device and stream, grow-only
        _LINEAR_SF[key] = buf
    per_token_group_quant_fp8(x, a_q, a_s, packed_sf=buf)
    fp8_gemm_nt_ue8m0(a_q, buf, b_q, packed_w, out, bias)


def fp8_gemm_nt_auto(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, out: torch.Tensor,
                     bias: torch.Tensor | None = None) -> None:
    """Dense block-scaled GEMM for activations quantised with power-of-two (UE8M0) scales, which is what
    per_token_group_quant_fp8 produces by default: takes the block-scaled tensor-core path when the weight
    scales are powers of two as well (checked once per weight tensor), the fp32-scale kernel otherwise."""
    n, k = b_q.shape
    if a_q.shape[0] <= 8:
        # decode-sized batch: the fp32-scale entry point streams the weights with a kernel of its own, as fast as the
        # block-scaled path at this size and without the scale-packing launch
        fp8_gemm_nt(a_q, a_s, b_q, b_s, out, bias)
        return
    packed = packed_weight_scales(b_s, n, k)
    if packed is not None:
        fp8_gemm_nt_ue8m0(a_q, pack_sf_rows(a_s, k), b_q, packed, out, bias)
    else:
        fp8_gemm_nt(a_q, a_s, b_q, b_s, out, bias)


def rmsnorm_quant_fp8(x: torch.Tensor, weight: torch.Tensor, out_fp8: torch.Tensor, out_scale: torch.Tensor, eps: float = 1e-6,
                      residual: torch.Tensor | None = None) -> None:
    """RMSNorm(x) * weight quantised 1x128 (UE8M0) into out_fp8 / out_scale.  With `residual`: residual += x
    (rounded to bf16) first, the norm is taken of the new residual, and x is overwritten with the normalised row."""
    tensors = [x, weight, out_fp8, out_scale] + ([residual] if residual is not None else [])
    dev = _cuda(*tensors)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise ValueError("x must be bf16 [M,H], contiguous along H")
    m, h = x.shape
    if weight.dtype != torch.bfloat16 or weight.numel() != h or not weight.is_contiguous():
        raise ValueError("weight must be contiguous bf16 [H]")
    if out_fp8.dtype != FP8 or tuple(out_fp8.shape) != (m, h) or out_fp8.stride(1) != 1:
        raise ValueError("out_fp8 must be float8_e4m3fn [M,H], contiguous along H")
    s_row, s_grp = _scale_strides(out_scale, m, (h + GROUP - 1) // GROUP)
    lib = _lib.load()
    with _on(dev):
        if residual is None:
            _lib.check(lib.kbn_rmsnorm_quant_1x128(x.data_ptr(), weight.data_ptr(), m, h, x.stride(0) if m > 1 else h, out_fp8.data_ptr(),
                                                   out_fp8.stride(0) if m > 1 else h, out_scale.data_ptr(), s_row, s_grp, eps, _stream(x)))
        else:
            if residual.dtype != torch.bfloat16 or tuple(residual.shape) != (m, h) or residual.stride(1) != 1:
                raise ValueError("residual must be bf16 [M,H], contiguous along H")
            _lib.check(lib.kbn_add_rmsnorm_quant_1x128(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), m, h,
                                                       x.stride(0) if m > 1 else h, residual.stride(0) if m > 1 else h,
                                                       out_fp8.data_ptr(), out_fp8.stride(0) if m > 1 else h, out_scale.data_ptr(),
                                                       s_row, s_grp, eps, _stream(x)))


def requant_weights_ue8m0(w_fp8: torch.Tensor, scale: torch.Tensor, eps: float = 1e-4) -> None:
    """In place: block-scaled FP8 weights [N,K] or [E,N,K] with fp32 128x128 scales -> the same weights
    re-quantised to power-of-two scales (load-time step; afterwards the UE8M0 GEMM path applies)."""
    dev = _cuda(w_fp8, scale)
    if w_fp8.dtype != FP8 or not w_fp8.is_contiguous() or w_fp8.dim() not in (2, 3):
        raise ValueError("w_fp8 must be contiguous float8_e4m3fn [N,K] or [E,N,K]")
    e = w_fp8.shape[0] if w_fp8.dim() == 3 else 1
    n, k = w_fp8.shape[-2], w_fp8.shape[-1]
    want = ((e,) if w_fp8.dim() == 3 else ()) + ((n + 127) // 128, (k + 127) // 128)
    if scale.dtype != torch.float32 or tuple(scale.shape) != want or not scale.is_contiguous():
        raise ValueError(f"scale must be contiguous float32 {want}")
    with _on(dev):
        _lib.check(_lib.load().kbn_requant_weights_ue8m0(w_fp8.data_ptr(), scale.data_ptr(), e, n, k, eps, _stream(w_fp8)))
    # the scales changed behind torch's version counter: forget any packed copy made from the old values
    for key in [k_ for k_ in _WEIGHT_SF_CACHE if k_[0] == scale.data_ptr()]:
        _WEIGHT_SF_CACHE.pop(key, None)
