"""ctypes binding of libkbn_fp8.so (the C ABI declared in include/kbn_fp8.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os


_i64 = ctypes.c_int64
_i32 = ctypes.c_int
_f32 = ctypes.c_float
_ptr = ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol include/kbn_fp8.h declares
SIGNATURES = {
    "kbn_version": (_i32, []),
    "kbn_last_error": (ctypes.c_char_p, []),
    "kbn_launch_count": (_i64, []),
    "kbn_quant_1x128": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _i32, _ptr]),
    "kbn_quant_1x128_sf": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _ptr, _ptr]),
    "kbn_silu_mul_quant_1x128": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _i32, _ptr]),
    "kbn_silu_bf16_table": (_i32, [_ptr, _ptr]),
    "kbn_rmsnorm_quant_1x128": (_i32, [_ptr, _ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _ptr]),
    "kbn_add_rmsnorm_quant_1x128": (_i32, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _ptr]),
    "kbn_silu_mul_quant_1x128_rows": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _i32, _ptr, _ptr]),
    "kbn_silu_mul_quant_1x128_list": (_i32, [_ptr, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _f32, _i32, _ptr, _i64, _ptr, _ptr]),
    "kbn_silu_mul_quant_1x128_masked": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr]),
    "kbn_fp8_gemm_nt": (_i32, [_ptr, _ptr, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_contig": (_i32, [_ptr, _ptr, _i64, _i64, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_masked": (_i32, [_ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_gemm_status": (_i32, [_ptr, _ptr]),
    "kbn_gemm_clear_status": (_i32, [_ptr]),
    "kbn_requant_weights_ue8m0": (_i32, [_ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "kbn_packed_sf_rows_bytes": (_i64, [_i64, _i64]),
    "kbn_packed_sf_weights_bytes": (_i64, [_i64, _i64, _i64]),
    "kbn_pack_sf_rows": (_i32, [_ptr, _i64, _i64, _i64, _i64, _ptr, _ptr]),
    "kbn_pack_sf_weights": (_i32, [_ptr, _i64, _i64, _i64, _ptr, _ptr]),
    "kbn_count_non_pow2_scales": (_i32, [_ptr, _i64, _ptr, _ptr]),
    "kbn_fp8_gemm_nt_ue8m0": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_contig_ue8m0": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_masked_ue8m0": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_contig_ue8m0_silu": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_fp8_grouped_gemm_masked_ue8m0_silu": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "kbn_moe_aligned_rows": (_i64, [_i64, _i64, _i64]),
    "kbn_moe_permute_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "kbn_moe_pair_experts": (_i32, [_ptr, _i64, _ptr, _i64, _i64, _i64, _ptr, _ptr]),
    "kbn_moe_permute": (_i32, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr]),
    "kbn_moe_permute_sf": (_i32, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr]),
    "kbn_ep_create": (_i32, [_i32, _i32, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.POINTER(_ptr)]),
    "kbn_ep_ipc_handle": (_i32, [_ptr, _ptr]),
    "kbn_ep_attach": (_i32, [_ptr, _ptr]),
    "kbn_ep_symmetric_bytes": (_i64, [_ptr]),
    "kbn_ep_moe_forward": (_i32, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "kbn_ep_moe_forward_routed": (_i32, [_ptr, _ptr, _ptr, _i32, _i64, _i64, _i32, _ptr, _i64, _i64, _i32, _f32, _f32, _i32, _ptr, _ptr, _ptr, _ptr,
                                         _ptr, _ptr, _ptr, _ptr]),
    "kbn_ep_last_routing": (_i32, [_ptr, _ptr, _ptr, _i64, _ptr]),
    "kbn_ep_status": (_i32, [_ptr, _ptr, _ptr]),
    "kbn_ep_clear_status": (_i32, [_ptr, _ptr]),
    "kbn_ep_expert_phase": (_i32, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _ptr]),
    "kbn_ep_destroy": (_i32, [_ptr]),
    "kbn_moe_route_topk": (_i32, [_ptr, _i32, _i64, _i64, _i64, _i32, _ptr, _i64, _i64, _i64, _i32, _f32, _f32, _i32, _ptr, _ptr, _ptr]),
    "kbn_moe_permute_static": (_i32, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr]),
    "kbn_moe_unpermute_combine": (_i32, [_ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr]),
}

_lib = None


class KbnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"kbn_fp8 error {code}: {message}")
        self.code = code


LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libkbn_fp8.so")


def lib_path() -> str:
    return LIB_PATH


def load(build_if_missing: bool = False) -> ctypes.CDLL:
    """Load the library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        if build_if_missing:
            from . import build as _build
            _build.build()
        else:
            raise RuntimeError(
                f"{path} is missing: run `python -m kb_nano_b200.build` (there is no CPU or torch fallback)")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        raise KbnError(code, load().kbn_last_error().decode("utf-8", "replace"))


def launch_count() -> int:
    return int(load().kbn_launch_count())
