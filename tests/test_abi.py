"""The C-ABI library builds (nvcc cross-compiles for sm_100a without a GPU), loads, and exports every
symbol include/kbn_fp8.h declares; the ctypes binding covers them all.  No compute calls here."""
import ctypes
import os
import re

from kb_nano_b200 import _lib, build

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "kbn_fp8.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kbn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_something():
    syms = declared_symbols()
    assert "kbn_quant_1x128" in syms and "kbn_fp8_gemm_nt" in syms and len(syms) >= 8


def test_library_builds_and_exports_every_declared_symbol(kbn_lib):
    assert os.path.exists(build.LIB_PATH)
    raw = ctypes.CDLL(build.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(raw, s), f"{s} declared in include/kbn_fp8.h but not exported"


def test_ctypes_binding_covers_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_error_string(kbn_lib):
    assert kbn_lib.kbn_version() >= 1
    assert isinstance(kbn_lib.kbn_last_error(), bytes)


def test_argument_validation_needs_no_gpu(kbn_lib):
    # rejected before any CUDA call: null pointers, bad shapes
    rc = kbn_lib.kbn_quant_1x128(None, 4, 128, 128, None, 128, None, 1, 1, 1e-10, 1, None)
    assert rc == -1 and b"null" in kbn_lib.kbn_last_error()
    rc = kbn_lib.kbn_silu_mul_quant_1x128(1024, 4, 100, 200, 2048, 100, 4096, 1, 4, 1e-10, 1, None)
    assert rc == -1 and b"multiple of 128" in kbn_lib.kbn_last_error()
    rc = kbn_lib.kbn_quant_1x128(None, 0, 128, 128, None, 128, None, 1, 1, 1e-10, 1, None)
    assert rc == 0   # empty input is a no-op


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from kb_nano_b200 import ops
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.per_token_group_quant_fp8(x, torch.empty(4, 128, dtype=torch.float8_e4m3fn), torch.empty(4, 1))
