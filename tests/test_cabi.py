"""CPU-side checks of the C-ABI boundary: the built library loads, exports every function that
include/nvfp4_b200.h declares, and rejects malformed calls before touching the device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nvfp4_b200.h")


@pytest.fixture(scope="module")
def lib():
    from nvfp4_training_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", src)))


def test_header_functions_are_exported_and_bound(lib):
    from nvfp4_training_b200 import _lib
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_strings(lib):
    assert lib.nvfp4_version() >= 100
    for code in range(0, -8, -1):
        assert lib.nvfp4_error_string(code)
    assert lib.nvfp4_error_string(-99) == b"unknown status"


def test_argument_validation_needs_no_device(lib):
    # null pointers, bad shapes, bad enums: all rejected before any CUDA call
    assert lib.nvfp4_amax_bf16(None, 8, None, None) == -1
    assert lib.nvfp4_amax_bf16(ctypes.c_void_p(16), 12, ctypes.c_void_p(16), None) == -2
    assert lib.nvfp4_quant_rows(None, 64, 128, 64, None, None, 0, None, None, 0, 0, None, None) == -1
    p = ctypes.c_void_p(1 << 20)
    assert lib.nvfp4_quant_rows(p, 64, 100, 64, p, p, 0, p, None, 0, 0, None, None) == -2
    assert lib.nvfp4_quant_rows(p, 64, 128, 64, p, p, 0, p, None, 9, 0, None, None) == -4
    assert lib.nvfp4_quant_cols_rht(p, 64, 100, p, p, 0, p, None, 0, 0, 0, None, None) == -2
    assert lib.nvfp4_quant_w2d(p, 5, 128, 128, p, p, p, p, 0, p, None, None) == -4
    assert lib.nvfp4_gemm(p, p, 64, p, p, 64, p, 1, 128, 128, 128, 100, 0, None, None, 1.0, 1.0, 0, 1, None, None) == -2
    assert lib.nvfp4_gemm_linear(p, p, 64, 8, p, p, 64, 8, p, 1, 128, 128, 128, 128, 0, None, None, 1.0, 1.0, 0, 1,
                                 None, 0, None, None) == -6
    # weight-gradient GEMM that adds row slabs into their owners: one address per rank, whole 128-row tiles per owner
    own = lambda *a: (ctypes.c_void_p * len(a))(*a)
    sc = lambda arr, n, M: lib.nvfp4_gemm_scatter_rows(p, p, 64, p, p, 64, arr, n, 128, M, 128, 128, 0, None, None, 1.0, 1.0, 1,
                                                       None, None)
    assert sc(None, 2, 512) == -1
    assert sc(own(1 << 20, 1 << 21), 2, 384) == -2            # M % 256
    assert sc(own(1 << 20, 1 << 21, 1 << 22, 1 << 23), 4, 768) == -2          # 192 rows per owner
    assert sc(own(*[1 << 20] * 9), 9, 2304) == -2              # more than 8 owners
    assert sc(own(1 << 20, None), 2, 512) == -1
    assert sc(own(1 << 20, (1 << 21) + 8), 2, 512) == -3
    # tile quantizer and operand emitters
    assert lib.nvfp4_quant_tile(p, 128, 128, 128, None, None, None, None, 0, p, None, None, 0, 0, 0, 0, None, None, None) == -1
    assert lib.nvfp4_quant_tile(p, 128, 100, 128, p, p, p, p, 0, p, None, None, 0, 0, 0, 0, None, None, None) == -2
    assert lib.nvfp4_quant_tile(p, 192, 128, 192, p, p, p, p, 0, p, None, None, 0, 0, 0, 0, None, None, None) == -2   # swizzled: C % 128
    assert lib.nvfp4_quant_tile(p, 128, 128, 128, p, p, p, p, 0, p, None, None, 0, 7, 0, 0, None, None, None) == -4
    assert lib.nvfp4_quant_tile(ctypes.c_void_p((1 << 20) + 4), 128, 128, 128, p, p, p, p, 0, p, None, None, 0, 0, 0, 0,
                                None, None, None) == -3
    assert lib.nvfp4_quant_tile_status(None, 0) == -1
    assert lib.nvfp4_quant_tile_set_path(3) == -4 and lib.nvfp4_quant_tile_set_path(2) == 0 and lib.nvfp4_quant_tile_set_path(0) == 0
    assert lib.nvfp4_emit_rows(p, 384, 128, 384, p, p, p, 0, None, 0, None) == -2          # C % 256
    assert lib.nvfp4_emit_rows(p, 256, 128, 256, p, p, p, 1, None, 0, None) == -1          # SR needs the device seed
    assert lib.nvfp4_emit_rows(p, 256, 128, 256, p, p, None, 0, None, 0, None) == -1
    assert lib.nvfp4_emit_rows(p, 256, 128, 256, p, p, p, 3, p, 0, None) == -4            # rounding mode 0, 1 or 2
    assert lib.nvfp4_emit_rows_set_path(2) == -4 and lib.nvfp4_emit_rows_set_path(1) == 0 and lib.nvfp4_emit_rows_set_path(0) == 0
    assert lib.nvfp4_emit_cols(p, 128, 128, 128, p, p, p, p, 0, None, 0, None) == -1       # rng carries the sign bits
    assert lib.nvfp4_emit_cols(p, 192, 128, 192, p, p, p, p, 0, p, 0, None) == -2          # C % 128
    assert lib.nvfp4_emit_cols(p, 128, 64, 128, p, p, p, p, 0, p, 0, None) == -2           # M % 128
    assert lib.nvfp4_gemm_linear_workspace_bytes(128, 256, 1024) == (128 + 256) * 64
    assert lib.nvfp4_gemm_force_tile_n(64) == -4 and lib.nvfp4_gemm_force_tile_n(448) == 0 and lib.nvfp4_gemm_force_tile_n(0) == 0
    # an SM budget of one SM cannot hold a CTA pair; negative budgets are refused too
    assert lib.nvfp4_gemm_set_sm_budget(1) == -2 and lib.nvfp4_gemm_set_sm_budget(-4) == -2
    assert lib.nvfp4_gemm_set_sm_budget(2) == 0 and lib.nvfp4_gemm_set_sm_budget(0) == 0
    # the wait self-test accepts 1..1000 microseconds only
    assert lib.nvfp4_selftest_wait_timeout(100, 0, None, None) == -1
    assert lib.nvfp4_selftest_wait_timeout(0, 0, p, None) == -7
    assert lib.nvfp4_selftest_wait_timeout(5000, 0, p, None) == -7


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from nvfp4_training_b200 import _lib, fp4ops, nvq
    x = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises(_lib.Nvfp4Error):
        nvq.quant_rows(x)
    with pytest.raises(_lib.Nvfp4Error):
        fp4ops.quant_rows(x, amax=torch.ones(1))


def test_missing_library_fails_loudly(monkeypatch):
    from nvfp4_training_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(_lib.Nvfp4Error):
        _lib.load()
