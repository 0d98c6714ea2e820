"""ctypes binding of the ahead-of-time built C-ABI library (include/nvfp4_b200.h).

There is no fallback: if `libnvfp4_b200.so` is missing or a call is rejected the caller gets an
exception.  Every call enqueues on `torch.cuda.current_stream()` and returns without synchronising,
like the reference launcher (llm-1b/nvrtc_util.py:53-67).
"""
import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnvfp4_b200.so")

SCALES_SWIZZLED, SCALES_LINEAR = 0, 1
DTYPE_BF16, DTYPE_FP32 = 0, 1
ROUND_NEAREST, ROUND_SR_DITHER, ROUND_SR_DITHER_K, ROUND_SR_HW = 0, 1, 2, 3
ALPHA_ONE, ALPHA_GS, ALPHA_AMAX, ALPHA_ROW = 0, 1, 2, 3

_c = ctypes
_vp, _ll, _i, _u, _f, _sz = _c.c_void_p, _c.c_longlong, _c.c_int, _c.c_uint, _c.c_float, _c.c_size_t

# name -> (restype, argtypes): exactly the declarations of include/nvfp4_b200.h
SIGNATURES = {
    "nvfp4_version": (_i, []),
    "nvfp4_error_string": (_c.c_char_p, [_i]),
    "nvfp4_amax_bf16": (_i, [_vp, _ll, _vp, _vp]),
    "nvfp4_amax_bf16_update": (_i, [_vp, _ll, _vp, _vp]),
    "nvfp4_set_pdl": (_i, [_i]),
    "nvfp4_gemm_reset_scheduler": (_i, []),
    "nvfp4_gemm_set_scheduler": (_i, [_i]),
    "nvfp4_quant_rows": (_i, [_vp, _ll, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _u, _vp, _vp]),
    "nvfp4_quant_cols_rht": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _u, _i, _u, _vp, _vp]),
    "nvfp4_quant_tile": (_i, [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _u, _i, _u, _u, _vp, _vp, _vp]),
    "nvfp4_quant_tile_status": (_i, [_vp, _i]),
    "nvfp4_quant_tile_set_path": (_i, [_i]),
    "nvfp4_rms_emit": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "nvfp4_swiglu_emit": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "nvfp4_mom_acc": (_i, [_vp, _vp, _vp, _f, _ll, _vp, _u, _vp]),
    "nvfp4_emit_rows": (_i, [_vp, _ll, _i, _i, _vp, _vp, _vp, _i, _vp, _u, _vp]),
    "nvfp4_emit_rows_set_path": (_i, [_i]),
    "nvfp4_emit_cols": (_i, [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _u, _vp]),
    "nvfp4_quant_w2d": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp]),
    "nvfp4_e2m1x4_sr": (_i, [_vp, _vp, _vp, _ll, _vp]),
    "nvfp4_swizzle_scales": (_i, [_vp, _ll, _i, _i, _vp, _vp]),
    "nvfp4_gemm": (_i, [_vp, _vp, _ll, _vp, _vp, _ll, _vp, _i, _ll, _i, _i, _i, _i, _vp, _vp, _f, _f, _i, _i, _vp, _vp]),
    "nvfp4_gemm_scatter_rows": (_i, [_vp, _vp, _ll, _vp, _vp, _ll, _vp, _i, _ll, _i, _i, _i, _i, _vp, _vp, _f, _f, _i, _vp, _vp]),
    "nvfp4_gemm_force_tile_n": (_i, [_i]),
    "nvfp4_gemm_set_sm_budget": (_i, [_i]),
    "nvfp4_gemm_linear_workspace_bytes": (_sz, [_i, _i, _i]),
    "nvfp4_gemm_linear": (_i, [_vp, _vp, _ll, _ll, _vp, _vp, _ll, _ll, _vp, _i, _ll, _i, _i, _i, _i, _vp, _vp, _f, _f,
                               _i, _i, _vp, _sz, _vp, _vp]),
    "nvfp4_gemm_linear_noalloc_max_scratch": (_sz, []),
    "nvfp4_selftest_wait_timeout": (_i, [_u, _i, _vp, _vp]),
    "nvfp4_gemm_linear_noalloc": (_i, [_vp, _vp, _ll, _ll, _vp, _vp, _ll, _ll, _vp, _i, _ll, _i, _i, _i, _i, _vp, _vp, _f, _f,
                                       _i, _i, _vp, _vp]),
}

_lib = None


class Nvfp4Error(RuntimeError):
    pass


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Nvfp4Error(f"{LIB_PATH} not found: build it with `python -m nvfp4_training_b200.build` "
                             "(there is no fallback path)")
        # NVFP4_LIB_PATH: load another build of the same library (A/B timing of kernel variants)
        lib = ctypes.CDLL(os.environ.get("NVFP4_LIB_PATH") or LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        # tuning knob: NVFP4_TILE_PATH=1 keeps nvfp4_quant_tile on its scalar kernel
        if os.environ.get("NVFP4_TILE_PATH"):
            lib.nvfp4_quant_tile_set_path(int(os.environ["NVFP4_TILE_PATH"]))
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        msg = load().nvfp4_error_string(rc).decode()
        raise Nvfp4Error(f"{what}: {msg} (status {rc})")


def ptr(t):
    return None if t is None else t.data_ptr()


def ptr_array(addresses):
    """A host array of `void*` for entry points that take one address per rank."""
    return (ctypes.c_void_p * len(addresses))(*[int(a) for a in addresses])


def seed_args(seed):
    """(host seed, device seed pointer): a CUDA int32/uint32 tensor selects the device-side seed."""
    if isinstance(seed, torch.Tensor):
        assert seed.is_cuda and seed.numel() >= 1 and seed.element_size() == 4
        return 0, seed.data_ptr()
    return seed & 0xFFFFFFFF, None


def stream():
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise Nvfp4Error("nvfp4_b200 kernels need CUDA tensors; there is no CPU path")


_status = {}


def status_word(device):
    """Per-device int32 that GEMM CTAs set when a bounded pipeline wait expires (never expected)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


def check_status(device=None):
    """Synchronising check of the status words of the GEMM and of the tile quantizer on `device`;
    raises if any CTA gave up waiting."""
    dev = torch.cuda.current_device() if device is None else device
    code = int(status_word(dev).item())
    if code:
        status_word(dev).zero_()
        with torch.cuda.device(dev):
            load().nvfp4_gemm_reset_scheduler()      # an abandoned launch may have left its work counter half-way
        raise Nvfp4Error(f"GEMM pipeline wait expired (role code {code})")
    qcode = ctypes.c_int(0)
    with torch.cuda.device(dev):
        check(load().nvfp4_quant_tile_status(ctypes.byref(qcode), 1), "quant_tile_status")
    if qcode.value:
        raise Nvfp4Error(f"tile quantizer pipeline wait expired (role code {qcode.value})")
