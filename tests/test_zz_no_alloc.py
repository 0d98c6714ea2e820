"""The allocation-free GEMM entry point (nvfp4_gemm_linear_noalloc), called through the C ABI.

It serves callers that cannot get device memory when they call -- a plugin inside a process whose
framework owns all GPU memory, a loop that must not take the driver's allocator lock -- by keeping
its scratch in a fixed array inside the library.  The check: two calls in a row give the same
result as nvfp4_gemm_linear with a caller-provided workspace, and oversize problems are refused.
This file sorts last on purpose, so a run that stops at the first failure has run everything else.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(seed, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda r: (torch.randint(0, 256, (r, K // 2), generator=g, device="cuda", dtype=torch.uint8),
                    torch.randint(0x30, 0x40, (r, K // 16), generator=g, device="cuda", dtype=torch.uint8))
    return mk(M), mk(N), torch.tensor([3.0], device="cuda"), torch.tensor([0.5], device="cuda")


def test_noalloc_matches_workspace_entry_point_twice():
    from nvfp4_training_b200 import _lib as L
    lib = L.load()
    st = L.stream()
    shapes = [(256, 384, 1024), (128, 512, 4096)]
    cases = []
    for seed, (M, N, K) in enumerate(shapes):
        (a, sa), (b, sb), pa, pb = _operands(seed, M, N, K)
        ref = torch.zeros(M, N, device="cuda")
        ws = torch.empty(lib.nvfp4_gemm_linear_workspace_bytes(M, N, K), dtype=torch.uint8, device="cuda")
        L.check(lib.nvfp4_gemm_linear(a.data_ptr(), sa.data_ptr(), K // 2, K // 16, b.data_ptr(), sb.data_ptr(), K // 2,
                                      K // 16, ref.data_ptr(), L.DTYPE_FP32, N, M, N, K, L.ALPHA_AMAX, pa.data_ptr(),
                                      pb.data_ptr(), 1.0, 4.0, 0, 1, ws.data_ptr(), ws.numel(), None, st), "ref")
        cases.append((M, N, K, a, sa, b, sb, pa, pb, ref, torch.zeros(M, N, device="cuda")))
    # two calls in a row on the shared scratch: the second must not see anything of the first
    for M, N, K, a, sa, b, sb, pa, pb, ref, out in cases:
        L.check(lib.nvfp4_gemm_linear_noalloc(a.data_ptr(), sa.data_ptr(), K // 2, K // 16, b.data_ptr(), sb.data_ptr(),
                                              K // 2, K // 16, out.data_ptr(), L.DTYPE_FP32, N, M, N, K, L.ALPHA_AMAX,
                                              pa.data_ptr(), pb.data_ptr(), 1.0, 4.0, 0, 1, None, st), "noalloc")
    torch.cuda.synchronize()
    # The claim itself: once every kernel variant these shapes select has been launched (above), further
    # calls take no device memory -- neither from the driver (free memory as cudaMemGetInfo reports it
    # does not drop) nor from torch's caching allocator.
    free0 = torch.cuda.mem_get_info()[0]
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(2):
        for M, N, K, a, sa, b, sb, pa, pb, ref, out in cases:
            L.check(lib.nvfp4_gemm_linear_noalloc(a.data_ptr(), sa.data_ptr(), K // 2, K // 16, b.data_ptr(), sb.data_ptr(),
                                                  K // 2, K // 16, out.data_ptr(), L.DTYPE_FP32, N, M, N, K, L.ALPHA_AMAX,
                                                  pa.data_ptr(), pb.data_ptr(), 1.0, 4.0, 0, 1, None, st), "noalloc")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (alloc0, reserved0)
    for M, N, K, a, sa, b, sb, pa, pb, ref, out in cases:
        r, o = ref.cpu().numpy().astype(np.float64), out.cpu().numpy().astype(np.float64)
        assert np.isfinite(o).all() and np.abs(r).max() > 0
        # tolerance of the FP32 GEMM tests: 1e-5 relative Frobenius, 1e-4 |Y| + 1e-6 max|Y| per element
        assert np.linalg.norm(o - r) <= 1e-5 * np.linalg.norm(r)
        assert (np.abs(o - r) <= 1e-4 * np.abs(r) + 1e-6 * np.abs(r).max()).all()


def test_noalloc_rejects_oversize():
    from nvfp4_training_b200 import _lib as L
    lib = L.load()
    limit = lib.nvfp4_gemm_linear_noalloc_max_scratch()
    assert limit == 8 << 20
    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    M, N, K = 65536, 65536, 4096                     # (M + N) * K / 16 = 32 MiB > 8 MiB
    rc = lib.nvfp4_gemm_linear_noalloc(p, p, K // 2, K // 16, p, p, K // 2, K // 16, p, L.DTYPE_FP32, N, M, N, K,
                                       L.ALPHA_ONE, None, None, 1.0, 1.0, 0, 1, None, L.stream())
    assert rc == -7
    assert b"maximum" in lib.nvfp4_error_string(rc)
