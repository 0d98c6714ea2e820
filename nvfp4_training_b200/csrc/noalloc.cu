// Allocation-free variant of the linear-scale GEMM entry point.
//
// nvfp4_gemm_linear needs a scratch buffer for the re-swizzled scale bytes and makes its caller
// provide one.  Some callers have no way to get device memory at call time: a plugin loaded into a
// process whose framework has already reserved all of the GPU's memory in its own pool, a
// latency-critical loop that must not take the driver's allocator lock (cudaMalloc synchronises the
// whole device), or host code that is only handed input and output pointers.  For them the scratch
// lives here, in a fixed array that is part of the library image.
#include "common.cuh"

#define NVFP4_NOALLOC_SCRATCH_BYTES (8u << 20)

// Resident in every GPU context that loads the library, from load until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NVFP4_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address, so the
// address is looked up once per device (with that device current) and kept.
static void* g_scratch_addr[64] = {nullptr};

extern "C" size_t nvfp4_gemm_linear_noalloc_max_scratch(void) { return NVFP4_NOALLOC_SCRATCH_BYTES; }

extern "C" int nvfp4_gemm_linear_noalloc(const void* a, const void* sa, long long lda, long long ldsa, const void* b,
                                         const void* sb, long long ldb, long long ldsb, void* c, int c_dtype, long long ldc,
                                         int M, int N, int K, int alpha_mode, const float* pa, const float* pb, float ka,
                                         float kb, int accumulate, int splitk, int* status, void* stream) {
  if (M < 0 || N < 0 || K < 0) return NVFP4_ERR_SHAPE;
  const size_t need = nvfp4_gemm_linear_workspace_bytes(M, N, K);
  if (need > NVFP4_NOALLOC_SCRATCH_BYTES) return NVFP4_ERR_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_ERR_CUDA;
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return NVFP4_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  return nvfp4_gemm_linear(a, sa, lda, ldsa, b, sb, ldb, ldsb, c, c_dtype, ldc, M, N, K, alpha_mode, pa, pb, ka, kb,
                           accumulate, splitk, g_scratch_addr[dev], NVFP4_NOALLOC_SCRATCH_BYTES, status, stream);
}
