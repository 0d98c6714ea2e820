// mbarrier / TMA wrappers and the tensor-map encoder shared by the GEMM and the tile quantizer.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace nvfp4 {

constexpr u64 kWaitLimitNs = 1000000000ull;   // 1 s per wait, far above any legitimate wait

__device__ __forceinline__ u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(u32 bar, u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(u32 bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u32 bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ u32 mbar_try_wait(u32 bar, u32 parity) {
  u32 ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ u64 globaltimer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one expired).
__device__ __forceinline__ bool mbar_wait(u32 bar, u32 parity, volatile int* abort_flag, u64 limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const u64 t0 = globaltimer_ns();
  for (u32 it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 127u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) { *abort_flag = 1; return false; }
    }
  }
}

// Bounded wait for warps that can afford to sleep: the try_wait carries a suspend-time hint, so a
// waiting warp polls rarely instead of competing for issue slots with the warps that have work.
__device__ __forceinline__ bool mbar_wait_parked(u32 bar, u32 parity, volatile int* abort_flag, u64 limit_ns = kWaitLimitNs) {
  u64 t0 = 0;
  for (u32 it = 1;; ++it) {
    u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    if (ok) return true;
    if ((it & 15u) == 0u) {
      if (*abort_flag) return false;
      const u64 now = globaltimer_ns();      // the clock is read only once a wait has lasted a while
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) { *abort_flag = 1; return false; }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(u32 dst, const CUtensorMap* map, int x, int y, u32 bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(u32 dst, const void* src, u32 bytes, u32 bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  u32 pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0u;
}

// ---------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

}  // namespace nvfp4
