// Self-test of the bounded-wait abort path shared by the GEMM and the tile quantizer.
//
// Every mbarrier wait in this library gives up after a time limit: the waiting CTA raises its abort
// flag, reports a role code and leaves.  Nothing in a healthy run makes a wait expire, so this entry
// point exists to execute that path once: a single CTA waits on a barrier that nobody ever arrives
// on, with a limit of at most one millisecond and no copies in flight, and writes what it saw.
#include "tma.cuh"

namespace nvfp4 {

__global__ void __launch_bounds__(64) wait_timeout_kernel(int* status, u64 limit_ns, int parked) {
  __shared__ __align__(8) u64 bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const u64 t0 = globaltimer_ns();
  // warp 0 waits with the limit (phase 0 never completes); warp 1 waits with the default limit and
  // must be released by warp 0's abort flag long before that
  const bool ok = warp == 0 ? (parked ? mbar_wait_parked(smem_u32(&bar), 0u, abort_flag, limit_ns)
                                      : mbar_wait(smem_u32(&bar), 0u, abort_flag, limit_ns))
                            : mbar_wait(smem_u32(&bar), 0u, abort_flag);
  const bool all_gave_up = !__any_sync(0xffffffffu, ok);
  const u64 waited = globaltimer_ns() - t0;
  if (lane == 0 && all_gave_up) {
    // bit 0: the limited wait expired, bit 1: the other warp left through the abort flag,
    // bits 8..: microseconds the warp waited (saturated)
    const u64 us = waited / 1000ull;
    atomicOr(status, (warp == 0 ? 1 : 2) | (warp == 0 ? (int)((us > 0xFFFFFull ? 0xFFFFFull : us) << 8) : 0));
  }
}

}  // namespace nvfp4

extern "C" int nvfp4_selftest_wait_timeout(unsigned limit_us, int parked, int* status, void* stream) {
  if (!status) return NVFP4_ERR_NULL;
  if (limit_us == 0 || limit_us > 1000) return NVFP4_ERR_TOO_LARGE;
  nvfp4::wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, (u64)limit_us * 1000ull, parked);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}
