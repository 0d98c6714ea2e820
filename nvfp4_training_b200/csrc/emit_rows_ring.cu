// Row-operand emitter with an exact per-row FP32 scale, TMA-fed (sm_100a): x [T, C] bf16 -> codes, swizzled
// block scales and rs[t] = rowmax / 2688 from ONE read of x, with no tensor-wide amax pass.
//
// A per-row scale needs the whole row before the first code can be written.  The warp-per-row kernel
// (emit_ops.cu) keeps the row in registers, so its loads in flight are bounded by registers and occupancy.  Here
// whole rows travel through a shared-memory ring: one warp issues a bulk copy per row (cp.async.bulk, the row is
// contiguous: up to 23 KB each, 8 or 16 rows in flight per SM) and eight consumer warps each own every eighth row:
// pass 1 reads the row's 16-value blocks from shared memory and keeps their maxima (a lane per block, packed bf16
// max), the row maximum is a warp reduction, pass 2 re-reads the blocks from shared memory, scales, rounds and
// stores 8 bytes of codes per lane (256 contiguous bytes per warp) and the scale byte.
// Arithmetic and random sequences are those of emit_ops.cu, bit for bit (the reference's `row_emit` /
// `row_emit_11264`, llm-1b/emit.cu:228-285); a third rounding mode uses the hardware stochastic convert with this
// library's counter-based words.
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, records a role code and returns.
#include "tma.cuh"

namespace nvfp4 {

constexpr int kRingWarps = 8;
constexpr int kRingThreads = 32 * (1 + kRingWarps);
constexpr int kRingMaxSlots = 16;
constexpr int kRingMaxCols = 11776;                         // 8 rows of 23 KB + the block-maxima scratch fit in shared memory
constexpr int kRingScratchFloats = kRingMaxCols / 16;       // block maxima of one row

__device__ int g_emit_ring_status;    // 0, or 1 (producer) / 2 (consumer) whose wait expired first

struct RingParams {
  const __nv_bfloat16* x; long long ldx;
  uint2* codes; unsigned char* scales; float* rs_out;
  const u32* rng; u32 salt;
  int T, C, slots;
};

// max |.| of both halves of packed bf16 words: |max| with the sign bits xor-ed (ignored later)
__device__ __forceinline__ u32 absmax_bf16x2(u32 a, u32 b) {
  u32 d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// MODE 0: round to nearest; 1: the reference's 11-bit mantissa dither with its per-lane LCG sequences;
// 2: hardware cvt.rs with the counter-based words of this library (key from rng[0] ^ salt and the block index).
// SUBS = 4: the four-sequence stream of the reference's 11264-column kernel (MODE 1 only).
template <int MODE, int SUBS>
__global__ void __launch_bounds__(kRingThreads, 1) emit_rows_ring_kernel(const RingParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) u64 bars[2 * kRingMaxSlots];
  __shared__ __align__(8) float2 lut[128];                // {dec(sb), RN(1/dec(sb))}, entry 0 = {0, 0}
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const u32 row_bytes = (u32)p.C * 2u;
  const u32 ring0 = (smem_u32(smem_raw) + 127u) & ~127u;
  const u32 scratch0 = ring0 + (u32)p.slots * row_bytes;  // [kRingWarps][kRingScratchFloats] floats
  const u32 full0 = smem_u32(bars), empty0 = full0 + 8 * kRingMaxSlots;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < p.slots; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 128) {
    const float sd = e4m3_dec(threadIdx.x);
    lut[threadIdx.x] = (threadIdx.x >= 1 && threadIdx.x <= 126) ? make_float2(sd, __frcp_rn(sd)) : make_float2(0.f, 0.f);
  }
  __syncthreads();
  const long long first = blockIdx.x, stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: one bulk copy per row
    u32 i = 0;
    for (long long r = first; r < p.T; r += stride, i++) {
      const u32 slot = i % (u32)p.slots, par = (i / (u32)p.slots) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait_parked(empty0 + 8 * slot, par ^ 1u, abort_flag))) {
        if (lane == 0) atomicCAS(&g_emit_ring_status, 0, 1);
        break;
      }
      if (elect_one()) {
        mbar_arrive_expect_tx(full0 + 8 * slot, row_bytes);
        bulk_load(ring0 + slot * row_bytes, p.x + r * p.ldx, row_bytes, full0 + 8 * slot);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ consumers: warp w owns rows w-1, w+7, ...
    const int cw = warp - 1;
    const int nblk = p.C >> 4;
    const int nj = (nblk + 31) >> 5;
    const u32 scratch = scratch0 + (u32)cw * (kRingScratchFloats * 4u);
    const u32 seed = (MODE != 0 ? __ldg(p.rng) : 0u) ^ p.salt;
    u32 i = (u32)cw;
    for (long long r = first + (long long)cw * stride; r < p.T; r += kRingWarps * stride, i += kRingWarps) {
      const u32 slot = i % (u32)p.slots, par = (i / (u32)p.slots) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait_parked(full0 + 8 * slot, par, abort_flag))) {
        if (lane == 0) atomicCAS(&g_emit_ring_status, 0, 2);
        break;
      }
      const u32 row = ring0 + slot * row_bytes;
      // ---- pass 1: block maxima (lane = block 32 j + lane), kept in this warp's scratch; row maximum
      u32 rowmax = 0u;
      for (int j = 0; j < nj; j++) {
        const int b = j * 32 + lane;
        if (b < nblk) {
          u32 w[8];
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(row + (u32)b * 32u));
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(row + (u32)b * 32u + 16u));
          u32 m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(w[0], w[1]), absmax_bf16x2(w[2], w[3])),
                                absmax_bf16x2(absmax_bf16x2(w[4], w[5]), absmax_bf16x2(w[6], w[7])));
          m = max(m & 0x7FFFu, (m >> 16) & 0x7FFFu);            // bf16 magnitudes order like integers
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(scratch + (u32)b * 4u), "r"(m << 16) : "memory");
          rowmax = max(rowmax, m);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) rowmax = max(rowmax, __shfl_xor_sync(0xffffffffu, rowmax, o));
      const float am = __uint_as_float(rowmax << 16);
      const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
      const bool huge = !(inv < 1e35f);       // rows of magnitude below 1e-31: inv * (1/scale) would overflow, divide instead
      if (lane == 0) p.rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
      // ---- random sequences of the dither mode.  The reference's lane l = (column / 8) % 32 walks its 8-column
      // chunks j = column / 256 in order, four LCG steps per chunk.  Here a lane owns 16 columns, i.e. the chunks of
      // reference lanes l0 = (2 lane) % 32 and l0 + 1 with j = 2 jj + (lane >= 16): after its four steps a sequence
      // skips the four steps of the chunk the other half-warp handles.  SUBS = 4: sequence s = j % 4 is seeded with
      // r*128 + s*32 + l and takes only its own chunks, so a lane alternates between two sequences per reference lane.
      u32 st[2][SUBS == 4 ? 2 : 1];
      if (MODE == 1) {
        const u32 l0 = (u32)(2 * lane) & 31u, hi = (u32)lane >> 4;
#pragma unroll
        for (int e = 0; e < 2; e++) {
          if (SUBS == 4) {
            st[e][0] = hash32(seed ^ hash32((u32)r * 128u + hi * 32u + l0 + e));
            st[e][1] = hash32(seed ^ hash32((u32)r * 128u + (hi + 2u) * 32u + l0 + e));
          } else {
            const u32 s0 = hash32(seed ^ hash32((u32)r * 32u + l0 + e));
            st[e][0] = hi ? s0 * lcg_jump_mul(4) + lcg_jump_add(4) : s0;
          }
        }
      }
      __syncwarp();
      // ---- pass 2: scale, round, store
      for (int j = 0; j < nj; j++) {
        const int b = j * 32 + lane;
        if (b < nblk) {
          u32 w[8]; u32 mbits;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(row + (u32)b * 32u));
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(row + (u32)b * 32u + 16u));
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(mbits) : "r"(scratch + (u32)b * 4u));
          const u32 sb = e4m3_enc(__fmul_rn(__fmul_rn(__uint_as_float(mbits), inv), 1.f / 6.f));
          const float2 e = lut[sb];
          // k = inv / dec(sb) correctly rounded (the scale has at most 4 significant bits), 0 for a zero scale
          const float q0 = __fmul_rn(inv, e.y);
          float k = __fmaf_rn(__fmaf_rn(-q0, e.x, inv), e.y, q0);
          if (huge) k = e.x > 0.f ? __fdiv_rn(inv, e.x) : 0.f;
          const u64 K = f2_pack(k, k);
          float y[16];
#pragma unroll
          for (int t = 0; t < 8; t++) {
            const u64 v = f2_mul(f2_from_bf16x2(w[t]), K);
            y[2 * t] = f2_lo(v); y[2 * t + 1] = f2_hi(v);
          }
          uint2 out;
          if (MODE == 1) {
            const int which = SUBS == 4 ? (j & 1) : 0;
#pragma unroll
            for (int e2 = 0; e2 < 2; e2++) {
              u32 s = (SUBS == 4 && which) ? st[e2][SUBS == 4 ? 1 : 0] : st[e2][0];
#pragma unroll
              for (int t = 0; t < 8; t += 2) {
                const u32 rnd = lcg_step(s);
                y[8 * e2 + t] = sr_dither11(y[8 * e2 + t], (rnd << 11) & 0x3FF800u);
                y[8 * e2 + t + 1] = sr_dither11(y[8 * e2 + t + 1], (rnd >> 5) & 0x3FF800u);
              }
              if (SUBS == 4) { if (which) st[e2][SUBS == 4 ? 1 : 0] = s; else st[e2][0] = s; }
              else st[e2][0] = s * lcg_jump_mul(4) + lcg_jump_add(4);
            }
            out = make_uint2(e2m1x8_rn(y), e2m1x8_rn(y + 8));
          } else if (MODE == 2) {
            u32 key = sr_hw_block_key(seed, (u32)(r * nblk + b));
            float (&y0)[8] = *reinterpret_cast<float(*)[8]>(&y[0]);
            float (&y1)[8] = *reinterpret_cast<float(*)[8]>(&y[8]);
            out.x = round8<NVFP4_ROUND_SR_HW>(y0, key, seed, 0u, 0);
            out.y = round8<NVFP4_ROUND_SR_HW>(y1, key, seed, 0u, 1);
          } else {
            out = make_uint2(e2m1x8_rn(y), e2m1x8_rn(y + 8));
          }
          p.codes[r * nblk + b] = out;
          p.scales[sw_off(r, b, nblk >> 2)] = (unsigned char)sb;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * slot);
    }
  }
  __syncwarp();
  if (*abort_flag) {
    // let a bulk copy that is still in flight land before shared memory is released
    const u64 t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

template <int MODE, int SUBS>
static int launch_ring(const RingParams& p, int grid, size_t smem, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(emit_rows_ring_kernel<MODE, SUBS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 128) != cudaSuccess)
      return NVFP4_ERR_CUDA;
    configured[dev] = true;
  }
  emit_rows_ring_kernel<MODE, SUBS><<<grid, kRingThreads, smem, st>>>(p);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

}  // namespace nvfp4

using namespace nvfp4;

int nvfp4_sm_budget_value();   // gemm.cu: nvfp4_gemm_set_sm_budget

// Whether the ring kernel takes this call (otherwise the warp-per-row kernel of emit_ops.cu runs).
bool nvfp4_emit_rows_ring_accepts(const void* x, long long ldx, int T, int C, const void* codes) {
  if (T <= 0 || C <= 0 || (C & 255) || C > kRingMaxCols || ldx < C) return false;
  return !((reinterpret_cast<uintptr_t>(x) & 15u) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes) & 7u));
}

// Arguments as nvfp4_emit_rows, already validated by it.  sr: 0 nearest, 1 reference dither, 2 hardware convert.
int nvfp4_emit_rows_ring_launch(const void* x, long long ldx, int T, int C, void* codes, void* scales, float* rs_out,
                                int sr, const unsigned* rng, unsigned salt, void* stream) {
  RingParams p;
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx;
  p.codes = static_cast<uint2*>(codes); p.scales = static_cast<unsigned char*>(scales); p.rs_out = rs_out;
  p.rng = rng; p.salt = salt; p.T = T; p.C = C;
  const size_t row_bytes = (size_t)C * 2;
  const size_t budget = 200 * 1024 - (size_t)kRingWarps * kRingScratchFloats * 4;
  int slots = (int)(budget / row_bytes);
  slots = slots >= kRingMaxSlots ? kRingMaxSlots : (slots / kRingWarps) * kRingWarps;     // a slot always serves the same warp
  if (slots < kRingWarps) return NVFP4_ERR_TOO_LARGE;
  p.slots = slots;
  const size_t smem = (size_t)slots * row_bytes + (size_t)kRingWarps * kRingScratchFloats * 4 + 128;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
  }
  { const int b = nvfp4_sm_budget_value(); if (b > 0 && b < sms) sms = b; }   // SMs left to a collective running beside this kernel
  int grid = sms;
  if (T < grid * kRingWarps) grid = (T + kRingWarps - 1) / kRingWarps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (sr == 0) return launch_ring<0, 1>(p, grid, smem, st);
  if (sr == 2) return launch_ring<2, 1>(p, grid, smem, st);
  if (C == 11264) return launch_ring<1, 4>(p, grid, smem, st);
  return launch_ring<1, 1>(p, grid, smem, st);
}

int nvfp4_emit_rows_ring_status(int* out, int reset) {
  if (cudaMemcpyFromSymbol(out, g_emit_ring_status, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (reset) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_emit_ring_status, &zero, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  }
  return NVFP4_OK;
}
