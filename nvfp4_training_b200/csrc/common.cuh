// Shared device helpers for the NVFP4 quantizers and the block-scaled GEMM (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/nvfp4_b200.h"

typedef uint32_t u32;
typedef uint64_t u64;

#define NVFP4_LAUNCH_CHECK()                                   \
  do {                                                         \
    if (cudaPeekAtLastError() != cudaSuccess) {                \
      (void)cudaGetLastError();                                \
      return NVFP4_ERR_CUDA;                                   \
    }                                                          \
  } while (0)

namespace nvfp4 {

constexpr float kFp4E4m3 = 2688.0f;   // 6 * 448
constexpr float kTiny = 1e-30f;

// 32-bit mixer shared with the reference's random streams (llm-1b/nvq.cu:13-15).
__device__ __forceinline__ u32 hash32(u32 x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

// non-negative f32 -> E4M3 byte, round to nearest even, saturating at 448
__device__ __forceinline__ u32 e4m3_enc(float s) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(s));
  return r & 0xFFu;
}

__device__ __forceinline__ float e4m3_dec(u32 b) {
  unsigned short h = (unsigned short)b;
  u32 r;
  asm("{.reg .b32 t; cvt.rn.f16x2.e4m3x2 t, %1; mov.b32 %0, t;}" : "=r"(r) : "h"(h));
  return __low2float(*reinterpret_cast<__half2*>(&r));
}

// two f32 -> one byte of E2M1 codes, `lo` in the low nibble; RN-even, saturating, sign kept on zero
__device__ __forceinline__ u32 e2m1x2_rn(float lo, float hi) {
  unsigned short r;
  asm("{.reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t;}" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// four f32 -> 16 bits of E2M1 codes with hardware stochastic rounding; v0 lands in the lowest nibble
// and consumes byte 0 of rbits, v3 the highest nibble and byte 3.
__device__ __forceinline__ u32 e2m1x4_rs(float v0, float v1, float v2, float v3, u32 rbits) {
  unsigned short r;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(v3), "f"(v2), "f"(v1), "f"(v0), "r"(rbits));
  return r;
}

// Stochastic rounding onto the E2M1 grid by adding 22 random bits below the kept mantissa bit
// and truncating (the reference's method, llm-1b/nvq.cu:32-39).  The result is exactly
// representable, so the round-to-nearest convert that follows is exact.
__device__ __forceinline__ float sr_dither(float v, u32 rnd) {
  float a = fminf(fabsf(v), 6.f);
  bool sub = a < 1.f;
  float b = sub ? __fadd_rn(a, 1.f) : a;
  u32 bits = (__float_as_uint(b) + (rnd & 0x3FFFFFu)) & ~0x3FFFFFu;
  float r = __fsub_rn(__uint_as_float(bits), sub ? 1.f : 0.f);
  return copysignf(fminf(r, 6.f), v);
}

// byte offset of the scale of (row r, 16-block c) in the swizzled layout; ncb = (C/16)/4
__device__ __forceinline__ long long sw_off(long long r, int c, int ncb) {
  return ((r >> 7) * ncb + (c >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

__device__ __forceinline__ float tensor_scale(float amax, float k) {
  return fmaxf(__fdiv_rn(amax * k, kFp4E4m3), kTiny);
}

// Quantize one block of 16 values that share a scale.
//   v      the 16 values (x, or the Hadamard-transformed x)
//   bmax   max |v| over everything that shares the scale (16 values, or a 16x16 weight block)
//   gs     tensor scale
// Defines  bs = e4m3(min((bmax/gs)/6, 448)),  y = (v/gs)/bs  in IEEE FP32 -- the operation order of
// the reference's torch path -- and rounds y.  For round-to-nearest a fast path multiplies by a
// reciprocal biased upward by 2^-20: the product then lies in (y, y*(1+1.5*2^-20)], so it rounds
// like y unless it sits within 32 ulp above a rounding boundary (all boundaries have 21 zero low
// mantissa bits); only then are the two divisions done.
template <int ROUNDING>
__device__ __forceinline__ void quant_block16(const float (&v)[16], float bmax, float gs, u32 seed,
                                              u32 blk_idx, u32 elt_idx, uint2& codes, u32& sbyte) {
  u32 sb = e4m3_enc(__fdiv_rn(__fdiv_rn(bmax, gs), 6.0f));
  sbyte = sb;
  u32 w[2] = {0u, 0u};
  if (sb == 0u) {
    // underflowed block: value 0 with the sign of the input
#pragma unroll
    for (int i = 0; i < 16; i++) w[i >> 3] |= ((__float_as_uint(v[i]) >> 31) << 3) << ((i & 7) * 4);
    codes = make_uint2(w[0], w[1]);
    return;
  }
  const float bsf = e4m3_dec(sb);
  float y[16];
  if (ROUNDING == NVFP4_ROUND_NEAREST) {
    const float kf = __fmul_rn(__frcp_rn(__fmul_rn(gs, bsf)), 1.00000095367431640625f);
    u32 nearest = 0xFFFFFFFFu;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      y[i] = __fmul_rn(v[i], kf);
      nearest = min(nearest, __float_as_uint(y[i]) & 0x1FFFE0u);
    }
    if (nearest == 0u) {
#pragma unroll
      for (int i = 0; i < 16; i++) y[i] = __fdiv_rn(__fdiv_rn(v[i], gs), bsf);
    }
#pragma unroll
    for (int i = 0; i < 16; i += 2) w[i >> 3] |= e2m1x2_rn(y[i], y[i + 1]) << ((i & 7) * 4);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i++) y[i] = __fdiv_rn(__fdiv_rn(v[i], gs), bsf);
    if (ROUNDING == NVFP4_ROUND_SR_HW) {
      const u32 hb = hash32(seed ^ hash32(blk_idx));
#pragma unroll
      for (int g = 0; g < 4; g++) {
        const u32 rb = hash32(hb + 0x9E3779B9u * (u32)(g + 1));
        w[g >> 1] |= e2m1x4_rs(y[4 * g], y[4 * g + 1], y[4 * g + 2], y[4 * g + 3], rb) << ((g & 1) * 16);
      }
    } else {
      const u32 hb = hash32(seed ^ hash32(blk_idx));
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const u32 h = (ROUNDING == NVFP4_ROUND_SR_DITHER) ? hash32(hb + (u32)i)
                                                          : hash32(seed ^ (elt_idx + (u32)i) * 0x9E3779B9u);
        const float a = sr_dither(y[i], h);
        const float b = sr_dither(y[i + 1], (h >> 10) | (h << 22));
        w[i >> 3] |= e2m1x2_rn(a, b) << ((i & 7) * 4);
      }
    }
  }
  codes = make_uint2(w[0], w[1]);
}

}  // namespace nvfp4
