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

// eight f32 -> one 32-bit word of E2M1 codes (v[0] in the lowest nibble), round to nearest even
__device__ __forceinline__ u32 e2m1x8_rn(const float* v) {
  u32 r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r) : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
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

// Correctly rounded a/b from the correctly rounded reciprocal rb = RN(1/b): one multiply and two
// fused multiply-adds (Markstein's final division step: q0 = RN(a*rb) is within an ulp of a/b, the
// remainder a - q0*b is exact in one FMA, and RN(q0 + rem*rb) = RN(a/b) unless b's significand is
// all ones).  The divisors here never have an all-ones significand: 6 and the E4M3 block scales
// have at most 4 significant bits, and a tensor scale RN(amax/2688) would need amax strictly
// between two neighbouring floats (2688 * (2^(e+1) - ulp) lies 0.33 to 0.98 of amax's ulp below the
// representable 1.3125 * 2^(e+12)).  The remainder is formed negated so that a zero keeps its sign
// (-0/b = -0).
__device__ __forceinline__ float div_by(float a, float b, float rb) {
  const float q0 = __fmul_rn(a, rb);
  const float nrem = __fmaf_rn(q0, b, -a);
  return __fmaf_rn(-nrem, rb, q0);
}

// Per-tensor constants of a quantizer launch.
struct TensorScale {
  float gs;      // max(k*amax/2688, 1e-30): the FP32 tensor scale
  float rgs;     // RN(1/gs)
  float inv_gs;  // 2688/(k*amax), 0 for an all-zero tensor: the reference kernels' scale (llm-1b/nvq.cu:101)
  const float2* lut;   // shared memory, 128 entries indexed by the scale byte, see make_tensor_scale
};

constexpr int kLutFloats = 256;

// Fill the per-CTA table: for round to nearest  lut[sb] = {RN(1/bs), bs},  for stochastic rounding
// lut[sb] = {inv_gs/bs, bs}  (the exact multiplier of the reference kernels).  `pre` is a power of
// two that the caller's values still have to be multiplied by (0.25 after the Hadamard butterflies,
// else 1): it is folded into gs, which changes no quotient.  Ends with a block barrier.
template <int ROUNDING>
__device__ __forceinline__ TensorScale make_tensor_scale(float amax, float k, float* lut, float* gs_out = nullptr,
                                                         float pre = 1.f) {
  TensorScale t;
  const float am = amax * k;
  const float gs = fmaxf(__fdiv_rn(am, kFp4E4m3), kTiny);
  if (gs_out) *gs_out = gs;
  t.gs = __fdiv_rn(gs, pre);
  t.rgs = __frcp_rn(t.gs);
  t.inv_gs = am > 0.f ? __fmul_rn(__fdiv_rn(kFp4E4m3, am), pre) : 0.f;
  t.lut = reinterpret_cast<const float2*>(lut);
  if (threadIdx.x < 128) {
    const float bsf = e4m3_dec(threadIdx.x);
    float m = 0.f;
    if (threadIdx.x >= 1 && threadIdx.x <= 126)
      m = (ROUNDING == NVFP4_ROUND_NEAREST) ? __frcp_rn(bsf) : __fdiv_rn(t.inv_gs, bsf);
    reinterpret_cast<float2*>(lut)[threadIdx.x] = make_float2(m, bsf);
  }
  __syncthreads();
  return t;
}

// Quantize one block of 16 values that share a scale.
//   v      the 16 values (x, or the Hadamard-transformed x before its power-of-two factor)
//   bmax   max |v| over everything that shares the scale (16 values, or a 16x16 weight block)
// Block scale, all modes:  bs = e4m3(min((bmax/gs)/6, 448))  in IEEE FP32 (the reference's torch path).
// Round to nearest:  y = (v/gs)/bs, the torch path's operation order, each division correctly
//   rounded by div_by() (three FMA-pipe instructions, no branch).
// Stochastic rounding:  y = v * (inv_gs / bs), the reference kernels' form (llm-1b/nvq.cu:50,54) in
//   IEEE arithmetic; the torch path draws torch.rand and so defines no bit-level result.
template <int ROUNDING>
__device__ __forceinline__ void quant_block16(const float (&v)[16], float bmax, const TensorScale& ts, u32 seed,
                                              u32 blk_idx, u32 elt_idx, uint2& codes, u32& sbyte) {
  const float sarg = div_by(div_by(bmax, ts.gs, ts.rgs), 6.0f, 0.16666667163372039794921875f);
  const u32 sb = e4m3_enc(sarg);
  sbyte = sb;
  u32 w[2] = {0u, 0u};
  if (sb == 0u) {
    // underflowed block: value 0 with the sign of the input
#pragma unroll
    for (int i = 0; i < 16; i++) w[i >> 3] |= ((__float_as_uint(v[i]) >> 31) << 3) << ((i & 7) * 4);
    codes = make_uint2(w[0], w[1]);
    return;
  }
  const float2 kf = ts.lut[sb];
  float y[16];
  if (ROUNDING == NVFP4_ROUND_NEAREST) {
#pragma unroll
    for (int i = 0; i < 16; i++) y[i] = div_by(div_by(v[i], ts.gs, ts.rgs), kf.y, kf.x);
    w[0] = e2m1x8_rn(y);
    w[1] = e2m1x8_rn(y + 8);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i++) y[i] = __fmul_rn(v[i], kf.x);
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
        y[i] = sr_dither(y[i], h);
        y[i + 1] = sr_dither(y[i + 1], (h >> 10) | (h << 22));
      }
      w[0] = e2m1x8_rn(y);
      w[1] = e2m1x8_rn(y + 8);
    }
  }
  codes = make_uint2(w[0], w[1]);
}

}  // namespace nvfp4
