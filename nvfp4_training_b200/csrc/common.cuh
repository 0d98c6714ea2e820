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

// Per-tensor constants of a quantizer launch.
struct TensorScale {
  float gs;      // max(k*amax/2688, 1e-30): the FP32 tensor scale
  float r6;      // 1/(6*gs), biased up by 2^-20: fast path of the block-scale argument
  float inv_gs;  // 2688/(k*amax), 0 for an all-zero tensor: the reference kernels' scale (llm-1b/nvq.cu:101)
  const float* lut;   // shared memory, 128 entries: per scale byte, the multiplier that turns v into y
};

// Fill the per-CTA table: for round to nearest  lut[sb] = (1/(gs*bs))*(1+2^-20)  (biased fast path),
// for stochastic rounding  lut[sb] = inv_gs/bs  (the exact multiplier).  Ends with a block barrier.
template <int ROUNDING>
__device__ __forceinline__ TensorScale make_tensor_scale(float amax, float k, float* lut) {
  TensorScale t;
  const float am = amax * k;
  t.gs = fmaxf(__fdiv_rn(am, kFp4E4m3), kTiny);
  t.r6 = __fmul_rn(__frcp_rn(__fmul_rn(t.gs, 6.0f)), 1.00000095367431640625f);
  t.inv_gs = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  t.lut = lut;
  if (threadIdx.x < 128) {
    const float bsf = e4m3_dec(threadIdx.x);
    float m = 0.f;
    if (threadIdx.x >= 1 && threadIdx.x <= 126)
      m = (ROUNDING == NVFP4_ROUND_NEAREST) ? __fmul_rn(__frcp_rn(__fmul_rn(t.gs, bsf)), 1.00000095367431640625f)
                                            : __fdiv_rn(t.inv_gs, bsf);
    lut[threadIdx.x] = m;
  }
  __syncthreads();
  return t;
}

// The exact (slow) forms live in functions that are never inlined: a call cannot be turned into
// straight-line speculated code, so the IEEE divisions really run only on the rare slow path.
static __device__ __noinline__ float exact_scale_arg(float bmax, float gs) { return __fdiv_rn(__fdiv_rn(bmax, gs), 6.0f); }
static __device__ __noinline__ float exact_scaled(float v, float gs, float bsf) { return __fdiv_rn(__fdiv_rn(v, gs), bsf); }

// Quantize one block of 16 values that share a scale.
//   v      the 16 values (x, or the Hadamard-transformed x)
//   bmax   max |v| over everything that shares the scale (16 values, or a 16x16 weight block)
// Block scale, all modes:  bs = e4m3(min((bmax/gs)/6, 448))  in IEEE FP32 (the reference's torch path).
// Round to nearest:  y = (v/gs)/bs, the torch path's operation order.  Both the scale argument and y
//   are first formed with a reciprocal biased upward by 2^-20: the product then lies in
//   (exact, exact*(1+1.5*2^-20)], so it rounds like the exact value unless it sits within 32 ulp above
//   a rounding boundary (E4M3 boundaries have 19 zero low mantissa bits, E2M1 boundaries 21); only
//   then are the divisions done.
// Stochastic rounding:  y = v * (inv_gs / bs), the reference kernels' form (llm-1b/nvq.cu:50,54) in
//   IEEE arithmetic; the torch path draws torch.rand and so defines no bit-level result.
template <int ROUNDING>
__device__ __forceinline__ void quant_block16(const float (&v)[16], float bmax, const TensorScale& ts, u32 seed,
                                              u32 blk_idx, u32 elt_idx, uint2& codes, u32& sbyte) {
  float sarg = __fmul_rn(bmax, ts.r6);
  if (sarg < 0.03125f || (__float_as_uint(sarg) & 0x7FFE0u) == 0u) sarg = exact_scale_arg(bmax, ts.gs);
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
  const float kf = ts.lut[sb];
  float y[16];
  if (ROUNDING == NVFP4_ROUND_NEAREST) {
    u32 nearest = 0xFFFFFFFFu;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      y[i] = __fmul_rn(v[i], kf);
      nearest = min(nearest, __float_as_uint(y[i]) & 0x1FFFE0u);
    }
    if (nearest == 0u) {
      const float bsf = e4m3_dec(sb);
#pragma unroll
      for (int i = 0; i < 16; i++)
        if ((__float_as_uint(y[i]) & 0x1FFFE0u) == 0u) y[i] = exact_scaled(v[i], ts.gs, bsf);
    }
    w[0] = e2m1x8_rn(y);
    w[1] = e2m1x8_rn(y + 8);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i++) y[i] = __fmul_rn(v[i], kf);
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
