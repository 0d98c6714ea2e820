// Pieces shared by the row-operand emitters (warp per row: lane l owns the 8-column chunks 256 j + 8 l).
#pragma once
#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ uint4 ld_chunk(const __nv_bfloat16* p) {
  return *reinterpret_cast<const uint4*>(p);
}

// bf16 magnitudes order like unsigned 16-bit integers: running max of both halves of each word
__device__ __forceinline__ u32 absmax_packed(u32 m, const uint4& q) {
  m = __vmaxu2(m, q.x & 0x7FFF7FFFu); m = __vmaxu2(m, q.y & 0x7FFF7FFFu);
  m = __vmaxu2(m, q.z & 0x7FFF7FFFu); m = __vmaxu2(m, q.w & 0x7FFF7FFFu);
  return m;
}

// Quantize one 8-column chunk (half a block; lane ^ 1 holds the other half) of row r.
// SR: 0 round to nearest, 1 the reference's dither and per-lane sequence, 2 hardware stochastic convert with the
// library's counter-based words (the words of the TMA-fed kernel: keyed by the block, half h = lane & 1 of it).
template <int SR>
__device__ __forceinline__ void emit_chunk_f32(const float (&v)[8], float inv, u32& lcg, long long r, int col, int C,
                                               u32* __restrict__ codes, unsigned char* __restrict__ scales, int lane) {
  float m = absmax3(v[0], v[1], v[2]);
  m = absmax3(m, v[3], v[4]);
  m = absmax3(m, v[5], v[6]);
  m = absmax3(m, v[7], m);
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  const u32 sb = e4m3_enc(__fmul_rn(__fmul_rn(m, inv), 1.f / 6.f));
  const float sd = e4m3_dec(sb);
  const float k = sd > 0.f ? __fdiv_rn(inv, sd) : 0.f;
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; i++) y[i] = __fmul_rn(v[i], k);
  if (SR == 1) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const u32 rnd = lcg_step(lcg);
      y[i] = sr_dither11(y[i], (rnd << 11) & 0x3FF800u);
      y[i + 1] = sr_dither11(y[i + 1], (rnd >> 5) & 0x3FF800u);
    }
  }
  if (SR == 2) {
    // `lcg` carries seed ^ salt here
    u32 key = sr_hw_block_key(lcg, (u32)(r * (C >> 4) + (col >> 4)));
    codes[(r * C + col) >> 3] = round8<NVFP4_ROUND_SR_HW>(y, key, lcg, 0u, lane & 1);
  } else {
    codes[(r * C + col) >> 3] = e2m1x8_rn(y);
  }
  if (!(lane & 1)) scales[sw_off(r, col >> 4, C >> 6)] = (unsigned char)sb;
}

// bf16 pairs of one 16-byte chunk -> eight FP32 values
__device__ __forceinline__ void unpack_chunk(const uint4& raw, float (&v)[8]) {
  const u32 w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}

template <int SR>
__device__ __forceinline__ void emit_chunk(const uint4& raw, float inv, u32& lcg, long long r, int col, int C,
                                           u32* __restrict__ codes, unsigned char* __restrict__ scales, int lane) {
  float v[8];
  unpack_chunk(raw, v);
  emit_chunk_f32<SR>(v, inv, lcg, r, col, C, codes, scales, lane);
}

// ---- a lane that owns a whole 16-value block (round to nearest only: the reference's random sequences are
// defined on the 8-column chunks above)
// k = inv / dec(sb), correctly rounded: the scale has at most 4 significant bits, so one correction step on
// q0 = inv * RN(1 / sd) gives the rounded quotient; `huge` (inv of the order of 1e35: rows of magnitude below 1e-31)
// divides instead, where inv * (1 / sd) could overflow.  A zero scale byte gives 0.
__device__ __forceinline__ float emit_block_k(float inv, u32 sb, bool huge) {
  const float sd = e4m3_dec(sb);
  if (!(sd > 0.f)) return 0.f;
  if (huge) return __fdiv_rn(inv, sd);
  const float r = __frcp_rn(sd);
  const float q0 = __fmul_rn(inv, r);
  return __fmaf_rn(__fmaf_rn(-q0, sd, inv), r, q0);
}

// Block b of row r from its 16 FP32 values (8 packed pairs): scale byte, codes.  nblk = blocks per row.
__device__ __forceinline__ void emit_block16(const u64 (&P)[8], float inv, bool huge, long long r, int b, int nblk,
                                             uint2* __restrict__ codes, unsigned char* __restrict__ scales) {
  const u32 sb = e4m3_enc(__fmul_rn(__fmul_rn(absmax16(P), inv), 1.f / 6.f));
  const float k = emit_block_k(inv, sb, huge);
  const u64 K = f2_pack(k, k);
  float y[16];
#pragma unroll
  for (int t = 0; t < 8; t++) {
    const u64 v = f2_mul(P[t], K);
    y[2 * t] = f2_lo(v); y[2 * t + 1] = f2_hi(v);
  }
  codes[r * nblk + b] = make_uint2(e2m1x8_rn(y), e2m1x8_rn(y + 8));
  scales[sw_off(r, b, nblk >> 2)] = (unsigned char)sb;
}

// 16 consecutive bf16 values (32 bytes, 16-byte aligned) <-> 8 packed FP32 pairs.  Raw16 keeps a block packed (8
// registers instead of 16) between its load and its use.
struct Raw16 { uint4 a, b; };
__device__ __forceinline__ Raw16 ld_raw16(const __nv_bfloat16* p) {
  Raw16 r;
  r.a = *reinterpret_cast<const uint4*>(p);
  r.b = *reinterpret_cast<const uint4*>(p + 8);
  return r;
}
__device__ __forceinline__ void unpack16(const Raw16& r, u64 (&P)[8]) {
  P[0] = f2_from_bf16x2(r.a.x); P[1] = f2_from_bf16x2(r.a.y); P[2] = f2_from_bf16x2(r.a.z); P[3] = f2_from_bf16x2(r.a.w);
  P[4] = f2_from_bf16x2(r.b.x); P[5] = f2_from_bf16x2(r.b.y); P[6] = f2_from_bf16x2(r.b.z); P[7] = f2_from_bf16x2(r.b.w);
}
__device__ __forceinline__ void ld_block16(const __nv_bfloat16* p, u64 (&P)[8]) { unpack16(ld_raw16(p), P); }
__device__ __forceinline__ u32 bf16x2_of(u64 v) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(f2_lo(v), f2_hi(v));
  return *reinterpret_cast<const u32*>(&h);
}
__device__ __forceinline__ void st_block16(__nv_bfloat16* p, const u64 (&P)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(bf16x2_of(P[0]), bf16x2_of(P[1]), bf16x2_of(P[2]), bf16x2_of(P[3]));
  *reinterpret_cast<uint4*>(p + 8) = make_uint4(bf16x2_of(P[4]), bf16x2_of(P[5]), bf16x2_of(P[6]), bf16x2_of(P[7]));
}

}  // namespace nvfp4
