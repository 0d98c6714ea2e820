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

}  // namespace nvfp4
