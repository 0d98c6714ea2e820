// Producer-fused row-operand emitters and the momentum accumulate of the reference's trainer (sm_100a):
//   rms_emit     residual add + RMSNorm + row quantization          (llm-1b/emit.cu:97-147)
//   swiglu_emit  SwiGLU on the raw gate/up GEMM output + row quant.  (llm-1b/emit.cu:149-222)
//   mom_acc      bf16 momentum += alpha * scale * gradient, stochastically rounded (llm-1b/emit.cu:343-363)
// They produce the row operand (codes, swizzled block scales, exact per-row FP32 scale) of the next GEMM straight
// from the values the normalisation / activation computes in FP32, so the activation never makes a round trip
// through HBM as bf16 before it is quantized.
//
// The reference compiles these with --use_fast_math (llm-1b/nvrtc_util.py:20); the arithmetic is restated here as
// explicit FP32 operations so that a CPU model can follow it: fused multiply-adds where the reference's
// expressions contract (x + y*s, ss += v*v, ss/D + eps, m + a*g), round-to-nearest multiplications and divisions
// elsewhere, and three hardware approximations kept as such: rsqrtf for the normalisation, __expf and the
// approximate division of the sigmoid.  What follows them (h, a, the row maximum, scales and codes) is exact
// IEEE arithmetic on their results; rms_emit hands rstd out, swiglu_emit can hand the FP32 activation out, so a
// test can check the approximate step against FP64 within a tolerance and everything after it bit for bit.
//
// A lane owns whole 16-value blocks (block 32 j + lane of the row: a warp reads 1 KB contiguous per step), so block
// maxima and scales need no shuffle and the arithmetic runs on packed FP32 pairs (mul / fma .f32x2).  The row's FP32
// values stay in registers between the row-maximum pass and the quantization pass: every input byte is read once.
// rms_emit: one warp per row; swiglu_emit: one to four warps per row, so that a lane holds at most 64 values.
#include "emit_chunk.cuh"

namespace nvfp4 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// ------------------------------------------------------------------------------------------ rms_emit
// x_new = x + y * (ys[t] * ygw) (stored to xout, and continued from the stored bf16 value); h = (x_new * rstd) * w;
// row operand of h.  D = 512 * NB columns.  Sum of squares: each lane accumulates its even and its odd elements
// separately (one packed fma per pair, blocks and pairs in column order), adds the two, then a butterfly over lanes.
template <int NB, bool HASY>
__global__ void __launch_bounds__(256) rms_emit_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                                       const float* __restrict__ ys, const float* __restrict__ ygw,
                                                       __nv_bfloat16* __restrict__ xout, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ h, uint2* __restrict__ codes,
                                                       unsigned char* __restrict__ scales, float* __restrict__ rs_out,
                                                       float* __restrict__ rstd_out, int T, float eps) {
  constexpr int D = 512 * NB;
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const long long base = r * D + lane * 16;
  u64 P[NB][8];
  {
    Raw16 rx[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) rx[j] = ld_raw16(x + base + j * 512);
#pragma unroll
    for (int j = 0; j < NB; j++) unpack16(rx[j], P[j]);
  }
  if (HASY) {
    const float ysc = __fmul_rn(ys[r], *ygw);
    const u64 YS = f2_pack(ysc, ysc);
    Raw16 ry[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) ry[j] = ld_raw16(y + base + j * 512);
#pragma unroll
    for (int j = 0; j < NB; j++) {
      u64 Y[8];
      unpack16(ry[j], Y);
#pragma unroll
      for (int t = 0; t < 8; t++) P[j][t] = f2_fma(Y[t], YS, P[j][t]);
      st_block16(xout + base + j * 512, P[j]);
      // continue from the stored (rounded) residual, as a recomputation would see it
#pragma unroll
      for (int t = 0; t < 8; t++) P[j][t] = f2_from_bf16x2(bf16x2_of(P[j][t]));
    }
  }
  u64 acc = f2_pack(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < NB; j++)
#pragma unroll
    for (int t = 0; t < 8; t++) acc = f2_fma(P[j][t], P[j][t], acc);
  const float ss = warp_sum(__fadd_rn(f2_lo(acc), f2_hi(acc)));
  const float rstd = rsqrtf(__fmaf_rn(ss, 1.f / D, eps));
  const u64 RS = f2_pack(rstd, rstd);
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < NB; j++) {
    u64 W[8];
    ld_block16(w + lane * 16 + j * 512, W);
#pragma unroll
    for (int t = 0; t < 8; t++) P[j][t] = f2_mul(f2_mul(P[j][t], RS), W[t]);
    am = fmaxf(am, absmax16(P[j]));
    if (h) st_block16(h + base + j * 512, P[j]);
  }
  if (lane == 0 && rstd_out) rstd_out[r] = rstd;
  if (!codes) return;
  am = warp_max(am);
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  const bool huge = !(inv < 1e35f);
  if (lane == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
#pragma unroll
  for (int j = 0; j < NB; j++) emit_block16(P[j], inv, huge, r, j * 32 + lane, D / 16, codes, scales);
}

// ------------------------------------------------------------------------------------------ swiglu_emit
// One activation pair from the raw gate / up outputs: xg = g*sc, xu = u*sc, a = (xg / (1 + exp(-xg))) * xu with the
// exponential and the division taken as the hardware approximations ex2.approx(xg * -log2(e)) and rcp.approx.
__device__ __forceinline__ float ex2_approx(float v) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v)); return r; }
__device__ __forceinline__ float rcp_approx(float v) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v)); return r; }
__device__ __forceinline__ u64 swiglu_pair(u64 G, u64 U, u64 SC) {
  const u64 XG = f2_mul(G, SC), XU = f2_mul(U, SC);
  const u64 Tt = f2_mul(XG, f2_pack(-1.4426950408889634f, -1.4426950408889634f));
  const u64 Dn = f2_add(f2_pack(ex2_approx(f2_lo(Tt)), ex2_approx(f2_hi(Tt))), f2_pack(1.f, 1.f));
  const u64 Rc = f2_pack(rcp_approx(f2_lo(Dn)), rcp_approx(f2_hi(Dn)));
  return f2_mul(f2_mul(XG, Rc), XU);
}

// Register version: NW warps per row (8 / NW rows per CTA); warp `sub` of a row owns the 512-column groups
// j * NW + sub, at most NBL of them per lane (one 16-value block each).  F = 512 * nbf.
template <int NW, int NBL>
__global__ void __launch_bounds__(256, NBL <= 3 ? 3 : 2) swiglu_emit_reg_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ rs_in,
                                                              const float* __restrict__ gw, int nbf, __nv_bfloat16* __restrict__ a_out,
                                                              float* __restrict__ a_f32, uint2* __restrict__ codes,
                                                              unsigned char* __restrict__ scales, float* __restrict__ rs_out,
                                                              int T) {
  __shared__ float red[8];
  const int F = 512 * nbf;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = warp % NW;
  const long long r = (long long)blockIdx.x * (8 / NW) + warp / NW;
  const bool ok = r < T;
  u64 A[NBL][8];
  float am = 0.f;
  if (ok) {
    const float sc = __fmul_rn(rs_in[r], *gw);
    const u64 SC = f2_pack(sc, sc);
    const __nv_bfloat16* g = gu + r * 2 * F + lane * 16;
    Raw16 rg[NBL], ru[NBL];          // all loads in flight first, packed; unpacked block by block
#pragma unroll
    for (int j = 0; j < NBL; j++)
      if (j * NW + sub < nbf) { rg[j] = ld_raw16(g + (j * NW + sub) * 512); ru[j] = ld_raw16(g + F + (j * NW + sub) * 512); }
#pragma unroll
    for (int j = 0; j < NBL; j++) {
      if (j * NW + sub < nbf) {
        u64 U[8];
        unpack16(rg[j], A[j]);
        unpack16(ru[j], U);
#pragma unroll
        for (int t = 0; t < 8; t++) A[j][t] = swiglu_pair(A[j][t], U[t], SC);
        am = fmaxf(am, absmax16(A[j]));
        const long long o = r * F + (j * NW + sub) * 512 + lane * 16;
        if (a_out) st_block16(a_out + o, A[j]);
        if (a_f32) {
#pragma unroll
          for (int t = 0; t < 8; t += 2)
            *reinterpret_cast<float4*>(a_f32 + o + 2 * t) = make_float4(f2_lo(A[j][t]), f2_hi(A[j][t]), f2_lo(A[j][t + 1]), f2_hi(A[j][t + 1]));
        }
      }
    }
  }
  if (!codes) return;
  am = warp_max(am);
  if (NW > 1) {
    if (lane == 0) red[warp] = am;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NW; i++) am = fmaxf(am, red[warp - sub + i]);
  }
  if (!ok) return;
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  const bool huge = !(inv < 1e35f);
  if (lane == 0 && sub == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
#pragma unroll
  for (int j = 0; j < NBL; j++)
    if (j * NW + sub < nbf) emit_block16(A[j], inv, huge, r, (j * NW + sub) * 32 + lane, F / 16, codes, scales);
}

// Any F that is a multiple of 256: warp per row, two passes (the second recomputes the activation from the
// gate / up values, which L1 / L2 still hold); a lane owns the 16-value blocks 32 j + lane.
__global__ void __launch_bounds__(256) swiglu_emit_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ rs_in,
                                                          const float* __restrict__ gw, int F, __nv_bfloat16* __restrict__ a_out,
                                                          float* __restrict__ a_f32, uint2* __restrict__ codes,
                                                          unsigned char* __restrict__ scales, float* __restrict__ rs_out, int T) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const float sc = __fmul_rn(rs_in[r], *gw);
  const u64 SC = f2_pack(sc, sc);
  const __nv_bfloat16* g = gu + r * 2 * F;
  const int nblk = F >> 4;
  float am = 0.f;
  for (int b = lane; b < nblk; b += 32) {
    u64 A[8], U[8];
    ld_block16(g + b * 16, A);
    ld_block16(g + F + b * 16, U);
#pragma unroll
    for (int t = 0; t < 8; t++) A[t] = swiglu_pair(A[t], U[t], SC);
    am = fmaxf(am, absmax16(A));
    if (a_out) st_block16(a_out + r * F + b * 16, A);
    if (a_f32) {
#pragma unroll
      for (int t = 0; t < 8; t += 2)
        *reinterpret_cast<float4*>(a_f32 + r * F + b * 16 + 2 * t) = make_float4(f2_lo(A[t]), f2_hi(A[t]), f2_lo(A[t + 1]), f2_hi(A[t + 1]));
    }
  }
  if (!codes) return;
  am = warp_max(am);
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  const bool huge = !(inv < 1e35f);
  if (lane == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
  for (int b = lane; b < nblk; b += 32) {
    u64 A[8], U[8];
    ld_block16(g + b * 16, A);
    ld_block16(g + F + b * 16, U);
#pragma unroll
    for (int t = 0; t < 8; t++) A[t] = swiglu_pair(A[t], U[t], SC);
    emit_block16(A, inv, huge, r, b, nblk, codes, scales);
  }
}

// ------------------------------------------------------------------------------------------ mom_acc
// m (bf16) <- sr_bf16(m + (alpha * scale) * g): 16 random bits are added below the bf16 mantissa and the sum is
// truncated.  Thread i handles values 8 i .. 8 i + 7 with an LCG started at hash32(seed ^ salt ^ hash32(i)), one
// step per pair of values (low half-word for the even value, high for the odd one).
__global__ void __launch_bounds__(256) mom_acc_kernel(__nv_bfloat16* __restrict__ m, const __nv_bfloat16* __restrict__ g,
                                                      const float* __restrict__ alpha, float scale, long long n8,
                                                      const u32* __restrict__ rng, u32 salt) {
  const float a = __fmul_rn(*alpha, scale);
  const u32 seed = rng[0] ^ salt;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float mv[8], gv[8];
    unpack_chunk(reinterpret_cast<const uint4*>(m)[i], mv);
    unpack_chunk(reinterpret_cast<const uint4*>(g)[i], gv);
    u32 hsh = hash32(seed ^ hash32((u32)i));
    u32 ow[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      hsh = hsh * 1664525u + 1013904223u;
      const float x0 = __fmaf_rn(a, gv[j], mv[j]), x1 = __fmaf_rn(a, gv[j + 1], mv[j + 1]);
      const u32 b0 = (__float_as_uint(x0) + (hsh & 0xFFFFu)) >> 16, b1 = (__float_as_uint(x1) + (hsh >> 16)) >> 16;
      ow[j >> 1] = b0 | (b1 << 16);
    }
    reinterpret_cast<uint4*>(m)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

}  // namespace nvfp4

using namespace nvfp4;

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int nvfp4_rms_emit(const void* x, const void* y, const float* ys, const float* ygw, void* xout, const void* w,
                              void* h, void* codes, void* scales, float* rs_out, float* rstd_out, int T, int D, float eps,
                              void* stream) {
  if (!x || !w) return NVFP4_ERR_NULL;
  if (y && (!ys || !ygw || !xout)) return NVFP4_ERR_NULL;
  if (codes && (!scales || !rs_out)) return NVFP4_ERR_NULL;
  if (T < 0 || (D != 1024 && D != 2048 && D != 4096)) return NVFP4_ERR_SHAPE;
  if (codes && (T & 127)) return NVFP4_ERR_SHAPE;       // swizzled scale tiles cover 128 rows
  if (!al16(x) || !al16(w) || (y && (!al16(y) || !al16(xout))) || (h && !al16(h)) ||
      (codes && (reinterpret_cast<uintptr_t>(codes) & 7u)))
    return NVFP4_ERR_ALIGN;
  if (T == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((T + 7) / 8);
#define NVFP4_RMS_LAUNCH(NK_)                                                                                              \
  if (y) rms_emit_kernel<NK_, true><<<blocks, 256, 0, st>>>(                                                               \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), ys, ygw, static_cast<__nv_bfloat16*>(xout),  \
        static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(h), static_cast<uint2*>(codes),                  \
        static_cast<unsigned char*>(scales), rs_out, rstd_out, T, eps);                                                    \
  else rms_emit_kernel<NK_, false><<<blocks, 256, 0, st>>>(                                                                \
        static_cast<const __nv_bfloat16*>(x), nullptr, nullptr, nullptr, nullptr, static_cast<const __nv_bfloat16*>(w),    \
        static_cast<__nv_bfloat16*>(h), static_cast<uint2*>(codes), static_cast<unsigned char*>(scales), rs_out, rstd_out, T, eps)
  if (D == 2048) { NVFP4_RMS_LAUNCH(4); }
  else if (D == 1024) { NVFP4_RMS_LAUNCH(2); }
  else { NVFP4_RMS_LAUNCH(8); }
#undef NVFP4_RMS_LAUNCH
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_swiglu_emit(const void* gu, const float* rs_in, const float* gw, int F, void* a_out, float* a_f32,
                                 void* codes, void* scales, float* rs_out, int T, void* stream) {
  if (!gu || !rs_in || !gw) return NVFP4_ERR_NULL;
  if (codes && (!scales || !rs_out)) return NVFP4_ERR_NULL;
  if (T < 0 || F <= 0 || (F & 255)) return NVFP4_ERR_SHAPE;
  if (codes && (T & 127)) return NVFP4_ERR_SHAPE;
  if (!al16(gu) || (a_out && !al16(a_out)) || (a_f32 && !al16(a_f32)) || (codes && (reinterpret_cast<uintptr_t>(codes) & 7u)))
    return NVFP4_ERR_ALIGN;
  if (T == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gu);
  __nv_bfloat16* ap = static_cast<__nv_bfloat16*>(a_out);
  uint2* cp = static_cast<uint2*>(codes);
  unsigned char* sp = static_cast<unsigned char*>(scales);
  const int nbf = F / 512;
  // warps per row chosen so that a lane holds at most three (four) 16-value blocks
  if ((F & 511) == 0 && nbf <= 4) swiglu_emit_reg_kernel<1, 4><<<(unsigned)((T + 7) / 8), 256, 0, st>>>(gp, rs_in, gw, nbf, ap, a_f32, cp, sp, rs_out, T);
  else if ((F & 511) == 0 && nbf <= 6) swiglu_emit_reg_kernel<2, 3><<<(unsigned)((T + 3) / 4), 256, 0, st>>>(gp, rs_in, gw, nbf, ap, a_f32, cp, sp, rs_out, T);
  else if ((F & 511) == 0 && nbf <= 12) swiglu_emit_reg_kernel<4, 3><<<(unsigned)((T + 1) / 2), 256, 0, st>>>(gp, rs_in, gw, nbf, ap, a_f32, cp, sp, rs_out, T);
  else swiglu_emit_kernel<<<(unsigned)((T + 7) / 8), 256, 0, st>>>(gp, rs_in, gw, F, ap, a_f32, cp, sp, rs_out, T);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_mom_acc(void* m, const void* g, const float* alpha, float scale, long long n, const unsigned* rng,
                             unsigned salt, void* stream) {
  if (!m || !g || !alpha || !rng) return NVFP4_ERR_NULL;
  if (n < 0 || (n & 7)) return NVFP4_ERR_SHAPE;
  if (!al16(m) || !al16(g)) return NVFP4_ERR_ALIGN;
  if (n == 0) return NVFP4_OK;
  const long long n8 = n >> 3;
  long long blocks = (n8 + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  mom_acc_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(m), static_cast<const __nv_bfloat16*>(g), alpha, scale, n8, rng, salt);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}
