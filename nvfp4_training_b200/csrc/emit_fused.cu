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
// One warp per row (rms_emit; two warps per row for the 5632-wide SwiGLU), the row's FP32 values held in registers
// between the row-maximum pass and the quantization pass: every input byte is read once.
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
__device__ __forceinline__ uint4 pack_chunk_bf16(const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

// ------------------------------------------------------------------------------------------ rms_emit
// x_new = x + y * (ys[t] * ygw) (stored to xout, and continued from the stored bf16 value); h = (x_new * rstd) * w;
// row operand of h.  D = 256 * NK columns.
template <int NK, bool HASY>
__global__ void __launch_bounds__(256) rms_emit_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                                       const float* __restrict__ ys, const float* __restrict__ ygw,
                                                       __nv_bfloat16* __restrict__ xout, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ h, u32* __restrict__ codes,
                                                       unsigned char* __restrict__ scales, float* __restrict__ rs_out,
                                                       float* __restrict__ rstd_out, int T, float eps) {
  constexpr int D = 256 * NK;
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const long long base = r * D + lane * 8;
  uint4 raw[NK];
#pragma unroll
  for (int j = 0; j < NK; j++) raw[j] = ld_chunk(x + base + j * 256);
  float v[NK][8];
  float ss = 0.f;
  if (HASY) {
    const float ysc = __fmul_rn(ys[r], *ygw);
    uint4 rawy[NK];
#pragma unroll
    for (int j = 0; j < NK; j++) rawy[j] = ld_chunk(y + base + j * 256);
#pragma unroll
    for (int j = 0; j < NK; j++) {
      float yy[8];
      unpack_chunk(raw[j], v[j]);
      unpack_chunk(rawy[j], yy);
#pragma unroll
      for (int i = 0; i < 8; i++) v[j][i] = __fmaf_rn(yy[i], ysc, v[j][i]);
      const uint4 o = pack_chunk_bf16(v[j]);
      *reinterpret_cast<uint4*>(xout + base + j * 256) = o;
      unpack_chunk(o, v[j]);        // continue from the stored (rounded) residual, as a recomputation would see it
    }
  } else {
#pragma unroll
    for (int j = 0; j < NK; j++) unpack_chunk(raw[j], v[j]);
  }
#pragma unroll
  for (int j = 0; j < NK; j++)
#pragma unroll
    for (int i = 0; i < 8; i++) ss = __fmaf_rn(v[j][i], v[j][i], ss);
  const float rstd = rsqrtf(__fmaf_rn(warp_sum(ss), 1.f / D, eps));
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < NK; j++) {
    float ww[8];
    unpack_chunk(ld_chunk(w + lane * 8 + j * 256), ww);
#pragma unroll
    for (int i = 0; i < 8; i++) v[j][i] = __fmul_rn(__fmul_rn(v[j][i], rstd), ww[i]);
    am = absmax3(am, v[j][0], v[j][1]); am = absmax3(am, v[j][2], v[j][3]);
    am = absmax3(am, v[j][4], v[j][5]); am = absmax3(am, v[j][6], v[j][7]);
    if (h) *reinterpret_cast<uint4*>(h + base + j * 256) = pack_chunk_bf16(v[j]);
  }
  if (lane == 0 && rstd_out) rstd_out[r] = rstd;
  if (!codes) return;
  am = warp_max(am);
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  if (lane == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
  u32 unused = 0u;
#pragma unroll
  for (int j = 0; j < NK; j++) emit_chunk_f32<0>(v[j], inv, unused, r, j * 256 + lane * 8, D, codes, scales, lane);
}

// ------------------------------------------------------------------------------------------ swiglu_emit
// One activation value from the raw gate / up outputs: xg = g*sc, xu = u*sc, a = (xg / (1 + exp(-xg))) * xu with
// the exponential and the division taken as the hardware approximations.
__device__ __forceinline__ float swiglu_value(float g, float u, float sc) {
  const float xg = __fmul_rn(g, sc), xu = __fmul_rn(u, sc);
  return __fmul_rn(__fdividef(xg, __fadd_rn(1.f, __expf(-xg))), xu);
}

// Register version: F = NW * 256 * NG, NW warps per row (8 / NW rows per CTA), NG chunks per lane kept in FP32.
// Warp `sub` of a row owns the chunks j * NW + sub.
template <int NW, int NG>
__global__ void __launch_bounds__(256) swiglu_emit_reg_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ rs_in,
                                                              const float* __restrict__ gw, __nv_bfloat16* __restrict__ a_out,
                                                              float* __restrict__ a_f32, u32* __restrict__ codes,
                                                              unsigned char* __restrict__ scales, float* __restrict__ rs_out,
                                                              int T) {
  constexpr int F = NW * 256 * NG;
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = warp % NW;
  const long long r = (long long)blockIdx.x * (8 / NW) + warp / NW;
  const bool ok = r < T;
  const float sc = ok ? __fmul_rn(rs_in[r], *gw) : 0.f;
  float a[NG][8];
  float am = 0.f;
  if (ok) {
    const __nv_bfloat16* g = gu + r * 2 * F + lane * 8;
    uint4 rg[NG], ru[NG];
#pragma unroll
    for (int j = 0; j < NG; j++) { rg[j] = ld_chunk(g + (j * NW + sub) * 256); ru[j] = ld_chunk(g + F + (j * NW + sub) * 256); }
#pragma unroll
    for (int j = 0; j < NG; j++) {
      float gv[8], uv[8];
      unpack_chunk(rg[j], gv);
      unpack_chunk(ru[j], uv);
#pragma unroll
      for (int i = 0; i < 8; i++) a[j][i] = swiglu_value(gv[i], uv[i], sc);
      am = absmax3(am, a[j][0], a[j][1]); am = absmax3(am, a[j][2], a[j][3]);
      am = absmax3(am, a[j][4], a[j][5]); am = absmax3(am, a[j][6], a[j][7]);
      const long long o = r * F + (j * NW + sub) * 256 + lane * 8;
      if (a_out) *reinterpret_cast<uint4*>(a_out + o) = pack_chunk_bf16(a[j]);
      if (a_f32) {
        *reinterpret_cast<float4*>(a_f32 + o) = make_float4(a[j][0], a[j][1], a[j][2], a[j][3]);
        *reinterpret_cast<float4*>(a_f32 + o + 4) = make_float4(a[j][4], a[j][5], a[j][6], a[j][7]);
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
  if (lane == 0 && sub == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
  u32 unused = 0u;
#pragma unroll
  for (int j = 0; j < NG; j++) emit_chunk_f32<0>(a[j], inv, unused, r, (j * NW + sub) * 256 + lane * 8, F, codes, scales, lane);
}

// Any F that is a multiple of 256: warp per row, two passes (the second recomputes the activation from the
// gate / up values, which L1 / L2 still hold).
__global__ void __launch_bounds__(256) swiglu_emit_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ rs_in,
                                                          const float* __restrict__ gw, int F, __nv_bfloat16* __restrict__ a_out,
                                                          float* __restrict__ a_f32, u32* __restrict__ codes,
                                                          unsigned char* __restrict__ scales, float* __restrict__ rs_out, int T) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const float sc = __fmul_rn(rs_in[r], *gw);
  const __nv_bfloat16* g = gu + r * 2 * F;
  float am = 0.f;
  for (int c = lane * 8; c < F; c += 256) {
    float gv[8], uv[8], a[8];
    unpack_chunk(ld_chunk(g + c), gv);
    unpack_chunk(ld_chunk(g + F + c), uv);
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = swiglu_value(gv[i], uv[i], sc);
    am = absmax3(am, a[0], a[1]); am = absmax3(am, a[2], a[3]); am = absmax3(am, a[4], a[5]); am = absmax3(am, a[6], a[7]);
    if (a_out) *reinterpret_cast<uint4*>(a_out + r * F + c) = pack_chunk_bf16(a);
    if (a_f32) {
      *reinterpret_cast<float4*>(a_f32 + r * F + c) = make_float4(a[0], a[1], a[2], a[3]);
      *reinterpret_cast<float4*>(a_f32 + r * F + c + 4) = make_float4(a[4], a[5], a[6], a[7]);
    }
  }
  if (!codes) return;
  am = warp_max(am);
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  if (lane == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
  u32 unused = 0u;
  for (int c = lane * 8; c < F; c += 256) {
    float gv[8], uv[8], a[8];
    unpack_chunk(ld_chunk(g + c), gv);
    unpack_chunk(ld_chunk(g + F + c), uv);
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = swiglu_value(gv[i], uv[i], sc);
    emit_chunk_f32<0>(a, inv, unused, r, c, F, codes, scales, lane);
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
      (codes && (reinterpret_cast<uintptr_t>(codes) & 3u)))
    return NVFP4_ERR_ALIGN;
  if (T == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((T + 7) / 8);
#define NVFP4_RMS_LAUNCH(NK_)                                                                                              \
  if (y) rms_emit_kernel<NK_, true><<<blocks, 256, 0, st>>>(                                                               \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), ys, ygw, static_cast<__nv_bfloat16*>(xout),  \
        static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(h), static_cast<u32*>(codes),                    \
        static_cast<unsigned char*>(scales), rs_out, rstd_out, T, eps);                                                    \
  else rms_emit_kernel<NK_, false><<<blocks, 256, 0, st>>>(                                                                \
        static_cast<const __nv_bfloat16*>(x), nullptr, nullptr, nullptr, nullptr, static_cast<const __nv_bfloat16*>(w),    \
        static_cast<__nv_bfloat16*>(h), static_cast<u32*>(codes), static_cast<unsigned char*>(scales), rs_out, rstd_out, T, eps)
  if (D == 2048) { NVFP4_RMS_LAUNCH(8); }
  else if (D == 1024) { NVFP4_RMS_LAUNCH(4); }
  else { NVFP4_RMS_LAUNCH(16); }
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
  if (!al16(gu) || (a_out && !al16(a_out)) || (a_f32 && !al16(a_f32)) || (codes && (reinterpret_cast<uintptr_t>(codes) & 3u)))
    return NVFP4_ERR_ALIGN;
  if (T == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gu);
  __nv_bfloat16* ap = static_cast<__nv_bfloat16*>(a_out);
  u32* cp = static_cast<u32*>(codes);
  unsigned char* sp = static_cast<unsigned char*>(scales);
  if (F == 5632) swiglu_emit_reg_kernel<2, 11><<<(unsigned)((T + 3) / 4), 256, 0, st>>>(gp, rs_in, gw, ap, a_f32, cp, sp, rs_out, T);
  else if (F == 2048) swiglu_emit_reg_kernel<1, 8><<<(unsigned)((T + 7) / 8), 256, 0, st>>>(gp, rs_in, gw, ap, a_f32, cp, sp, rs_out, T);
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
