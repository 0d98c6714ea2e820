// NVFP4 quantizer kernels for sm_100a: per-tensor amax, 1x16 row quantizer, transposed
// RHT16 quantizer, 16x16 weight quantizer (W and W^T), scale re-swizzle.  All HBM-bound:
// 128-bit coalesced loads, register-resident blocks, warp shuffles for exchanges/reductions.
#include <stdlib.h>

#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const u32 w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ uint4 ldg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// ------------------------------------------------------------------------------------------ amax
// max|x| via atomicMax on the float bit pattern (non-negative floats order like unsigned ints).
__device__ __forceinline__ uint4 ld_cg_128(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint4* __restrict__ x, long long n8, float* out) {
  pdl_trigger();
  pdl_wait();
  u32 m = 0u;  // running max of |x| as bf16 bit patterns in both halves of a word
  const long long stride = (long long)gridDim.x * blockDim.x;
  // batches of four loads in flight per thread.  The last, partial batch clamps the indices past the end to the last
  // element (a maximum does not mind reading it again) rather than walking one load at a time: on a 33 MB tensor a
  // thread has seven loads, and three of them in sequence cost more than the first four together.
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n8; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = ld_cg_128(x + i + j * stride);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      m = __vmaxu2(m, v[j].x & 0x7FFF7FFFu); m = __vmaxu2(m, v[j].y & 0x7FFF7FFFu);
      m = __vmaxu2(m, v[j].z & 0x7FFF7FFFu); m = __vmaxu2(m, v[j].w & 0x7FFF7FFFu);
    }
  }
  if (i < n8) {
    const long long last = n8 - 1;
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = ld_cg_128(x + min(i + j * stride, last));
#pragma unroll
    for (int j = 0; j < 4; j++) {
      m = __vmaxu2(m, v[j].x & 0x7FFF7FFFu); m = __vmaxu2(m, v[j].y & 0x7FFF7FFFu);
      m = __vmaxu2(m, v[j].z & 0x7FFF7FFFu); m = __vmaxu2(m, v[j].w & 0x7FFF7FFFu);
    }
  }
  u32 mm = max(m & 0xFFFFu, m >> 16);
  // NaN patterns (> 0x7F80) count as +inf
  mm = min(mm, 0x7F80u);
#pragma unroll
  for (int o = 16; o; o >>= 1) mm = max(mm, __shfl_xor_sync(0xffffffffu, mm, o));
  __shared__ u32 sm[8];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mm;
  __syncthreads();
  if (threadIdx.x < 32) {
    mm = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0u;
#pragma unroll
    for (int o = 4; o; o >>= 1) mm = max(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    if (threadIdx.x == 0 && mm) atomicMax(reinterpret_cast<unsigned*>(out), mm << 16);
  }
}

// ------------------------------------------------------------------------------------------ rows
template <bool WIDE>
__device__ __forceinline__ Block32 load_block(const __nv_bfloat16* p) {
  Block32 r;
  if (WIDE) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
                 : "l"(p));
  } else {
    const uint4 a = ldg128(p), b = ldg128(p + 8);
    r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
  }
  return r;
}

// One warp per (row, 512-column segment); a lane owns one 16-block (32 contiguous bytes, one
// 256-bit load when rows are 32-byte aligned), so the warp reads 1 KB contiguous and needs no
// exchange.  The next item's load is issued before the current one is processed.
template <int ROUNDING, bool WIDE>
__global__ void __launch_bounds__(256, 4) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                          uint2* __restrict__ codes, unsigned char* __restrict__ scales,
                                                          const float* __restrict__ amax, int R, int C, int linear,
                                                          u32 seed, const u32* __restrict__ seed_dev,
                                                          float* __restrict__ gs_out) {
  if (ROUNDING != NVFP4_ROUND_NEAREST && seed_dev) seed = __ldg(seed_dev);
  const int lane = threadIdx.x & 31;
  const int nblk = C >> 4;
  const int nseg = (nblk + 31) >> 5;
  __shared__ __align__(8) float lut[kLutFloats];
  const TensorScale ts = make_tensor_scale<ROUNDING>(__ldg(amax), 1.f, lut,
                                                     (blockIdx.x == 0 && threadIdx.x == 0) ? gs_out : nullptr);
  // walk (row, segment) pairs with a fixed warp stride, without a division per item
  const unsigned nwarps = gridDim.x * (blockDim.x >> 5);
  const unsigned w0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int dr = (int)(nwarps / (unsigned)nseg), ds = (int)(nwarps % (unsigned)nseg);
  int r = (int)(w0 / (unsigned)nseg), seg = (int)(w0 % (unsigned)nseg);
  Block32 cur = {};
  if (r < R && seg * 32 + lane < nblk) cur = load_block<WIDE>(x + (long long)r * ldx + (seg * 32 + lane) * 16);
  while (r < R) {
    int rn = r + dr, sn = seg + ds;
    if (sn >= nseg) { sn -= nseg; rn++; }
    Block32 nxt = {};
    if (rn < R && sn * 32 + lane < nblk) nxt = load_block<WIDE>(x + (long long)rn * ldx + (sn * 32 + lane) * 16);
    const int blk = seg * 32 + lane;
    if (blk < nblk) {
      u64 P[8];
#pragma unroll
      for (int i = 0; i < 8; i++) P[i] = f2_from_bf16x2(cur.w[i]);
      const u32 sb = block_scale_byte(absmax16(P), ts);
      const long long b = (long long)r * nblk + blk;
      codes[b] = quant_block16<ROUNDING>(P, sb, ts, seed, (u32)b, (u32)(b * 16));
      scales[linear ? b : sw_off(r, blk, nblk >> 2)] = (unsigned char)sb;
    }
    r = rn; seg = sn; cur = nxt;
  }
}

// ------------------------------------------------------------------------------------------ cols + RHT16
// CTA tile: 128 columns x 256 tokens.  A thread loads 16 tokens x 8 columns with 16 coalesced
// 128-bit loads (half-warp = 256 contiguous bytes of one token row), so each 16-token column
// block lives in its registers: sign flip, 4 butterfly stages, x0.25 and quantization need no
// shared memory.  Outputs: 8 bytes of codes + 1 scale byte per (column, token block).
template <int ROUNDING>
__global__ void __launch_bounds__(256, 2) quant_cols_rht_kernel(const __nv_bfloat16* __restrict__ x,
                                                              unsigned char* __restrict__ codes,
                                                              unsigned char* __restrict__ scales,
                                                              const float* __restrict__ amax, int M, int C, int linear,
                                                              u32 signs, u32 seed, const u32* __restrict__ seed_dev,
                                                              float* __restrict__ gs_out) {
  if (ROUNDING != NVFP4_ROUND_NEAREST && seed_dev) seed = __ldg(seed_dev);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cchunk = blockIdx.x * 16 + (lane & 15);            // 8-column chunk index
  const int mb = blockIdx.y * 16 + warp * 2 + (lane >> 4);     // 16-token block index
  const int nmb = M >> 4;
  __shared__ __align__(8) float lut[kLutFloats];
  // the x0.25 that follows the butterflies is folded into the tensor scale (a power of two)
  const TensorScale ts = make_tensor_scale<ROUNDING>(__ldg(amax), 4.f, lut,
      (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ? gs_out : nullptr, 0.25f);
  if (cchunk * 8 >= C || mb >= nmb) return;
  uint4 raw[16];
  const __nv_bfloat16* p = x + (long long)mb * 16 * C + cchunk * 8;
#pragma unroll
  for (int i = 0; i < 16; i++) raw[i] = ldg128(p + (long long)i * C);
  // apply the sign vector on the packed bf16 words: token i is negated when bit i of signs is set
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const u32 f = ((signs >> i) & 1u) ? 0x80008000u : 0u;
    raw[i].x ^= f; raw[i].y ^= f; raw[i].z ^= f; raw[i].w ^= f;
  }
  // four rounds of two columns (one packed word per token): the words are rotated so that the
  // loop body exists once in the instruction stream.  The two columns ride in the two halves of
  // packed FP32 pairs through the butterflies and the scaling.
#pragma unroll 1
  for (int jw = 0; jw < 4; jw++) {
    u64 P[16];
#pragma unroll
    for (int i = 0; i < 16; i++) P[i] = f2_from_bf16x2(raw[i].x);
#pragma unroll
    for (int h = 1; h < 16; h <<= 1)
#pragma unroll
      for (int i = 0; i < 16; i++)
        if (!(i & h)) { const u64 a = P[i], b = P[i + h]; P[i] = f2_add(a, b); P[i + h] = f2_sub(a, b); }
    const long long c = (long long)cchunk * 8 + jw * 2;
    const long long b0 = c * nmb + mb, b1 = b0 + nmb;
    uint2 o0, o1; u32 sb0, sb1;
    quant_block16x2<ROUNDING>(P, ts, seed, (u32)b0, (u32)b1, block_key<ROUNDING>(seed, (u32)b0), block_key<ROUNDING>(seed, (u32)b1),
                              o0, o1, sb0, sb1);
    *reinterpret_cast<uint2*>(codes + b0 * 8) = o0;
    *reinterpret_cast<uint2*>(codes + b1 * 8) = o1;
    scales[linear ? b0 : sw_off(c, mb, nmb >> 2)] = (unsigned char)sb0;
    scales[linear ? b1 : sw_off(c + 1, mb, nmb >> 2)] = (unsigned char)sb1;
#pragma unroll
    for (int i = 0; i < 16; i++) { raw[i].x = raw[i].y; raw[i].y = raw[i].z; raw[i].z = raw[i].w; }
  }
}

// ------------------------------------------------------------------------------------------ 16x16 weights
// Persistent CTAs; one warp per group of four 16x16 blocks that are neighbours along N (same K
// block): lane = (row, 8-column half) of each block, four independent 16-byte loads in flight per
// lane.  Block max by warp shuffles, codes for W written as one word per lane and block, codes for
// W^T gathered with shuffles (lane = (k row, 8-row half)) and, after one exchange inside each lane
// pair, stored as 16 contiguous bytes per lane: a k row's 32 bytes for the four blocks leave together.
template <typename T>
__global__ void __launch_bounds__(256) quant_w2d_kernel(const T* __restrict__ w, u32* __restrict__ q,
                                                         unsigned char* __restrict__ s, u32* __restrict__ qt,
                                                         unsigned char* __restrict__ st, const float* __restrict__ amax,
                                                         int N, int K, int linear, float* __restrict__ gs_out) {
  const int lane = threadIdx.x & 31;
  const int nb = N >> 4, kb = K >> 4;
  const int ngrp = (nb + 3) >> 2;
  __shared__ __align__(8) float lut[kLutFloats];
  const TensorScale ts = make_tensor_scale<NVFP4_ROUND_NEAREST>(__ldg(amax), 1.f, lut,
                                                               (blockIdx.x == 0 && threadIdx.x == 0) ? gs_out : nullptr);
  const u64 G = f2_pack(ts.gs, ts.gs), NRG = f2_pack(ts.nrgs, ts.nrgs);
  const int r = lane >> 1, c0 = (lane & 1) * 8;
  const bool wide_t = !(N & 31) && !(reinterpret_cast<uintptr_t>(qt) & 15u);   // 16-byte stores of W^T codes possible
  const long long nitems = (long long)ngrp * kb;
  const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < nitems; item += wstride) {
    // consecutive warps walk K: the loads of a CTA are contiguous along each row
    const int grp = (int)(item / kb), bk = (int)(item - (long long)grp * kb);
    float v[4][8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int bn = grp * 4 + j;
      if (bn < nb) {
        const T* src = w + (long long)(bn * 16 + r) * K + bk * 16 + c0;
        if constexpr (sizeof(T) == 2) {
          unpack8(ldg128(src), v[j]);
        } else {
          const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src) + 1);
          v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w; v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[j][i] = 0.f;
      }
    }
    u32 wt[4], sbs[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int bn = grp * 4 + j;
      float bmax = absmax3(v[j][0], v[j][1], v[j][2]);
      bmax = absmax3(bmax, v[j][3], v[j][4]);
      bmax = absmax3(bmax, v[j][5], v[j][6]);
      bmax = absmax3(bmax, v[j][7], bmax);
#pragma unroll
      for (int o = 16; o; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
      const u32 sb = block_scale_byte(bmax, ts);
      sbs[j] = sb;
      const float2 kf = lut_entry(ts, sb);
      const u64 NRH = f2_pack(kf.x, kf.x), NRL = f2_pack(kf.y, kf.y);
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const u64 t = f2_div_bs(f2_ndiv(f2_pack(v[j][i], v[j][i + 1]), G, NRG), NRH, NRL);
        y[i] = f2_lo(t); y[i + 1] = f2_hi(t);
      }
      const u32 word = e2m1x8_rn(y);
      if (q && bn < nb) {
        q[((long long)(bn * 16 + r) * K + bk * 16 + c0) >> 3] = word;
        if (!(lane & 1)) s[linear ? (long long)(bn * 16 + r) * kb + bk : sw_off(bn * 16 + r, bk, kb >> 2)] = (unsigned char)sb;
      }
      // transposed block: this lane builds k-row kk = lane>>1, n values (lane&1)*8 .. +7
      const int kk = lane >> 1;
      u32 t = 0u;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const u32 ww = __shfl_sync(0xffffffffu, word, 2 * (c0 + i) + (kk >> 3));
        t |= ((ww >> (4 * (kk & 7))) & 15u) << (4 * i);
      }
      wt[j] = t;
    }
    if (qt) {
      const int kk = lane >> 1;
      const long long krow = (long long)bk * 16 + kk;
      if (grp * 4 + 3 < nb && wide_t) {
        // even lane keeps blocks 0,1 (both 8-row halves), odd lane blocks 2,3: 16 contiguous bytes each
        const bool odd = lane & 1;
        const u32 give0 = odd ? wt[0] : wt[2], give1 = odd ? wt[1] : wt[3];
        const u32 got0 = __shfl_xor_sync(0xffffffffu, give0, 1), got1 = __shfl_xor_sync(0xffffffffu, give1, 1);
        const uint4 o = odd ? make_uint4(got0, wt[2], got1, wt[3]) : make_uint4(wt[0], got0, wt[1], got1);
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(qt) + krow * (N >> 1) + grp * 32 + (odd ? 16 : 0)) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (grp * 4 + j < nb) qt[(krow * N + (grp * 4 + j) * 16 + c0) >> 3] = wt[j];
      }
      if (!(lane & 1)) {
        if (grp * 4 + 3 < nb && (!linear || !(nb & 3))) {
          // the four blocks' scale bytes are neighbours in both layouts
          const long long o = linear ? krow * nb + grp * 4 : sw_off(krow, grp * 4, nb >> 2);
          *reinterpret_cast<u32*>(st + o) = sbs[0] | (sbs[1] << 8) | (sbs[2] << 16) | (sbs[3] << 24);
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int bn = grp * 4 + j;
            if (bn < nb) st[linear ? krow * nb + bn : sw_off(krow, bn, nb >> 2)] = (unsigned char)sbs[j];
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ scale re-swizzle
__global__ void __launch_bounds__(256) swizzle_scales_kernel(const unsigned char* __restrict__ src, long long lds,
                                                              int R, int C16, unsigned char* __restrict__ dst) {
  const int ncb = C16 >> 2;
  const long long total = (long long)R * ncb;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    // consecutive threads walk the destination so stores coalesce
    const long long tile = i >> 7;           // (row block, column tile)
    const int in = (int)(i & 127);           // (r%32)*4 + (r%128)/32
    const long long rb = tile / ncb; const int cb = (int)(tile - rb * ncb);
    const long long r = rb * 128 + (in & 3) * 32 + (in >> 2);
    const unsigned char* p = src + r * lds + cb * 4;
    const u32 v = (u32)p[0] | ((u32)p[1] << 8) | ((u32)p[2] << 16) | ((u32)p[3] << 24);
    *reinterpret_cast<u32*>(dst + i * 4) = v;
  }
}

// ------------------------------------------------------------------------------------------ raw SR convert
__global__ void __launch_bounds__(256) e2m1x4_sr_kernel(const float4* __restrict__ y, const u32* __restrict__ rbits,
                                                         unsigned short* __restrict__ out, long long n4) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = y[i];
  out[i] = (unsigned short)e2m1x4_rs(v.x, v.y, v.z, v.w, rbits[i]);
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace nvfp4

using namespace nvfp4;

static int g_pdl = -1;      // -1: not decided yet (environment NVFP4_PDL=1 switches it on), else 0 / 1
bool nvfp4_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("NVFP4_PDL");
    g_pdl = (e && e[0] == '1') ? 1 : 0;
  }
  return g_pdl != 0;
}
extern "C" int nvfp4_set_pdl(int on) {
  g_pdl = on ? 1 : 0;
  return NVFP4_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int amax_launch(const void* x, long long n, float* out, bool clear, void* stream) {
  if (!out || (!x && n > 0)) return NVFP4_ERR_NULL;
  if (n < 0 || (n & 7)) return NVFP4_ERR_SHAPE;
  if (!aligned16(x)) return NVFP4_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (clear && cudaMemsetAsync(out, 0, sizeof(float), st) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (n == 0) return NVFP4_OK;
  const long long n8 = n >> 3;
  long long blocks = (n8 + 256 * 4 - 1) / (256 * 4);
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (nvfp4_launch_kernel(amax_bf16_kernel, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const uint4*>(x), n8, out) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVFP4_ERR_CUDA;
  }
  return NVFP4_OK;
}

extern "C" int nvfp4_amax_bf16(const void* x, long long n, float* out, void* stream) {
  return amax_launch(x, n, out, true, stream);
}

extern "C" int nvfp4_amax_bf16_update(const void* x, long long n, float* out, void* stream) {
  return amax_launch(x, n, out, false, stream);
}

extern "C" int nvfp4_quant_rows(const void* x, long long ldx, int R, int C, void* codes, void* scales,
                                int scale_layout, const float* amax, float* gs_out, int rounding, unsigned seed,
                                const unsigned* seed_dev, void* stream) {
  if (!x || !codes || !scales || !amax) return NVFP4_ERR_NULL;
  if (scale_layout != NVFP4_SCALES_SWIZZLED && scale_layout != NVFP4_SCALES_LINEAR) return NVFP4_ERR_ENUM;
  if (rounding < NVFP4_ROUND_NEAREST || rounding > NVFP4_ROUND_SR_HW) return NVFP4_ERR_ENUM;
  if (R < 0 || C < 0 || (C & 15) || ldx < C) return NVFP4_ERR_SHAPE;
  if (scale_layout == NVFP4_SCALES_SWIZZLED && ((R & 127) || (C & 63))) return NVFP4_ERR_SHAPE;
  if (!aligned16(x) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes) & 7u)) return NVFP4_ERR_ALIGN;
  if (R == 0 || C == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long nitems = (long long)R * (((C >> 3) + 63) >> 6);
  long long blocks = (nitems + 7) / 8;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const int linear = scale_layout == NVFP4_SCALES_LINEAR;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  uint2* cp = static_cast<uint2*>(codes);
  unsigned char* sp = static_cast<unsigned char*>(scales);
  // 256-bit loads need 32-byte aligned rows
  const bool wide = (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && (ldx & 15) == 0;
#define NVFP4_ROWS(RND)                                                                                              \
  do {                                                                                                               \
    if (wide) quant_rows_kernel<RND, true><<<(unsigned)blocks, 256, 0, st>>>(xp, ldx, cp, sp, amax, R, C, linear, seed, seed_dev, gs_out); \
    else quant_rows_kernel<RND, false><<<(unsigned)blocks, 256, 0, st>>>(xp, ldx, cp, sp, amax, R, C, linear, seed, seed_dev, gs_out);     \
  } while (0)
  switch (rounding) {
    case NVFP4_ROUND_NEAREST: NVFP4_ROWS(NVFP4_ROUND_NEAREST); break;
    case NVFP4_ROUND_SR_DITHER: NVFP4_ROWS(NVFP4_ROUND_SR_DITHER); break;
    case NVFP4_ROUND_SR_DITHER_K: NVFP4_ROWS(NVFP4_ROUND_SR_DITHER_K); break;
    default: NVFP4_ROWS(NVFP4_ROUND_SR_HW); break;
  }
#undef NVFP4_ROWS
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_quant_cols_rht(const void* x, int M, int C, void* codes, void* scales, int scale_layout,
                                    const float* amax, float* gs_out, unsigned signs, int rounding, unsigned seed,
                                    const unsigned* seed_dev, void* stream) {
  if (!x || !codes || !scales || !amax) return NVFP4_ERR_NULL;
  if (scale_layout != NVFP4_SCALES_SWIZZLED && scale_layout != NVFP4_SCALES_LINEAR) return NVFP4_ERR_ENUM;
  if (rounding < NVFP4_ROUND_NEAREST || rounding > NVFP4_ROUND_SR_HW) return NVFP4_ERR_ENUM;
  if (M < 0 || C < 0 || (M & 15) || (C & 7)) return NVFP4_ERR_SHAPE;
  if (scale_layout == NVFP4_SCALES_SWIZZLED && ((C & 127) || (M & 63))) return NVFP4_ERR_SHAPE;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 7u)) return NVFP4_ERR_ALIGN;
  if (M == 0 || C == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((C + 127) / 128), (unsigned)((M + 255) / 256));
  if (grid.y > 65535u) return NVFP4_ERR_TOO_LARGE;
  const int linear = scale_layout == NVFP4_SCALES_LINEAR;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  unsigned char* cp = static_cast<unsigned char*>(codes);
  unsigned char* sp = static_cast<unsigned char*>(scales);
  signs &= 0xFFFFu;
  switch (rounding) {
    case NVFP4_ROUND_NEAREST:
      quant_cols_rht_kernel<NVFP4_ROUND_NEAREST><<<grid, 256, 0, st>>>(xp, cp, sp, amax, M, C, linear, signs, seed, seed_dev, gs_out); break;
    case NVFP4_ROUND_SR_DITHER:
      quant_cols_rht_kernel<NVFP4_ROUND_SR_DITHER><<<grid, 256, 0, st>>>(xp, cp, sp, amax, M, C, linear, signs, seed, seed_dev, gs_out); break;
    case NVFP4_ROUND_SR_DITHER_K:
      quant_cols_rht_kernel<NVFP4_ROUND_SR_DITHER_K><<<grid, 256, 0, st>>>(xp, cp, sp, amax, M, C, linear, signs, seed, seed_dev, gs_out); break;
    default:
      quant_cols_rht_kernel<NVFP4_ROUND_SR_HW><<<grid, 256, 0, st>>>(xp, cp, sp, amax, M, C, linear, signs, seed, seed_dev, gs_out); break;
  }
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_quant_w2d(const void* w, int w_dtype, int N, int K, void* q, void* s, void* qt, void* st_,
                               int scale_layout, const float* amax, float* gs_out, void* stream) {
  if (!w || !amax || (!q && !qt) || (q && !s) || (qt && !st_)) return NVFP4_ERR_NULL;
  if (scale_layout != NVFP4_SCALES_SWIZZLED && scale_layout != NVFP4_SCALES_LINEAR) return NVFP4_ERR_ENUM;
  if (w_dtype != NVFP4_DTYPE_BF16 && w_dtype != NVFP4_DTYPE_FP32) return NVFP4_ERR_ENUM;
  if (N < 0 || K < 0 || (N & 15) || (K & 15)) return NVFP4_ERR_SHAPE;
  if (scale_layout == NVFP4_SCALES_SWIZZLED && ((N & 127) || (K & 127))) return NVFP4_ERR_SHAPE;
  if (!aligned16(w) || (q && (reinterpret_cast<uintptr_t>(q) & 3u)) || (qt && ((reinterpret_cast<uintptr_t>(qt) | reinterpret_cast<uintptr_t>(st_)) & 3u)))
    return NVFP4_ERR_ALIGN;
  if (N == 0 || K == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long nwarps = (long long)(((N >> 4) + 3) >> 2) * (K >> 4);
  long long blocks = (nwarps + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const int linear = scale_layout == NVFP4_SCALES_LINEAR;
  if (w_dtype == NVFP4_DTYPE_BF16)
    quant_w2d_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), static_cast<u32*>(q),
        static_cast<unsigned char*>(s), static_cast<u32*>(qt), static_cast<unsigned char*>(st_), amax, N, K, linear, gs_out);
  else
    quant_w2d_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const float*>(w), static_cast<u32*>(q),
        static_cast<unsigned char*>(s), static_cast<u32*>(qt), static_cast<unsigned char*>(st_), amax, N, K, linear, gs_out);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_swizzle_scales(const void* s_linear, long long lds, int R, int C16, void* s_swizzled, void* stream) {
  if (!s_linear || !s_swizzled) return NVFP4_ERR_NULL;
  if (R < 0 || C16 < 0 || (R & 127) || (C16 & 3) || lds < C16) return NVFP4_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(s_swizzled) & 3u) return NVFP4_ERR_ALIGN;
  if (R == 0 || C16 == 0) return NVFP4_OK;
  const long long total = (long long)R * (C16 >> 2);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  swizzle_scales_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(s_linear), lds, R, C16, static_cast<unsigned char*>(s_swizzled));
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

extern "C" int nvfp4_e2m1x4_sr(const float* y, const unsigned* rbits, void* codes, long long n4, void* stream) {
  if (!y || !rbits || !codes) return NVFP4_ERR_NULL;
  if (n4 < 0) return NVFP4_ERR_SHAPE;
  if (!aligned16(y) || (reinterpret_cast<uintptr_t>(rbits) & 3u) || (reinterpret_cast<uintptr_t>(codes) & 1u)) return NVFP4_ERR_ALIGN;
  if (n4 == 0) return NVFP4_OK;
  const long long blocks = (n4 + 255) / 256;
  if (blocks > 0x7FFFFFFFLL) return NVFP4_ERR_TOO_LARGE;
  e2m1x4_sr_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(y), rbits, static_cast<unsigned short*>(codes), n4);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}
