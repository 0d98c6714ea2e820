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

// Programmatic dependent launch.  A kernel launched through launch_kernel() may become resident while the kernel
// before it in the stream still runs: its prologue (barrier set-up, tensor-memory allocation, constant tables) then
// overlaps the predecessor's last wave, and the launch latency disappears.  The contract every kernel launched this
// way keeps: pdl_trigger() first thing (its own successor may be staged), and pdl_wait() executed by every thread
// before the first access to global memory -- it returns once all earlier kernels of the stream have completed and
// their writes are visible.  Both are no-ops in a kernel launched the ordinary way.  Such a kernel also reads global
// memory only past the L1 cache (ld.global.cg, TMA, atomics): it is launched, and its SM's L1 invalidated, while
// older kernels still run, so a line one of them reads afterwards (say a scale word at an address the allocator
// hands out again) would otherwise still sit in L1, stale, when the staged kernel gets to read the new value.
bool nvfp4_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t nvfp4_launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = nvfp4_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

namespace nvfp4 {

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// loads served by L2 (see above)
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ u32 ld_cg_u32(const u32* p) {
  u32 v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

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

// Internal modes of the operand emitters (llm-1b/emit.cu arithmetic: block scale and values by
// multiplications, no exact divisions); not part of the public rounding enum.
#define NVFP4_EMIT_NEAREST 4   /* y = v * (inv/bs), round to nearest */
#define NVFP4_EMIT_SR      5   /* same, 11-bit mantissa dither driven by a per-thread LCG */
#define NVFP4_EMIT_SR_HW   6   /* same scaling, hardware cvt.rs with this library's counter-based words */

// dither with bits already in place (11 random bits at positions 11..21), truncate to the E2M1
// grid, clamp to 6, restore the sign (llm-1b/emit.cu:38-43)
__device__ __forceinline__ float sr_dither11(float v, u32 r22) {
  const float a = fabsf(v), lift = a < 1.f ? 1.f : 0.f;
  const float b = __fadd_rn(a, lift);
  const float q = __fsub_rn(__uint_as_float((__float_as_uint(b) + r22) & 0xFFC00000u), lift);
  return __uint_as_float(__float_as_uint(fminf(q, 6.f)) | (__float_as_uint(v) & 0x80000000u));
}
// the emitters' generator (llm-1b/emit.cu:45) and its n-step jump  s -> A^n s + C_n
__device__ __forceinline__ u32 lcg_step(u32& s) { s = s * 1664525u + 1013904223u; return s ^ (s >> 16); }
__host__ __device__ constexpr u32 lcg_jump_mul(int n) { u32 a = 1u; for (int i = 0; i < n; i++) a *= 1664525u; return a; }
__host__ __device__ constexpr u32 lcg_jump_add(int n) { u32 c = 0u; for (int i = 0; i < n; i++) c = c * 1664525u + 1013904223u; return c; }

// byte offset of the scale of (row r, 16-block c) in the swizzled layout; ncb = (C/16)/4
__device__ __forceinline__ long long sw_off(long long r, int c, int ncb) {
  return ((r >> 7) * ncb + (c >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

// ---- packed FP32 pairs (sm_100 f32x2 arithmetic: one issue slot for two IEEE operations) ----
__device__ __forceinline__ u64 f2_pack(float lo, float hi) { u64 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ float f2_lo(u64 p) { return __uint_as_float((u32)p); }
__device__ __forceinline__ float f2_hi(u64 p) { return __uint_as_float((u32)(p >> 32)); }
__device__ __forceinline__ u64 f2_mul(u64 a, u64 b) { u64 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ u64 f2_add(u64 a, u64 b) { u64 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ u64 f2_sub(u64 a, u64 b) { u64 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ u64 f2_fma(u64 a, u64 b, u64 c) { u64 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
// max(|a|, |b|, |c|) in one instruction (sm_100 three-input max)
__device__ __forceinline__ float absmax3(float a, float b, float c) {
  float d;
  asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// the two bf16 values of a packed word as an FP32 pair (low half first)
__device__ __forceinline__ u64 f2_from_bf16x2(u32 w) { return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u)); }

struct Block32 { u32 w[8]; };   // one 16-value bf16 block

// max |.| over the 16 values of 8 packed pairs
__device__ __forceinline__ float absmax16(const u64 (&P)[8]) {
  float m = absmax3(f2_lo(P[0]), f2_hi(P[0]), f2_lo(P[1]));
  m = absmax3(m, f2_hi(P[1]), f2_lo(P[2]));
  m = absmax3(m, f2_hi(P[2]), f2_lo(P[3]));
  m = absmax3(m, f2_hi(P[3]), f2_lo(P[4]));
  m = absmax3(m, f2_hi(P[4]), f2_lo(P[5]));
  m = absmax3(m, f2_hi(P[5]), f2_lo(P[6]));
  m = absmax3(m, f2_hi(P[6]), f2_lo(P[7]));
  return absmax3(m, f2_hi(P[7]), m);
}

// Correctly rounded -(a/b) from nrb = -RN(1/b): one multiply and two fused multiply-adds
// (Markstein's final division step: m = RN(a*nrb) is within an ulp of -a/b, the remainder
// a + m*b is exact in one FMA, and RN(m + rem*nrb) = -RN(a/b) unless b's significand is all
// ones).  The divisors here never have an all-ones significand: 6 and the E4M3 block scales have
// at most 4 significant bits, and a tensor scale RN(amax/2688) would need amax strictly between
// two neighbouring floats (2688 * (2^(e+1) - ulp) lies 0.33 to 0.98 of amax's ulp below the
// representable 1.3125 * 2^(e+12)).  The form returns the NEGATED quotient so that no operand
// needs a sign flip and a zero keeps its sign exactly: a = +0 gives -0, a = -0 gives +0.  Two
// divisions in a row therefore give +(a/b1)/b2 with the sign of a, zeros included.
__device__ __forceinline__ float ndiv(float a, float b, float nrb) {
  const float m = __fmul_rn(a, nrb);
  return __fmaf_rn(__fmaf_rn(m, b, a), nrb, m);
}
__device__ __forceinline__ u64 f2_ndiv(u64 a, u64 b, u64 nrb) {
  const u64 m = f2_mul(a, nrb);
  return f2_fma(f2_fma(m, b, a), nrb, m);
}

// t / bs for a block scale bs (an E4M3 value: at most 4 significant bits), from the negated reciprocal split in two
// words, nrh = -RD(1/bs) (rounded DOWN, so that the remainder 1/bs - RD(1/bs) is never negative and both words
// have the same sign: a zero numerator then keeps its sign through the sum) and nrl = -RN(1/bs - RD(1/bs)):
// RN(t*nrh + RN(t*nrl)).  The quotient feeds a
// round-to-E2M1 whose result only depends on how t/bs compares with the seven rounding boundaries b (0.25 .. 5).
// RN(t/bs) < b, = b, > b exactly when t < c, = c, > c for c = b*bs (exactly representable), and this form --
// accurate to 2^-46, against 0.03 ulp between the nearest t/bs and a rounding midpoint next to b -- maps
// pred(c), c, succ(c) below, onto and above b for every scale byte and boundary (checked exhaustively by
// tests/test_division_model.py); it is monotone in t, so the codes equal those of the correctly rounded division.
// Like ndiv() it takes the NEGATED numerator and returns the quotient with the original sign, zeros included.
__device__ __forceinline__ u64 f2_div_bs(u64 nt, u64 nrh, u64 nrl) { return f2_fma(nt, nrh, f2_mul(nt, nrl)); }

// Per-tensor constants of a quantizer launch.
struct TensorScale {
  float gs;      // max(k*amax/2688, 1e-30)/pre: the FP32 tensor scale the values are divided by
  float nrgs;    // -RN(1/gs)
  float inv_gs;  // pre*2688/(k*amax), 0 for an all-zero tensor: the reference kernels' scale (llm-1b/nvq.cu:101)
  u32 lut;       // shared-memory address of 128 float2 entries indexed by the scale byte, see make_tensor_scale
};

constexpr int kLutFloats = 256;

// Fill the per-CTA table: for round to nearest  lut[sb] = {-RD(1/bs), -RN(1/bs - RD(1/bs))} (see f2_div_bs),  for stochastic rounding
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
  t.nrgs = -__frcp_rn(t.gs);
  t.inv_gs = am > 0.f ? __fmul_rn(__fdiv_rn(kFp4E4m3, am), pre) : 0.f;
  t.lut = (u32)__cvta_generic_to_shared(lut);
  if (threadIdx.x < 128) {
    const float bsf = e4m3_dec(threadIdx.x);
    // entry 0 (underflowed block): -0 / +0 make every scaled value a zero with the input's sign
    float m = (ROUNDING == NVFP4_ROUND_NEAREST) ? -0.f : 0.f;
    float second = (ROUNDING == NVFP4_ROUND_NEAREST) ? -0.f : bsf;
    if (threadIdx.x >= 1 && threadIdx.x <= 126) {
      if (ROUNDING == NVFP4_ROUND_NEAREST) {
        const float rh = __frcp_rd(bsf);
        const float res = __fmaf_rn(-rh, bsf, 1.f);        // exact and >= +0: 1 - rh*bs has few significant bits
        m = -rh;
        second = -__fmul_rn(res, rh);                       // -(1/bs - rh) to 2^-24 of itself
      } else {
        m = __fdiv_rn(t.inv_gs, bsf);                       // emit modes: inv/bs too
      }
    }
    reinterpret_cast<float2*>(lut)[threadIdx.x] = make_float2(m, second);
  }
  __syncthreads();
  return t;
}

// table entry of a scale byte (explicit shared-memory load: a generic one takes the long path)
__device__ __forceinline__ float2 lut_entry(const TensorScale& ts, u32 sb) {
  float2 r;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "r"(ts.lut + sb * 8u));
  return r;
}

// Scale byte of a block:  e4m3(min((bmax/gs)/6, 448))  in IEEE FP32 (the reference's torch path).
__device__ __forceinline__ u32 block_scale_byte(float bmax, const TensorScale& ts) {
  return e4m3_enc(ndiv(ndiv(bmax, ts.gs, ts.nrgs), 6.0f, -0.16666667163372039794921875f));
}
// the emitters' form (llm-1b/emit.cu:85): e4m3((bmax * inv) * (1/6))
__device__ __forceinline__ u32 block_scale_byte_mul(float bmax, const TensorScale& ts) {
  return e4m3_enc(__fmul_rn(__fmul_rn(bmax, ts.inv_gs), 1.f / 6.f));
}

// Random words of the hardware-SR mode, a counter-based generator of this library: one word per group of four
// consecutive elements of a block.  key = mix(blk * 0x9E3779B9 ^ hash32(seed)) with one xorshift-multiply round
// (hash32(seed) does not depend on the block and is computed once per thread); word g = lo ^ hi of the 64-bit
// product key * mult[g].  Seven plus two instructions per block and word; bit balance, adjacent-block and
// cross-bit correlations of the words are at the level of the full hash32 mixer.
__device__ __forceinline__ u32 sr_hw_block_key(u32 seed, u32 blk_idx) {
  u32 t = (blk_idx * 0x9E3779B9u) ^ hash32(seed);
  t ^= t >> 16; t *= 0x7feb352du; t ^= t >> 15;
  return t;
}
__device__ __forceinline__ u32 sr_hw_word(u32 key, int g) {
  const u32 mult[4] = {0x9E3779B1u, 0x85EBCA77u, 0xC2B2AE3Du, 0x27D4EB2Fu};
  const u64 p = (u64)key * (u64)mult[g];
  return (u32)p ^ (u32)(p >> 32);
}

// Per-block key of the random stream of a rounding mode (0 where the mode needs none).
template <int ROUNDING>
__device__ __forceinline__ u32 block_key(u32 seed, u32 blk_idx) {
  if (ROUNDING == NVFP4_ROUND_SR_HW) return sr_hw_block_key(seed, blk_idx);
  if (ROUNDING == NVFP4_ROUND_SR_DITHER) return hash32(seed ^ hash32(blk_idx));
  return 0u;
}

// Eight scaled values (elements 8h .. 8h+7 of a block, h = 0 or 1) -> one 32-bit word of codes.
template <int ROUNDING>
__device__ __forceinline__ u32 round8(float (&y)[8], u32& key, u32 seed, u32 elt_idx, int h) {
  if (ROUNDING == NVFP4_EMIT_SR) {
    // `key` is the running LCG state of this thread: one step per pair of values
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const u32 rnd = lcg_step(key);
      y[j] = sr_dither11(y[j], (rnd << 11) & 0x3FF800u);
      y[j + 1] = sr_dither11(y[j + 1], (rnd >> 5) & 0x3FF800u);
    }
    return e2m1x8_rn(y);
  }
  if (ROUNDING == NVFP4_ROUND_SR_HW || ROUNDING == NVFP4_EMIT_SR_HW)
    return e2m1x4_rs(y[0], y[1], y[2], y[3], sr_hw_word(key, 2 * h)) | (e2m1x4_rs(y[4], y[5], y[6], y[7], sr_hw_word(key, 2 * h + 1)) << 16);
  if (ROUNDING == NVFP4_ROUND_SR_DITHER || ROUNDING == NVFP4_ROUND_SR_DITHER_K) {
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const u32 i = 8u * (u32)h + (u32)j;
      const u32 hh = (ROUNDING == NVFP4_ROUND_SR_DITHER) ? hash32(key + i) : hash32(seed ^ (elt_idx + i) * 0x9E3779B9u);
      y[j] = sr_dither(y[j], hh);
      y[j + 1] = sr_dither(y[j + 1], (hh >> 10) | (hh << 22));
    }
  }
  return e2m1x8_rn(y);
}

// Quantize one block of 16 values that share a scale.
//   v      the 16 values (x, or the Hadamard-transformed x before its power-of-two factor)
//   sb     the block's scale byte (block_scale_byte of max |v| over everything that shares the scale)
// Round to nearest:  y = (v/gs)/bs, the torch path's operation order: v/gs correctly rounded by f2_ndiv()
//   (three packed FMA-pipe instructions per two values), the division by the block scale by f2_div_bs()
//   (two), which gives the same codes as a correctly rounded one; no branch.
// Stochastic rounding:  y = v * (inv_gs / bs), the reference kernels' form (llm-1b/nvq.cu:50,54) in
//   IEEE arithmetic; the torch path draws torch.rand and so defines no bit-level result.
// A block whose scale byte is 0 needs no branch: table entry 0 turns every value into a zero with
// the sign of the input, which the converts keep.
template <int ROUNDING>
__device__ __forceinline__ uint2 quant_block16(const u64 (&P)[8], u32 sb, const TensorScale& ts, u32 seed,
                                               u32 blk_idx, u32 elt_idx) {
  const float2 kf = lut_entry(ts, sb);
  u32 key = block_key<ROUNDING>(seed, blk_idx);
  const u64 G = f2_pack(ts.gs, ts.gs), NRG = f2_pack(ts.nrgs, ts.nrgs);
  const u64 B = f2_pack(kf.y, kf.y), K = f2_pack(kf.x, kf.x);
  u32 w[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    float y[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const u64 r = (ROUNDING == NVFP4_ROUND_NEAREST) ? f2_div_bs(f2_ndiv(P[4 * h + j], G, NRG), K, B) : f2_mul(P[4 * h + j], K);
      y[2 * j] = f2_lo(r); y[2 * j + 1] = f2_hi(r);
    }
    w[h] = round8<ROUNDING>(y, key, seed, elt_idx, h);
  }
  return make_uint2(w[0], w[1]);
}

// Two blocks at once, interleaved: P[i] = (value i of block 0, value i of block 1), e.g. two
// neighbouring columns of 16 tokens.  Same arithmetic as quant_block16, the two blocks' scales
// riding in the two halves of the packed constants.
template <int ROUNDING>
__device__ __forceinline__ void quant_block16x2(const u64 (&P)[16], const TensorScale& ts, u32 seed, u32 blk0, u32 blk1,
                                                u32 key0, u32 key1, uint2& o0, uint2& o1, u32& sb0, u32& sb1,
                                                float* bmax_out = nullptr) {
  constexpr bool EMIT = ROUNDING == NVFP4_EMIT_NEAREST || ROUNDING == NVFP4_EMIT_SR || ROUNDING == NVFP4_EMIT_SR_HW;
  float m0 = absmax3(f2_lo(P[0]), f2_lo(P[1]), f2_lo(P[2])), m1 = absmax3(f2_hi(P[0]), f2_hi(P[1]), f2_hi(P[2]));
#pragma unroll
  for (int i = 3; i < 15; i += 2) { m0 = absmax3(m0, f2_lo(P[i]), f2_lo(P[i + 1])); m1 = absmax3(m1, f2_hi(P[i]), f2_hi(P[i + 1])); }
  m0 = absmax3(m0, f2_lo(P[15]), m0); m1 = absmax3(m1, f2_hi(P[15]), m1);
  if (bmax_out) *bmax_out = fmaxf(m0, m1);
  sb0 = EMIT ? block_scale_byte_mul(m0, ts) : block_scale_byte(m0, ts);
  sb1 = EMIT ? block_scale_byte_mul(m1, ts) : block_scale_byte(m1, ts);
  const float2 k0 = lut_entry(ts, sb0), k1 = lut_entry(ts, sb1);
  const u64 G = f2_pack(ts.gs, ts.gs), NRG = f2_pack(ts.nrgs, ts.nrgs);
  const u64 B = f2_pack(k0.y, k1.y), K = f2_pack(k0.x, k1.x);
  u32 w0[2], w1[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    float y0[8], y1[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const u64 r = (ROUNDING == NVFP4_ROUND_NEAREST) ? f2_div_bs(f2_ndiv(P[8 * h + j], G, NRG), K, B) : f2_mul(P[8 * h + j], K);
      y0[j] = f2_lo(r); y1[j] = f2_hi(r);
    }
    w0[h] = round8<ROUNDING>(y0, key0, seed, blk0 * 16u, h);
    w1[h] = round8<ROUNDING>(y1, key1, seed, blk1 * 16u, h);
  }
  o0 = make_uint2(w0[0], w0[1]);
  o1 = make_uint2(w1[0], w1[1]);
}

}  // namespace nvfp4
