// One-read NVFP4 quantizer for sm_100a, tensor-core fed: the row operand (1x16 blocks along the
// columns) and the transposed RHT16 operand (16-token blocks per column) of a bf16 [M, C] tensor
// from a single pass over HBM.
//
// What the quantizer's threads spend their issue slots on is not the arithmetic of the format but
// getting values into the right thread in FP32: unpacking bf16 pairs, and for the transposed operand
// walking a shared-memory tile column-wise and staging the outputs back into rows.  Here the tensor
// core does that data movement, exactly:
//   * TMA streams 128-token x 128-column tiles (two 128 x 64 boxes, 128-byte swizzle) into a ring;
//   * one thread issues tcgen05.mma kind::f16 (bf16 in, FP32 out) with tiny 0/+-1 matrices as the B
//     operand.  Row operand: D1[token, col] = X * I (K-major A): the tile converted to FP32, one
//     token per tensor-memory lane.  Transposed operand: D2[col, slot] = X^T * P (MN-major A straight
//     from the same tile, no transpose in shared memory): one column per lane, and P both applies
//     the Hadamard sign vector and interleaves two 16-token blocks (slot 2k = token k of the first
//     block, 2k+1 = token k of the second), so that the butterflies run on packed FP32 pairs.
//     Every output is ONE product +-1 * x plus exact zeros, so D holds the bf16 values bit for bit
//     whatever the accumulation order;
//   * eight consumer warps read their lane quadrant with tcgen05.ld (16 values of a 1x16 block, or 32
//     values of two 16-token blocks, per instruction), quantize, and store 32 contiguous bytes of
//     codes per thread for each operand: no staging, no shared-memory traffic in the consumers.
// One difference to the scalar kernels: an input that is exactly -0 arrives as +0 (an IEEE sum of
// signed zeros), so its code is 0x0 where the scalar kernels and the reference's convert give 0x8; the
// dequantized value is the same.  Inf/NaN inputs poison their 16-value group (0 * Inf), as they
// poison the tensor's amax in every implementation.
//
// Optional mode (nvfp4_quant_tile_set_path(2)): the 16-point Hadamard transform itself in the MMA -- P then holds
// the rows of H diag(s) instead of a signed permutation and the consumers skip the butterflies.  The tensor core
// sums the 16 signed bf16 values of a block in FP32 in its own order, so the result equals the butterflies' whenever
// the exact sum is representable (all values of a block within 2^12 of its largest: every partial sum then fits 24
// bits) and can differ in the last bit otherwise: not the bit-exact default.
//
// Two CTAs per SM, each with nine warps (one loads tiles and issues the MMAs, eight quantize) and 256
// tensor-memory columns used as two buffers, so that MMAs into one buffer run while the consumers work on
// the other; the consumers' tensor-memory loads are software-pipelined.  Every mbarrier wait is bounded: on
// expiry the CTA raises an abort flag, stores a role code in the quantizer status word, lets copies
// in flight land, frees its tensor memory and returns.
#include "tma.cuh"

namespace nvfp4 {

constexpr int kQTok = 128;                    // tokens per tile
constexpr int kQCol = 128;                    // columns per tile (two TMA boxes of 64)
constexpr int kQBoxBytes = kQTok * 64 * 2;    // 16 KB
constexpr int kQTileBytes = 2 * kQBoxBytes;
constexpr int kQStages = 3;
constexpr int kQConsumerWarps = 8;
constexpr int kQThreads = 32 * (1 + kQConsumerWarps);
constexpr int kQPermBytes = 32 * 128;
constexpr int kQSmem = kQStages * kQTileBytes + 1024 /*I16, padded*/ + 1024 + 2 * kQPermBytes + 1024 /*alignment slack*/;
constexpr int kQTmemCols = 256;               // two buffers of 128 columns

__device__ int g_quant_tc_status;             // 0, or the role code of the first wait that expired

struct TcParams {
  unsigned char* codes_r; unsigned char* scales_r;    // row operand [M, C/2], scales [M, C/16]
  unsigned char* codes_c; unsigned char* scales_c;    // transposed operand [C, M/2], scales [C, M/16]
  const float* amax;
  float* gs_r_out; float* gs_c_out;
  int M, C, linear;
  u32 signs;
  u32 seed_r, seed_c;
  const u32* seed_r_dev; const u32* seed_c_dev;
  int tc_rht;       // 1: the 16-point Hadamard transform itself runs in the MMA (B = signed Hadamard rows), see below
};

// ---- tcgen05 wrappers (cta_group::1)
__device__ __forceinline__ void q_tmem_alloc(u32 smem_dst, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void q_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void q_tmem_dealloc(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void q_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q_commit(u32 bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void q_mma_bf16(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void q_ld32(u32 taddr, u32 (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void q_ld16(u32 taddr, u32 (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// Wait for this thread's tensor-memory loads.  The loaded registers pass through the statement as in/out operands,
// so that the compiler cannot schedule a use of them before the wait.
__device__ __forceinline__ void q_wait_ld16(u32 (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]) :: "memory");
}
__device__ __forceinline__ void q_wait_ld32(u32 (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}

__device__ __forceinline__ u64 q_pack64(u32 lo, u32 hi) {
  u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Shared-memory matrix descriptors (tcgen05): start address >> 4 in bits 0..13, leading byte offset >> 4 in
// bits 16..29, stride byte offset >> 4 in bits 32..45, version 1 at bit 46, 128-byte swizzle (2) in bits 61..63.
//   K-major operand (rows of 128 bytes along K): stride offset = 1024 B between 8-row groups, leading offset unused (1)
//   MN-major operand (rows of 128 bytes along M, one row per K index): leading offset = distance between 64-element
//   groups along M (the two TMA boxes, 16 KB apart), stride offset = 1024 B between 8-row (8 K index) groups
constexpr u32 kQDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ u64 q_desc_k(u32 saddr) { return q_pack64(((saddr & 0x3FFFFu) >> 4) | (1u << 16), kQDescHi); }
__device__ __forceinline__ u64 q_desc_mn(u32 saddr) {
  return q_pack64(((saddr & 0x3FFFFu) >> 4) | ((u32)(kQBoxBytes >> 4) << 16), kQDescHi);
}
// Instruction descriptor, kind::f16: FP32 accumulator (1 at bit 4), A and B bf16 (1 at bits 7 and 10), A major at
// bit 15 (1 = MN-major), B K-major, N / 8 at bit 17, M / 16 at bit 24.
__host__ __device__ constexpr u32 q_idesc(int n, bool a_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((u32)(n >> 3) << 17) | ((u32)(128 >> 4) << 24);
}

__device__ __forceinline__ void q_settle_copies() {
  const u64 t0 = globaltimer_ns();
  while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
}

// Walks the tiles of one CTA in (token tile, column tile) coordinates without a division per tile.
struct TcWalk {
  int mt, ct, dq, dr, nct, nmt;
  __device__ __forceinline__ TcWalk(int M, int C) {
    nct = C / kQCol; nmt = M / kQTok;
    mt = (int)blockIdx.x / nct; ct = (int)blockIdx.x - mt * nct;
    dq = (int)gridDim.x / nct; dr = (int)gridDim.x - dq * nct;
  }
  __device__ __forceinline__ bool valid() const { return mt < nmt; }
  __device__ __forceinline__ void next() { mt += dq; ct += dr; if (ct >= nct) { ct -= nct; mt++; } }
};

template <int ROUNDING, bool ROWS, bool COLS, bool TCRHT>
__global__ void __launch_bounds__(kQThreads, 2) quant_tc_kernel(const __grid_constant__ CUtensorMap map, const TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) float lut_r[kLutFloats];
  __shared__ __align__(8) float lut_c[kLutFloats];
  __shared__ __align__(8) u64 bars[2 * kQStages + 4];
  __shared__ u32 tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const u32 tiles0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const u32 i16_s = tiles0 + kQStages * kQTileBytes;            // 16 rows x 128 B, then padding to 1024
  const u32 p1_s = i16_s + 2048, p2_s = p1_s + kQPermBytes;     // 32 rows x 128 B each (1024-byte aligned)
  const u32 full0 = smem_u32(bars), empty0 = full0 + 8 * kQStages;
  const u32 tfull = empty0 + 8 * kQStages, tempty = tfull + 16;     // two tensor-memory buffers: [2] each

  // ---- barriers first, and the loads of the first tiles at once: their latency (1-2 us) runs under the set-up below
  // (tables, tensor-memory allocation), which matters for tensors of a few tens of MB where a launch lasts 20-40 us
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < kQStages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(tfull + 8 * b, 1); mbar_init(tempty + 8 * b, kQConsumerWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  auto load_tile = [&](const TcWalk& tw, u32 stage) {
    if (elect_one()) {
      const u32 bar = full0 + 8 * stage, dst = tiles0 + stage * kQTileBytes;
      mbar_arrive_expect_tx(bar, kQTileBytes);
      tma_load_2d(dst, &map, tw.ct * kQCol, tw.mt * kQTok, bar);
      tma_load_2d(dst + kQBoxBytes, &map, tw.ct * kQCol + 64, tw.mt * kQTok, bar);
    }
    __syncwarp();
  };
  TcWalk ahead(p.M, p.C);            // the producer's position: kQStages tiles ahead of the MMAs
  if (warp == 0) {
    __syncwarp();
    pdl_wait();                      // x may be the previous kernel's output
    for (u32 s = 0; s < (u32)kQStages && ahead.valid(); s++, ahead.next()) load_tile(ahead, s);
  }

  // ---- constants of the MMAs: identity and the two sign/interleave matrices, in the K-major 128-byte-swizzle
  // layout (row n at n * 128 bytes, its 16-byte chunk j at position j ^ (n & 7)); only K columns 0..15 are read
  for (u32 i = threadIdx.x; i < (2048u + 2u * kQPermBytes) / 4u; i += kQThreads)
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(i16_s + 4u * i), "r"(0u) : "memory");
  __syncthreads();
  if (threadIdx.x < 16) {
    const u32 n = threadIdx.x;                                  // I16: row n has 1.0 at K index n
    const u32 off = n * 128u + ((((n >> 3) ^ (n & 7u)) << 4) | ((n & 7u) << 1));
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(i16_s + off), "h"((unsigned short)0x3F80) : "memory");
  } else if (threadIdx.x >= 32 && threadIdx.x < 64) {
    // P1 row 2k and P2 row 2k+1 hold s_k at K index k: slot 2k = token k of the first 16-token block, slot 2k+1 =
    // token k of the second; bit k of `signs` negates token k
    const u32 n = threadIdx.x - 32u, k = n >> 1;
    const u32 base = (n & 1u) ? p2_s : p1_s;
    if (!TCRHT) {
      const unsigned short v = ((p.signs >> k) & 1u) ? (unsigned short)0xBF80 : (unsigned short)0x3F80;
      const u32 off = n * 128u + ((((k >> 3) ^ (n & 7u)) << 4) | ((k & 7u) << 1));
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(base + off), "h"(v) : "memory");
    } else {
      // Hadamard in the MMA: row 2k (+1) holds row k of H diag(s), H[k][i] = (-1)^popcount(k & i) (Sylvester order,
      // the order the butterflies of strides 1, 2, 4, 8 produce); slot 2k + j = transformed value k of block j
#pragma unroll
      for (u32 i = 0; i < 16; i++) {
        const u32 neg = (__popc(k & i) ^ (p.signs >> i)) & 1u;
        const u32 off = n * 128u + ((((i >> 3) ^ (n & 7u)) << 4) | ((i & 7u) << 1));
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(base + off), "h"(neg ? (unsigned short)0xBF80 : (unsigned short)0x3F80) : "memory");
      }
    }
  }
  // the tensor core reads shared memory through the asynchronous proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    q_tmem_alloc(smem_u32(&tmem_slot), kQTmemCols);
    q_tmem_relinquish();
  }
  // everything above touches shared and tensor memory only; the tensor's amax is the previous kernel's result
  pdl_wait();
  const float amax = ld_cg_f32(p.amax);
  const bool first = blockIdx.x == 0 && threadIdx.x == 0;
  TensorScale ts_r, ts_c;
  if (ROWS) ts_r = make_tensor_scale<ROUNDING>(amax, 1.f, lut_r, first ? p.gs_r_out : nullptr);
  // the x0.25 that follows the butterflies is folded into the tensor scale (a power of two)
  if (COLS) ts_c = make_tensor_scale<ROUNDING>(amax, 4.f, lut_c, first ? p.gs_c_out : nullptr, 0.25f);
  q_fence_before();
  __syncthreads();
  q_fence_after();
  const u32 tmem_base = tmem_slot;

  // Tensor memory holds two buffers of 128 columns, each with its own full / empty barrier.  With both outputs
  // buffer 0 is D1 (row operand) and buffer 1 is D2 (transposed operand) of the same tile: the consumers hand D1
  // back after its last load, so the next tile's row MMAs run while they quantize the transposed half, and vice
  // versa.  With one output the two buffers hold the same kind of result for alternating tiles.
  constexpr bool BOTH = ROWS && COLS;
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer and MMA issuer (one warp)
    // Loads run kQStages tiles ahead (the first ones were issued at the top of the kernel): the load of tile
    // n + kQStages is issued once the MMAs of tile n have released their stage.
    constexpr u32 idesc_row = q_idesc(16, false), idesc_col = q_idesc(32, true);
    const u64 b_i16 = q_desc_k(i16_s), b_p1 = q_desc_k(p1_s), b_p2 = q_desc_k(p2_s);
    // D[token, 64 b + 16 kk + n] = sum_k X[token, 64 b + 16 kk + k] * I[n, k]
    auto row_mmas = [&](u32 tile, u32 d) {
#pragma unroll
      for (int b = 0; b < 2; b++)
#pragma unroll
        for (int kk = 0; kk < 4; kk++)
          q_mma_bf16(d + (u32)(64 * b + 16 * kk), q_desc_k(tile + b * kQBoxBytes + kk * 32), b_i16, idesc_row, 0u);
    };
    // D[col, 32 pr + 2 k + j] = s_k * X[32 pr + 16 j + k, col]   (j = 0: first K = 16 step, j = 1: second)
    auto col_mmas = [&](u32 tile, u32 d) {
#pragma unroll
      for (int pr = 0; pr < 4; pr++) {
        q_mma_bf16(d + (u32)(32 * pr), q_desc_mn(tile + (32 * pr) * 128), b_p1, idesc_col, 0u);
        q_mma_bf16(d + (u32)(32 * pr), q_desc_mn(tile + (32 * pr + 16) * 128), b_p2, idesc_col, 1u);
      }
    };
    u32 stage = 0, phase = 0, n = 0;
    for (TcWalk tw(p.M, p.C); tw.valid(); tw.next(), n++) {
      // buffers and their parities: with both outputs each buffer is used once per tile, else once per two tiles
      const u32 buf0 = BOTH ? 0u : (n & 1u), par = BOTH ? (n & 1u) : ((n >> 1) & 1u);
      bool ok = mbar_wait(full0 + 8 * stage, phase, abort_flag);                 // the tile's bytes have landed
      ok = ok && mbar_wait(tempty + 8 * buf0, par ^ 1u, abort_flag);             // and the first buffer is free
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicCAS(&g_quant_tc_status, 0, 1);
        break;
      }
      q_fence_after();
      const u32 tile = tiles0 + stage * kQTileBytes;
      if (elect_one()) {
        if (ROWS) row_mmas(tile, tmem_base + 128u * buf0); else col_mmas(tile, tmem_base + 128u * buf0);
        if (!BOTH) q_commit(empty0 + 8 * stage);      // the stage is free once the MMAs have read it
        q_commit(tfull + 8 * buf0);                   // and the consumers may read this buffer
      }
      __syncwarp();
      if (BOTH) {
        if (!__all_sync(0xffffffffu, mbar_wait(tempty + 8, par ^ 1u, abort_flag))) {
          if (lane == 0) atomicCAS(&g_quant_tc_status, 0, 1);
          break;
        }
        q_fence_after();
        if (elect_one()) {
          col_mmas(tile, tmem_base + 128u);
          q_commit(empty0 + 8 * stage);
          q_commit(tfull + 8);
        }
        __syncwarp();
      }
      if (ahead.valid()) {
        // refill this stage as soon as the MMAs just issued have read it
        if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * stage, phase, abort_flag))) {
          if (lane == 0) atomicCAS(&g_quant_tc_status, 0, 3);
          break;
        }
        load_tile(ahead, stage);
        ahead.next();
      }
      if (++stage == kQStages) { stage = 0; phase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------------ consumers (warps 1..8)
    // The tensor-memory loads are software-pipelined, also across tiles: while a chunk (a 1x16 block of the row
    // operand, or two 16-token blocks of the transposed one) is being quantized, the load of the next chunk is in
    // flight, and the first chunk of the next tile is requested before the last chunk of this one is quantized.
    const int quad = warp & 3;                      // tensor-memory lanes 32 * quad .. + 31 (fixed by the warp index)
    const int half = (warp - 1) >> 2;               // columns 64 * half .. + 63 of a buffer
    u32 seed_r = p.seed_r, seed_c = p.seed_c;
    if (ROUNDING != NVFP4_ROUND_NEAREST) {
      if (p.seed_r_dev) seed_r = ld_cg_u32(p.seed_r_dev);
      if (p.seed_c_dev) seed_c = ld_cg_u32(p.seed_c_dev);
    }
    const int nblk = p.C >> 4;                      // 16-column blocks per row
    const int nmb = p.M >> 4;                       // 16-token blocks per column
    const u32 t_lane = tmem_base + ((u32)(quad * 32) << 16) + (u32)(64 * half);
    // per-thread output positions of tile (0, 0); a tile adds a multiple of its coordinates
    const long long tok0 = quad * 32 + lane, col0 = quad * 32 + lane;
    const long long row_code_stride = (long long)kQTok * (p.C >> 1), col_code_stride = (long long)kQCol * nmb * 8;
    const long long row_sc0 = p.linear ? tok0 * nblk + half * 4 : (long long)half * 512 + lane * 16 + quad * 4;
    const long long col_sc0 = p.linear ? col0 * nmb + half * 4 : (long long)half * 512 + lane * 16 + quad * 4;

    bool alive = true;
    // wait for buffer `buf` to be full; false (for the whole warp) when the CTA is aborting
    auto wait_full = [&](u32 buf, u32 par) {
      if (!__all_sync(0xffffffffu, mbar_wait_parked(tfull + 8 * buf, par, abort_flag))) {
        if (lane == 0) atomicCAS(&g_quant_tc_status, 0, 2);
        alive = false;
      } else {
        q_fence_after();
      }
      return alive;
    };
    // a buffer has been read completely: the next MMAs into it may start
    auto release = [&](u32 buf) {
      q_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + 8 * buf);
    };

    TcWalk tw(p.M, p.C);
    u32 n = 0;
    u32 first16[16], first32[32];                   // the first chunk of the current tile (loaded one tile ahead)
    if (tw.valid() && wait_full(0u, 0u)) {
      if (ROWS) q_ld16(t_lane, first16); else q_ld32(t_lane, first32);
    }
    for (; alive && tw.valid(); n++) {
      const int mt = tw.mt, ct = tw.ct;
      const u32 buf0 = BOTH ? 0u : (n & 1u), par = BOTH ? (n & 1u) : ((n >> 1) & 1u);
      tw.next();
      const bool more = tw.valid();
      const u32 nbuf = BOTH ? 0u : ((n + 1u) & 1u), npar = BOTH ? ((n + 1u) & 1u) : (((n + 1u) >> 1) & 1u);

      const long long tok = (long long)mt * kQTok + tok0;      // lane = token of the row operand
      const long long col = (long long)ct * kQCol + col0;      // lane = column of the transposed operand
      const int blk0 = ct * (kQCol / 16) + half * 4;           // first of this warp's four 1x16 blocks of a row
      const int mb0 = mt * (kQTok / 16) + half * 4;            // first of this warp's four 16-token blocks of a column
      uint2 orow[4], ocol[4];
      u32 sb_row = 0u, sb_col = 0u;

      auto row_block = [&](const u32 (&r)[16], int j) {
        u64 P[8];
#pragma unroll
        for (int i = 0; i < 8; i++) P[i] = q_pack64(r[2 * i], r[2 * i + 1]);
        const u32 sb = block_scale_byte(absmax16(P), ts_r);
        const u32 b = (u32)(tok * nblk + blk0 + j);
        orow[j] = quant_block16<ROUNDING>(P, sb, ts_r, seed_r, b, b * 16u);
        sb_row |= sb << (8 * j);
      };
      auto col_pair = [&](const u32 (&r)[32], int pp) {
        u64 P[16];
#pragma unroll
        for (int i = 0; i < 16; i++) P[i] = q_pack64(r[2 * i], r[2 * i + 1]);
        if (!TCRHT) {
#pragma unroll
          for (int h = 1; h < 16; h <<= 1)
#pragma unroll
            for (int i = 0; i < 16; i++)
              if (!(i & h)) { const u64 a = P[i], b = P[i + h]; P[i] = f2_add(a, b); P[i + h] = f2_sub(a, b); }
        }
        const u32 b0 = (u32)(col * nmb + mb0 + 2 * pp), b1 = b0 + 1u;
        u32 sb0, sb1;
        quant_block16x2<ROUNDING>(P, ts_c, seed_c, b0, b1, block_key<ROUNDING>(seed_c, b0), block_key<ROUNDING>(seed_c, b1),
                                  ocol[2 * pp], ocol[2 * pp + 1], sb0, sb1);
        sb_col |= (sb0 | (sb1 << 8)) << (16 * pp);
      };
      auto store_rows = [&]() {
        unsigned char* dst = p.codes_r + (long long)mt * row_code_stride + tok0 * (p.C >> 1) + ct * (kQCol / 2) + half * 32;
        *reinterpret_cast<uint4*>(dst) = make_uint4(orow[0].x, orow[0].y, orow[1].x, orow[1].y);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(orow[2].x, orow[2].y, orow[3].x, orow[3].y);
        // the four scale bytes are neighbours in both layouts
        const long long so = p.linear ? (long long)mt * kQTok * nblk + ct * (kQCol / 16) + row_sc0
                                      : ((long long)mt * (nblk >> 2) + ct * 2) * 512 + row_sc0;
        *reinterpret_cast<u32*>(p.scales_r + so) = sb_row;
      };
      auto store_cols = [&]() {
        unsigned char* dst = p.codes_c + (long long)ct * col_code_stride + (col0 * nmb + mb0) * 8;
        *reinterpret_cast<uint4*>(dst) = make_uint4(ocol[0].x, ocol[0].y, ocol[1].x, ocol[1].y);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(ocol[2].x, ocol[2].y, ocol[3].x, ocol[3].y);
        const long long so = p.linear ? (long long)ct * kQCol * nmb + mt * (kQTok / 16) + col_sc0
                                      : ((long long)ct * (nmb >> 2) + mt * 2) * 512 + col_sc0;
        *reinterpret_cast<u32*>(p.scales_c + so) = sb_col;
      };

      if (ROWS) {
        const u32 t = t_lane + 128u * buf0;
        u32 r1[16], r2[16], r3[16];
        q_wait_ld16(first16);
        q_ld16(t + 16, r1); row_block(first16, 0); q_wait_ld16(r1);
        q_ld16(t + 32, r2); row_block(r1, 1);      q_wait_ld16(r2);
        q_ld16(t + 48, r3); row_block(r2, 2);      q_wait_ld16(r3);
        release(buf0);
        if (BOTH) {
          // the transposed half of the same tile: start its first load before the last row block is quantized
          if (!wait_full(1u, par)) break;
          q_ld32(t_lane + 128u, first32);
        } else if (more) {
          if (!wait_full(nbuf, npar)) break;
          q_ld16(t_lane + 128u * nbuf, first16);
        }
        row_block(r3, 3);
        store_rows();
      }
      if (COLS) {
        const u32 cbuf = BOTH ? 1u : buf0;
        const u32 t = t_lane + 128u * cbuf;
        u32 c1[32];
        q_wait_ld32(first32);
        q_ld32(t + 32, c1);
        col_pair(first32, 0);
        q_wait_ld32(c1);
        release(cbuf);
        if (more) {
          // first chunk of the next tile, requested before this tile's last chunk is quantized
          if (!wait_full(nbuf, npar)) break;
          if (ROWS) q_ld16(t_lane + 128u * nbuf, first16); else q_ld32(t_lane + 128u * nbuf, first32);
        }
        col_pair(c1, 1);
        store_cols();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) q_settle_copies();
  q_fence_before();
  __syncthreads();
  if (warp == 0) {
    q_fence_after();
    q_tmem_dealloc(tmem_base, kQTmemCols);
  }
}

static bool make_tc_map(CUtensorMap* map, const void* x, long long M, long long C, long long ldx) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)(ldx * 2)};
  const cuuint32_t box[2] = {64u, (cuuint32_t)kQTok};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int ROUNDING, bool ROWS, bool COLS, bool TCRHT = false>
static int launch_tc(const CUtensorMap& map, const TcParams& p, int grid, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(quant_tc_kernel<ROUNDING, ROWS, COLS, TCRHT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kQSmem) != cudaSuccess)
      return NVFP4_ERR_CUDA;
    configured[dev] = true;
  }
  if (nvfp4_launch_kernel(quant_tc_kernel<ROUNDING, ROWS, COLS, TCRHT>, dim3((unsigned)grid), dim3(kQThreads), kQSmem, st, map, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVFP4_ERR_CUDA;
  }
  return NVFP4_OK;
}

template <int ROUNDING>
static int launch_tc_mode(const CUtensorMap& map, const TcParams& p, int grid, cudaStream_t st) {
  if (p.tc_rht && p.codes_c) {
    if (p.codes_r) return launch_tc<ROUNDING, true, true, true>(map, p, grid, st);
    return launch_tc<ROUNDING, false, true, true>(map, p, grid, st);
  }
  if (p.codes_r && p.codes_c) return launch_tc<ROUNDING, true, true>(map, p, grid, st);
  if (p.codes_c) return launch_tc<ROUNDING, false, true>(map, p, grid, st);
  return launch_tc<ROUNDING, true, false>(map, p, grid, st);
}

}  // namespace nvfp4

using namespace nvfp4;

int nvfp4_sm_budget_value();   // gemm.cu: nvfp4_gemm_set_sm_budget

// Whether the tensor-core-fed kernel takes this call (shape and alignment); otherwise the scalar tile kernel runs.
bool nvfp4_quant_tc_accepts(const void* x, long long ldx, int M, int C, const void* codes_r, const void* scales_r,
                            const void* codes_c, const void* scales_c) {
  if (M <= 0 || C <= 0 || (M % kQTok) || (C % kQCol) || ldx < C) return false;
  return !((reinterpret_cast<uintptr_t>(x) & 15u) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes_r) & 15u) ||
           (reinterpret_cast<uintptr_t>(codes_c) & 15u) || (reinterpret_cast<uintptr_t>(scales_r) & 3u) ||
           (reinterpret_cast<uintptr_t>(scales_c) & 3u));
}

static int g_tc_rht = 0;
// 1: the Hadamard transform of the transposed operand runs inside the MMA instead of FP32 butterflies
void nvfp4_quant_tc_set_rht(int on) { g_tc_rht = on ? 1 : 0; }

// Arguments as nvfp4_quant_tile, already validated by it.
int nvfp4_quant_tc_launch(const void* x, long long ldx, int M, int C, void* codes_r, void* scales_r, void* codes_c,
                          void* scales_c, int scale_layout, const float* amax, float* gs_r_out, float* gs_c_out,
                          unsigned signs, int rounding, unsigned seed_r, unsigned seed_c,
                          const unsigned* seed_r_dev, const unsigned* seed_c_dev, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap map;
  if (!make_tc_map(&map, x, M, C, ldx)) return NVFP4_ERR_CUDA;
  TcParams p = {};
  p.codes_r = static_cast<unsigned char*>(codes_r); p.scales_r = static_cast<unsigned char*>(scales_r);
  p.codes_c = static_cast<unsigned char*>(codes_c); p.scales_c = static_cast<unsigned char*>(scales_c);
  p.amax = amax; p.gs_r_out = gs_r_out; p.gs_c_out = gs_c_out;
  p.M = M; p.C = C; p.linear = scale_layout == NVFP4_SCALES_LINEAR;
  p.signs = signs & 0xFFFFu;
  p.seed_r = seed_r; p.seed_c = seed_c; p.seed_r_dev = seed_r_dev; p.seed_c_dev = seed_c_dev;
  p.tc_rht = g_tc_rht;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
  }
  const long long ntiles = (long long)(M / kQTok) * (C / kQCol);
  { const int b = nvfp4_sm_budget_value(); if (b > 0 && b < sms) sms = b; }   // SMs left to a collective running beside this kernel
  int grid = 2 * sms;
  if (ntiles < grid) grid = (int)ntiles;
  switch (rounding) {
    case NVFP4_ROUND_NEAREST: return launch_tc_mode<NVFP4_ROUND_NEAREST>(map, p, grid, st);
    case NVFP4_ROUND_SR_DITHER: return launch_tc_mode<NVFP4_ROUND_SR_DITHER>(map, p, grid, st);
    case NVFP4_ROUND_SR_DITHER_K: return launch_tc_mode<NVFP4_ROUND_SR_DITHER_K>(map, p, grid, st);
    default: return launch_tc_mode<NVFP4_ROUND_SR_HW>(map, p, grid, st);
  }
}

// Status word of the tensor-core-fed kernel on the current device (merged into nvfp4_quant_tile_status).
int nvfp4_quant_tc_status(int* out, int reset) {
  if (cudaMemcpyFromSymbol(out, g_quant_tc_status, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (reset) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_quant_tc_status, &zero, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  }
  return NVFP4_OK;
}
