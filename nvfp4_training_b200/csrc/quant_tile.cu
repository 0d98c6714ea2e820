// One-read NVFP4 quantizer for sm_100a: the row operand (1x16 blocks along the columns) and the
// transposed RHT16 operand (16-token blocks per column) of a bf16 [M, C] tensor from a single
// pass over HBM.  Persistent CTAs; warp 0 streams 128-token x 64-column tiles (16 KB, 128-byte
// swizzle) into a shared-memory ring with TMA, eight consumer warps quantize each tile twice from
// shared memory.  Loads in flight no longer depend on the consumers' registers or occupancy, which
// is what bounded the register-tiled column kernel.
//
// Every mbarrier wait is bounded: on expiry the CTA raises an abort flag, stores a role code in the
// library's quantizer status word, lets copies in flight land and returns.
#include "tma.cuh"

namespace nvfp4 {

constexpr int kTileTok = 128;                 // tokens per tile
constexpr int kTileCol = 64;                  // columns per tile (128 bytes of bf16: one swizzle row)
constexpr int kTileBytes = kTileTok * kTileCol * 2;
constexpr int kTileStages = 5;
constexpr int kTileConsumerWarps = 8;
constexpr int kTileThreads = 32 * (1 + kTileConsumerWarps);
constexpr int kTileSmem = kTileStages * kTileBytes + 1024 /*alignment slack*/;

__device__ int g_quant_status;   // 0, or the role code of the first wait that expired

// after an expired wait: give copies that are still in flight time to land before the CTA's
// shared memory is released
__device__ __forceinline__ void settle_copies() {
  const u64 t0 = globaltimer_ns();
  while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
}

struct TileParams {
  uint2* codes_r; unsigned char* scales_r;            // row operand [M, C/2], scales [M, C/16]
  unsigned char* codes_c; unsigned char* scales_c;    // transposed operand [C, M/2], scales [C, M/16]
  const float* amax;
  float* gs_r_out; float* gs_c_out;
  int M, C, linear;
  u32 signs;
  u32 seed_r, seed_c;
  const u32* seed_r_dev; const u32* seed_c_dev;
  // operand-emitter mode only (llm-1b/emit.cu `col_emit`): `amax` is the delayed RHT-domain amax
  unsigned* amax_cur;      // observed RHT-domain amax of this tensor, float bits, atomicMax
  const u32* rng;          // device words: rng[0] = SR seed, rng[1] = Hadamard sign bits
  u32 salt;
};

// barrier over the 256 consumer threads (named barrier 1) with an AND of `ok`
__device__ __forceinline__ bool consumers_all(bool ok) {
  u32 r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
               : "=r"(r) : "r"((u32)ok) : "memory");
  return r != 0u;
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Walks the tiles of one CTA in (token tile, column tile) coordinates without a division per tile.
struct TileWalk {
  int mt, ct, dq, dr, nct, nmt;
  __device__ __forceinline__ TileWalk(int M, int C) {
    nct = C / kTileCol; nmt = M / kTileTok;
    mt = (int)blockIdx.x / nct; ct = (int)blockIdx.x - mt * nct;
    dq = (int)gridDim.x / nct; dr = (int)gridDim.x - dq * nct;
  }
  __device__ __forceinline__ bool valid() const { return mt < nmt; }
  __device__ __forceinline__ void next() { mt += dq; ct += dr; if (ct >= nct) { ct -= nct; mt++; } }
};

// Write the staged transposed-operand outputs of tile (mt, ct): every consumer thread moves 16
// bytes of codes (a quarter of one column's 64-byte run, `code_off` = its offset inside the tile's
// output), the first 64 threads 8 scale bytes each.
__device__ __forceinline__ void drain_cols(const TileParams& p, const u32* src, const unsigned char* ss, int mt, int ct,
                                           int ctid, long long code_off) {
  const int nmb = p.M >> 4;
  const uint4 v = make_uint4(src[0], src[1], src[2], src[3]);
  const long long c0 = (long long)ct * kTileCol;
  *reinterpret_cast<uint4*>(p.codes_c + (c0 * nmb + mt * (kTileTok / 16)) * 8 + code_off) = v;
  if (ctid < 64) {
    const uint2 sv = *reinterpret_cast<const uint2*>(ss + ctid * 8);
    long long off;
    if (p.linear) {
      off = (c0 + ctid) * nmb + mt * (kTileTok / 16);
    } else {
      // 512-byte chunk (128 columns x 4 token blocks); this tile owns bytes [hi0*4, hi0*4+8) of every 16-byte slot
      const long long chunk = (c0 >> 7) * (nmb >> 2) + mt * 2 + (ctid >> 5);
      off = chunk * 512 + (ctid & 31) * 16 + ((c0 >> 5) & 3) * 4;
    }
    *reinterpret_cast<uint2*>(p.scales_c + off) = sv;
  }
}

template <int ROUNDING, bool ROWS, bool COLS>
__global__ void __launch_bounds__(kTileThreads, 2) quant_tile_kernel(const __grid_constant__ CUtensorMap map, const TileParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) float lut_r[kLutFloats];
  __shared__ __align__(8) float lut_c[kLutFloats];
  __shared__ __align__(8) u64 bars[2 * kTileStages];
  // transposed-operand outputs of a tile, staged so that they leave in 16-byte pieces of whole
  // 64-byte column runs: codes [parity of the column][column / 2][17 words] (+1 word skew for odd
  // columns: conflict-free both ways), scale bytes in the order they have in global memory
  __shared__ u32 stage_codes[2][2 * 32 * 17 + 1];
  __shared__ __align__(8) unsigned char stage_scales[2][512];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const u32 tiles0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const u32 full0 = smem_u32(bars), empty0 = full0 + 8 * kTileStages;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < kTileStages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kTileConsumerWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const float amax = __ldg(p.amax);
  const bool first = blockIdx.x == 0 && threadIdx.x == 0;
  TensorScale ts_r, ts_c;
  if (ROWS) ts_r = make_tensor_scale<ROUNDING>(amax, 1.f, lut_r, first ? p.gs_r_out : nullptr);
  // the x0.25 that follows the butterflies is folded into the tensor scale (a power of two); the
  // emitter's delayed amax is already an RHT-domain value (no factor 4)
  constexpr bool EMIT = ROUNDING == NVFP4_EMIT_NEAREST || ROUNDING == NVFP4_EMIT_SR || ROUNDING == NVFP4_EMIT_SR_HW;
  if (COLS) ts_c = make_tensor_scale<ROUNDING>(amax, EMIT ? 1.f : 4.f, lut_c, first ? p.gs_c_out : nullptr, 0.25f);
  __syncthreads();

  if (warp == 0) {
    // ---- producer
    u32 stage = 0, phase = 0;
    for (TileWalk tw(p.M, p.C); tw.valid(); tw.next()) {
      if (!__all_sync(0xffffffffu, mbar_wait_parked(empty0 + 8 * stage, phase ^ 1u, abort_flag))) {
        if (lane == 0) atomicCAS(&g_quant_status, 0, 1);
        break;
      }
      if (elect_one()) {
        mbar_arrive_expect_tx(full0 + 8 * stage, kTileBytes);
        tma_load_2d(tiles0 + stage * kTileBytes, &map, tw.ct * kTileCol, tw.mt * kTileTok, full0 + 8 * stage);
      }
      __syncwarp();
      if (++stage == kTileStages) { stage = 0; phase ^= 1u; }
    }
    if (*abort_flag) settle_copies();
    return;
  }

  // ---- consumers
  const int cw = warp - 1;                       // 0..7
  const int ctid = threadIdx.x - 32;             // 0..255
  u32 seed_r = p.seed_r, seed_c = p.seed_c;
  if (ROUNDING != NVFP4_ROUND_NEAREST && !EMIT) {
    if (p.seed_r_dev) seed_r = __ldg(p.seed_r_dev);
    if (p.seed_c_dev) seed_c = __ldg(p.seed_c_dev);
  }
  u32 signs = p.signs;
  float seen = 0.f;                              // emitter: largest transformed magnitude this thread met
  if (EMIT) {
    seed_c = (ROUNDING != NVFP4_EMIT_NEAREST ? __ldg(p.rng) : 0u) ^ p.salt;
    if (p.rng) signs = __ldg(p.rng + 1) & 0xFFFFu;
  }
  const int nblk = p.C >> 4;                     // 16-column blocks per row
  const int nmb = p.M >> 4;                      // 16-token blocks per column
  // per-thread constants of the transposed path: swizzled shared-memory offsets of the thread's word
  // column for the 8 values of (token & 7), its slots in the staging buffers and in a tile's output
  u32 xoff[8];
#pragma unroll
  for (int k = 0; k < 8; k++) xoff[k] = (u32)(cw * 2048 + ((((lane >> 2) ^ k) << 4) | ((lane & 3) << 2)));
  const int thr_cblk = 2 * lane * nmb + cw;                        // transposed block index inside the tile's range
  const int sc_off = lane * 17 + cw * 2;                           // staging slot of column 2*lane (codes)
  const int ss_off = p.linear ? 2 * lane * 8 + cw
                              : (cw >> 2) * 256 + ((2 * lane) & 31) * 8 + ((2 * lane) >> 5) * 4 + (cw & 3);
  // row path: unit j = (token tok0 + 64*j, 16-column block rblk); all offsets are tile base + constant
  const int tok0 = ctid >> 2, rblk = ctid & 3;
  const u32 r_off0 = (u32)(tok0 * 128 + (((2 * rblk) ^ (tok0 & 7)) << 4));
  const u32 r_off1 = (u32)(tok0 * 128 + ((((2 * rblk) ^ (tok0 & 7)) ^ 1) << 4));
  const int thr_rblk = tok0 * nblk + rblk;
  const int thr_rsc = p.linear ? thr_rblk : (tok0 & 31) * 16 + ((tok0 >> 5) & 3) * 4 + rblk;
  const int dcl = ctid >> 2, dq4 = ctid & 3;                       // drain: column of the tile, quarter of its run
  const int drain_src = (dcl & 1) * (32 * 17 + 1) + (dcl >> 1) * 17 + dq4 * 4;
  const long long drain_dst = (long long)dcl * nmb * 8 + dq4 * 16;
  u32 stage = 0, phase = 0;
  int prev_mt = -1, prev_ct = 0, buf = 0;        // tile whose transposed outputs wait in stage_*[buf ^ 1]
  for (TileWalk tw(p.M, p.C); tw.valid(); tw.next()) {
    const int mt = tw.mt, ct = tw.ct;
    // one consumer-wide barrier per tile: it makes the abort decision uniform and orders the
    // staging buffers (everyone has staged the previous tile, everyone has drained the one before it)
    if (!consumers_all(mbar_wait_parked(full0 + 8 * stage, phase, abort_flag))) {
      if (threadIdx.x == 32) atomicCAS(&g_quant_status, 0, 2);
      prev_mt = -1;
      break;
    }
    if (COLS && prev_mt >= 0)
      drain_cols(p, stage_codes[buf ^ 1] + drain_src, stage_scales[buf ^ 1], prev_mt, prev_ct, ctid, drain_dst);
    const u32 tile = tiles0 + stage * kTileBytes;

    if (COLS) {
      // thread = (word column `lane` = columns 2*lane, 2*lane+1; token block `cw`).  Row r of the
      // tile keeps its 16-byte chunk j at position j ^ (r & 7); r & 7 == i & 7 here.
      u64 P[16];
#pragma unroll
      for (int i = 0; i < 16; i++) {
        u32 w;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(tile + xoff[i & 7] + (u32)(i * 128)));
        const u32 f = ((signs >> i) & 1u) << 31;             // token i is negated when bit i of signs is set
        P[i] = f2_pack(__uint_as_float((w << 16) + f), __uint_as_float((w & 0xFFFF0000u) ^ f));
      }
#pragma unroll
      for (int h = 1; h < 16; h <<= 1)
#pragma unroll
        for (int i = 0; i < 16; i++)
          if (!(i & h)) { const u64 a = P[i], b = P[i + h]; P[i] = f2_add(a, b); P[i + h] = f2_sub(a, b); }
      const u32 b0 = (u32)((long long)ct * kTileCol * nmb + mt * (kTileTok / 16)) + (u32)thr_cblk, b1 = b0 + (u32)nmb;
      uint2 o0, o1; u32 sb0, sb1;
      u32 key0, key1;
      float bmax = 0.f;
      if (ROUNDING == NVFP4_EMIT_SR_HW) {
        key0 = sr_hw_block_key(seed_c, b0);
        key1 = sr_hw_block_key(seed_c, b1);
      } else if (EMIT) {
        // the reference's thread of (column, 64-token group) walks its four blocks in order: jump to block mb & 3
        const u32 c = (u32)(ct * kTileCol + 2 * lane), mb = (u32)(mt * (kTileTok / 16) + cw);
        key0 = hash32(seed_c ^ hash32(c * 4099u + (mb >> 2)));
        key1 = hash32(seed_c ^ hash32((c + 1u) * 4099u + (mb >> 2)));
        constexpr u32 jm[4] = {1u, lcg_jump_mul(8), lcg_jump_mul(16), lcg_jump_mul(24)};
        constexpr u32 ja[4] = {0u, lcg_jump_add(8), lcg_jump_add(16), lcg_jump_add(24)};
        key0 = key0 * jm[mb & 3u] + ja[mb & 3u];
        key1 = key1 * jm[mb & 3u] + ja[mb & 3u];
      } else {
        key0 = block_key<ROUNDING>(seed_c, b0);
        key1 = block_key<ROUNDING>(seed_c, b1);
      }
      quant_block16x2<ROUNDING>(P, ts_c, seed_c, b0, b1, key0, key1, o0, o1, sb0, sb1, EMIT ? &bmax : nullptr);
      if (EMIT) seen = fmaxf(seen, bmax);
      u32* sc = stage_codes[buf] + sc_off;
      sc[0] = o0.x; sc[1] = o0.y;                                   // column 2*lane
      sc[32 * 17 + 1] = o1.x; sc[32 * 17 + 2] = o1.y;               // column 2*lane+1
      unsigned char* ss = stage_scales[buf] + ss_off;
      ss[0] = (unsigned char)sb0; ss[8] = (unsigned char)sb1;
      prev_mt = mt; prev_ct = ct; buf ^= 1;
    }

    if (ROWS) {
      // thread = two (token, 16-column block) units; four neighbouring lanes cover one token's 128 bytes
      const long long tile_b = (long long)mt * kTileTok * nblk + ct * (kTileCol / 16);
      const long long tile_s = p.linear ? tile_b : ((long long)mt * (nblk >> 2) + ct) * 512;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        Block32 cur;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(cur.w[0]), "=r"(cur.w[1]), "=r"(cur.w[2]), "=r"(cur.w[3]) : "r"(tile + r_off0 + (u32)(j * 64 * 128)));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(cur.w[4]), "=r"(cur.w[5]), "=r"(cur.w[6]), "=r"(cur.w[7]) : "r"(tile + r_off1 + (u32)(j * 64 * 128)));
        u64 P[8];
#pragma unroll
        for (int i = 0; i < 8; i++) P[i] = f2_from_bf16x2(cur.w[i]);
        const u32 sb = block_scale_byte(absmax16(P), ts_r);
        const long long b = tile_b + thr_rblk + (long long)j * 64 * nblk;
        p.codes_r[b] = quant_block16<ROUNDING>(P, sb, ts_r, seed_r, (u32)b, (u32)b * 16u);
        // 64 tokens further: same 512-byte scale chunk, 8 bytes on (swizzled) / 64 rows on (linear)
        p.scales_r[tile_s + thr_rsc + (p.linear ? (long long)j * 64 * nblk : (long long)j * 8)] = (unsigned char)sb;
      }
    }

    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * stage);
    if (++stage == kTileStages) { stage = 0; phase ^= 1u; }
  }
  if (EMIT && p.amax_cur) {
#pragma unroll
    for (int o = 16; o; o >>= 1) seen = fmaxf(seen, __shfl_xor_sync(0xffffffffu, seen, o));
    if (lane == 0) atomicMax(p.amax_cur, __float_as_uint(__fmul_rn(seen, 0.25f)));
  }
  if (COLS && prev_mt >= 0) {
    consumers_sync();
    drain_cols(p, stage_codes[buf ^ 1] + drain_src, stage_scales[buf ^ 1], prev_mt, prev_ct, ctid, drain_dst);
  }
  if (*abort_flag) settle_copies();
}

static bool make_tile_map(CUtensorMap* map, const void* x, long long M, long long C, long long ldx) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)(ldx * 2)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileCol, (cuuint32_t)kTileTok};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int ROUNDING, bool ROWS, bool COLS>
static int launch_tile(const CUtensorMap& map, const TileParams& p, int grid, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(quant_tile_kernel<ROUNDING, ROWS, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmem) != cudaSuccess)
      return NVFP4_ERR_CUDA;
    configured[dev] = true;
  }
  quant_tile_kernel<ROUNDING, ROWS, COLS><<<grid, kTileThreads, kTileSmem, st>>>(map, p);
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}

template <int ROUNDING>
static int launch_tile_mode(const CUtensorMap& map, const TileParams& p, int grid, cudaStream_t st) {
  if (p.codes_r && p.codes_c) return launch_tile<ROUNDING, true, true>(map, p, grid, st);
  if (p.codes_c) return launch_tile<ROUNDING, false, true>(map, p, grid, st);
  return launch_tile<ROUNDING, true, false>(map, p, grid, st);
}

}  // namespace nvfp4

using namespace nvfp4;

int nvfp4_sm_budget_value();   // gemm.cu: nvfp4_gemm_set_sm_budget

// the tensor-core-fed kernel (quant_mma.cu)
bool nvfp4_quant_tc_accepts(const void* x, long long ldx, int M, int C, const void* codes_r, const void* scales_r,
                            const void* codes_c, const void* scales_c);
int nvfp4_quant_tc_launch(const void* x, long long ldx, int M, int C, void* codes_r, void* scales_r, void* codes_c,
                          void* scales_c, int scale_layout, const float* amax, float* gs_r_out, float* gs_c_out,
                          unsigned signs, int rounding, unsigned seed_r, unsigned seed_c,
                          const unsigned* seed_r_dev, const unsigned* seed_c_dev, void* stream);
int nvfp4_quant_tc_status(int* out, int reset);
void nvfp4_quant_tc_set_rht(int on);
int nvfp4_emit_rows_ring_status(int* out, int reset);

// 0 = tensor-core-fed kernel where it applies, 1 = always the scalar tile kernel, 2 = tensor-core-fed kernel with the
// Hadamard transform inside the MMA
static int g_tile_path = 0;

extern "C" int nvfp4_quant_tile_set_path(int path) {
  if (path < 0 || path > 2) return NVFP4_ERR_ENUM;
  g_tile_path = path;
  nvfp4_quant_tc_set_rht(path == 2);
  return NVFP4_OK;
}

extern "C" int nvfp4_quant_tile(const void* x, long long ldx, int M, int C, void* codes_r, void* scales_r, void* codes_c,
                                void* scales_c, int scale_layout, const float* amax, float* gs_r_out, float* gs_c_out,
                                unsigned signs, int rounding, unsigned seed_r, unsigned seed_c,
                                const unsigned* seed_r_dev, const unsigned* seed_c_dev, void* stream) {
  if (!x || !amax || (!codes_r && !codes_c) || (codes_r && !scales_r) || (codes_c && !scales_c)) return NVFP4_ERR_NULL;
  if (scale_layout != NVFP4_SCALES_SWIZZLED && scale_layout != NVFP4_SCALES_LINEAR) return NVFP4_ERR_ENUM;
  if (rounding < NVFP4_ROUND_NEAREST || rounding > NVFP4_ROUND_SR_HW) return NVFP4_ERR_ENUM;
  if (M < 0 || C < 0 || (M % kTileTok) || (C % kTileCol) || ldx < C) return NVFP4_ERR_SHAPE;
  if (codes_c && scale_layout == NVFP4_SCALES_SWIZZLED && (C & 127)) return NVFP4_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes_r) & 7u) ||
      (reinterpret_cast<uintptr_t>(codes_c) & 15u) || (reinterpret_cast<uintptr_t>(scales_c) & 7u))
    return NVFP4_ERR_ALIGN;
  if (M == 0 || C == 0) return NVFP4_OK;
  if (g_tile_path != 1 && nvfp4_quant_tc_accepts(x, ldx, M, C, codes_r, scales_r, codes_c, scales_c))
    return nvfp4_quant_tc_launch(x, ldx, M, C, codes_r, scales_r, codes_c, scales_c, scale_layout, amax, gs_r_out, gs_c_out,
                                 signs, rounding, seed_r, seed_c, seed_r_dev, seed_c_dev, stream);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap map;
  if (!make_tile_map(&map, x, M, C, ldx)) return NVFP4_ERR_CUDA;
  TileParams p = {};
  p.codes_r = static_cast<uint2*>(codes_r); p.scales_r = static_cast<unsigned char*>(scales_r);
  p.codes_c = static_cast<unsigned char*>(codes_c); p.scales_c = static_cast<unsigned char*>(scales_c);
  p.amax = amax; p.gs_r_out = gs_r_out; p.gs_c_out = gs_c_out;
  p.M = M; p.C = C; p.linear = scale_layout == NVFP4_SCALES_LINEAR;
  p.signs = signs & 0xFFFFu;
  p.seed_r = seed_r; p.seed_c = seed_c; p.seed_r_dev = seed_r_dev; p.seed_c_dev = seed_c_dev;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
  }
  const long long ntiles = (long long)(M / kTileTok) * (C / kTileCol);
  { const int b = nvfp4_sm_budget_value(); if (b > 0 && b < sms) sms = b; }   // SMs left to a collective running beside this kernel
  int grid = 2 * sms;
  if (ntiles < grid) grid = (int)ntiles;
  switch (rounding) {
    case NVFP4_ROUND_NEAREST: return launch_tile_mode<NVFP4_ROUND_NEAREST>(map, p, grid, st);
    case NVFP4_ROUND_SR_DITHER: return launch_tile_mode<NVFP4_ROUND_SR_DITHER>(map, p, grid, st);
    case NVFP4_ROUND_SR_DITHER_K: return launch_tile_mode<NVFP4_ROUND_SR_DITHER_K>(map, p, grid, st);
    default: return launch_tile_mode<NVFP4_ROUND_SR_HW>(map, p, grid, st);
  }
}

extern "C" int nvfp4_emit_cols(const void* x, long long ldx, int M, int C, void* codes, void* scales,
                               const float* amax_use, unsigned* amax_cur, int sr, const unsigned* rng, unsigned salt,
                               void* stream) {
  if (!x || !codes || !scales || !amax_use || !rng) return NVFP4_ERR_NULL;
  if (sr < 0 || sr > 2) return NVFP4_ERR_ENUM;
  if (M < 0 || C < 0 || (M % kTileTok) || (C & 127) || ldx < C) return NVFP4_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes) & 15u) ||
      (reinterpret_cast<uintptr_t>(scales) & 7u))
    return NVFP4_ERR_ALIGN;
  if (M == 0 || C == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap map;
  if (!make_tile_map(&map, x, M, C, ldx)) return NVFP4_ERR_CUDA;
  TileParams p = {};
  p.codes_c = static_cast<unsigned char*>(codes); p.scales_c = static_cast<unsigned char*>(scales);
  p.amax = amax_use; p.amax_cur = amax_cur; p.rng = rng; p.salt = salt;
  p.M = M; p.C = C; p.linear = 0;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
  }
  const long long ntiles = (long long)(M / kTileTok) * (C / kTileCol);
  { const int b = nvfp4_sm_budget_value(); if (b > 0 && b < sms) sms = b; }   // SMs left to a collective running beside this kernel
  int grid = 2 * sms;
  if (ntiles < grid) grid = (int)ntiles;
  if (sr == 2) return launch_tile<NVFP4_EMIT_SR_HW, false, true>(map, p, grid, st);
  return sr ? launch_tile<NVFP4_EMIT_SR, false, true>(map, p, grid, st)
            : launch_tile<NVFP4_EMIT_NEAREST, false, true>(map, p, grid, st);
}

extern "C" int nvfp4_quant_tile_status(int* out, int reset) {
  if (!out) return NVFP4_ERR_NULL;
  if (cudaMemcpyFromSymbol(out, g_quant_status, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  if (reset) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_quant_status, &zero, sizeof(int)) != cudaSuccess) return NVFP4_ERR_CUDA;
  }
  int tc = 0;
  const int rc = nvfp4_quant_tc_status(&tc, reset);
  if (rc != NVFP4_OK) return rc;
  int ring = 0;
  const int rc2 = nvfp4_emit_rows_ring_status(&ring, reset);
  if (rc2 != NVFP4_OK) return rc2;
  if (*out == 0 && ring) *out = 32 + ring;  // TMA-fed row emitter: 33 producer, 34 consumer
  if (*out == 0 && tc) *out = 16 + tc;    // tensor-core-fed kernel: 17 / 19 its loading and MMA-issuing warp (waiting for a tile / a free stage), 18 a consumer
  return NVFP4_OK;
}
