// Block-scaled FP4 GEMM for sm_100a:  C[M,N] (+)= alpha * A[M,K] * B[N,K]^T
//   A, B   packed E2M1 (2 per byte), K-major; one UE4M3 scale per 16 values in the 128x4-tile
//          swizzled layout (512-byte tiles, consecutive K tiles of one 128-row block contiguous).
//
// Persistent, warp-specialised kernel, one CTA per SM, 320 threads:
//   warp 0      TMA producer: per K tile (256 elements) one 128-byte-swizzled box load each for A and
//               B plus plain bulk copies of the scale tiles (2 KB per 128 rows), all completing on
//               the stage's `full` mbarrier
//   warp 1      MMA issuer: copies the stage's scale tiles shared memory -> tensor memory
//               (tcgen05.cp 32x128b.warpx4), issues four tcgen05.mma kind::mxf4nvf4 block16 (K = 64
//               each) into the FP32 accumulator in tensor memory, releases the stage with
//               tcgen05.commit; owns tensor-memory allocation
//   warps 2..9  epilogue: each warp drains half the columns of its 32-lane quadrant with tcgen05.ld
//               into registers, hands the accumulator back at once, then applies alpha, casts and
//               stores (or FP32 vector atomic adds for split-K / accumulate)
// With BN = 128 two accumulators alternate; with BN = 256 the single accumulator is free again as
// soon as it has been read, so the next tile's MMAs overlap the conversion and the stores.
// The issuing threads keep their per-K-tile instruction count minimal (descriptor low words are
// advanced by adds, high words are constants): a single thread feeds the whole tensor core.
// Every mbarrier wait is bounded: on expiry the CTA raises an abort flag, reports a code through
// `status`, lets copies in flight land, frees its tensor memory and returns.
#include <atomic>

#include "tma.cuh"

// Waits of warps that have nothing else to do (producer waiting for a free stage, epilogue waiting
// for an accumulator) carry a suspend-time hint: the warp sleeps in hardware instead of polling,
// which measured 1-2 % faster on the large shapes (fewer issue slots and less power spent spinning).
#define NVFP4_IDLE_WAIT mbar_wait_parked

// 16-byte store of finished bf16 output with the streaming hint: the output is not read again by this
// kernel and should not push operand tiles out of L2 (measured +3 % on 16384x11264x2048, neutral elsewhere)
#define NVFP4_STORE_C16(ptr, v) __stcs(reinterpret_cast<uint4*>(ptr), v)

namespace nvfp4 {

constexpr int kBM = 128;            // rows of A per tile (UMMA M)
constexpr int kBKBytes = 128;       // bytes of K per stage row = 256 FP4 values = one 128B swizzle row
constexpr int kBK = 256;            // FP4 values of K per stage
constexpr int kEpiWarps = 8;         // two warps per 32-lane quadrant of tensor memory
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kPairThreads = kThreads + 32;   // CTA-pair kernel: one more warp, which draws the work items

template <int BN>
struct Cfg {
  static constexpr int kStages = BN == 128 ? 6 : 4;
  static constexpr int kAccStages = BN == 128 ? 2 : 1;
  static constexpr int kABytes = kBM * kBKBytes;           // 16 KB
  static constexpr int kBBytes = BN * kBKBytes;            // 16 / 32 KB
  static constexpr int kSFABytes = 2048;                   // 4 K-chunks x 512 B
  static constexpr int kSFBBytes = 2048 * (BN / 128);
  static constexpr int kStageBytes = kABytes + kBBytes + kSFABytes + kSFBBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // tensor-memory columns: accumulators first, then scale factors of the stage being multiplied
  static constexpr int kSfaCol = kAccStages * BN;
  static constexpr int kSfbCol = kSfaCol + 16;
  static constexpr int kSfBufCols = 16 + 16 * (BN / 128);   // columns of one scale buffer; two alternate per K tile
  static constexpr int kTmemCols = 512;
};

struct GemmParams {
  const unsigned char* sfa;
  const unsigned char* sfb;
  void* c;
  const float* pa;
  const float* pb;
  int* status;
  long long ldc;
  float kscale;       // ka*kb/2688^2 for NVFP4_ALPHA_AMAX
  int M, N, K;
  int alpha_mode;
  int c_fp32;
  int atomic;         // 1: add into C with FP32 atomics
  int splitk;         // number of K slices
  int ktiles_per_split;
};

// ---------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tmem_alloc(u32 smem_dst, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(u32 bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(u32 taddr, u64 sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 sfa_tmem, u32 sfb_tmem,
                                            u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(u32 taddr, u32 (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(u32 taddr, u32 (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05): start address, leading/stride byte offsets in 16-byte
// units, descriptor version 1 at bit 46, swizzle mode in bits 61..63 (0 none, 2 = 128 bytes).
__device__ __forceinline__ u64 smem_desc(u32 saddr, u32 lbo_bytes, u32 sbo_bytes, u32 swizzle) {
  return (u64)((saddr & 0x3FFFFu) >> 4) | ((u64)(lbo_bytes >> 4) << 16) | ((u64)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | ((u64)swizzle << 61);
}

// Instruction descriptor for kind::mxf4nvf4 with UE4M3 scales: A/B format E2M1 (code 1) at bits 7 and
// 10, both operands K-major, N/8 at bit 17, scale format UE4M3 (0) at bit 23, M/16 at bit 24, K = 64.
__host__ __device__ constexpr u32 make_idesc(int n) {
  return (1u << 7) | (1u << 10) | ((u32)(n >> 3) << 17) | ((u32)(kBM >> 4) << 24);
}

// ---------------------------------------------------------------------------------------- kernel
__device__ __forceinline__ u64 pack64(u32 lo, u32 hi) {
  u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// high words of the shared-memory descriptors (constant for the whole kernel):
//   operand tiles: stride offset 1024 B (8 rows x 128 B), version 1, 128-byte swizzle
//   scale tiles:   stride offset 128 B (8 rows x 16 B), version 1, no swizzle
constexpr u32 kDescHiAB = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr u32 kDescHiSF = (128u >> 4) | (1u << 14);

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_nvf4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  using C = Cfg<BN>;
  pdl_trigger();
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* bar_mem = smem + C::kStages * C::kStageBytes;
  u64* full_bar = reinterpret_cast<u64*>(bar_mem);
  u64* empty_bar = full_bar + C::kStages;
  u64* acc_full = empty_bar + C::kStages;
  u64* acc_empty = acc_full + 2;
  u32* tmem_slot = reinterpret_cast<u32*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = p.M / kBM, tiles_n = p.N / BN;
  const int ktiles = (p.K + kBK - 1) / kBK;
  const int num_work = tiles_m * tiles_n * p.splitk;
  const u32 smem_base = smem_u32(smem);
  const u32 full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(smem_u32(acc_full + a), 1); mbar_init(smem_u32(acc_empty + a), kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const u32 tmem_base = *tmem_slot;
  pdl_wait();         // operands, scales and alpha words are earlier kernels' results; C may still be read by them

  // The two issuing warps run their loops with all 32 lanes converged, so that loop state,
  // addresses and descriptors stay warp-uniform (the asynchronous-copy and tensor-core instructions
  // take uniform operands); only the instruction issue itself is predicated on one elected lane.
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    int stage = 0; u32 phase = 0;
    u32 st_addr = smem_base;
    const long long sf_row_bytes = (long long)(p.K >> 6) * 512;   // scale bytes of one 128-row block
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      const int mt = w % tiles_m;
      const int rest = w / tiles_m;
      const int nt = rest % tiles_n;
      const int z = rest / tiles_n;
      const int kt0 = z * p.ktiles_per_split;
      const int kt1 = min(ktiles, kt0 + p.ktiles_per_split);
      const unsigned char* sfa = p.sfa + (long long)mt * sf_row_bytes + (long long)kt0 * 2048;
      const unsigned char* sfb = p.sfb + (long long)(nt * (BN / 128)) * sf_row_bytes + (long long)kt0 * 2048;
      const int ya = mt * kBM, yb = nt * BN;
      int x = kt0 * kBKBytes;
      for (int kt = kt0; kt < kt1; kt++) {
        if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag))) { ok = false; break; }
        const u32 bar = full0 + 8 * stage;
        const int krem = p.K - kt * kBK;
        const u32 sf_bytes = krem >= kBK ? 2048u : (u32)(krem >> 6) * 512u;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, (u32)(C::kABytes + C::kBBytes) + sf_bytes * (1 + BN / 128));
          tma_load_2d(st_addr, &map_a, x, ya, bar);
          tma_load_2d(st_addr + C::kABytes, &map_b, x, yb, bar);
          bulk_load(st_addr + C::kABytes + C::kBBytes, sfa, sf_bytes, bar);
#pragma unroll
          for (int h = 0; h < BN / 128; h++)
            bulk_load(st_addr + C::kABytes + C::kBBytes + C::kSFABytes + h * 2048, sfb + h * sf_row_bytes, sf_bytes, bar);
        }
        x += kBKBytes; sfa += 2048; sfb += 2048;
        st_addr += C::kStageBytes;
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; st_addr = smem_base; }
      }
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 1);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr u32 idesc = make_idesc(BN);
    u32 sfa_t = tmem_base + C::kSfaCol, sfb_t = tmem_base + C::kSfbCol;
    u32 sf_flip = C::kSfBufCols;
    int stage = 0; u32 phase = 0;
    // low descriptor words of the current stage: operand tiles carry leading offset 16 B (bit 16)
    const u32 a_lo0 = (smem_base >> 4) | (1u << 16);
    u32 a_lo = a_lo0;
    int acc = 0; u32 acc_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      const int z = w / (tiles_m * tiles_n);
      const int kt0 = z * p.ktiles_per_split;
      const int kt1 = min(ktiles, kt0 + p.ktiles_per_split);
      // the epilogue must have drained this accumulator
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(acc_empty + acc), acc_phase ^ 1u, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const u32 d_tmem = tmem_base + (u32)(acc * BN);
      u32 accum = 0u;
      for (int kt = kt0; kt < kt1; kt++) {
        if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * stage, phase, abort_flag))) { ok = false; break; }
        const u32 b_lo = a_lo + (C::kABytes >> 4);
        const u32 sfa_lo = (a_lo & 0xFFFFu) + ((C::kABytes + C::kBBytes) >> 4);
        const u32 sfb_lo = sfa_lo + (C::kSFABytes >> 4);
        const int krem = p.K - kt * kBK;
        if (elect_one()) {
          if (krem >= kBK) {
            // scale tiles of the four K chunks: shared memory -> tensor memory
#pragma unroll
            for (int j = 0; j < 4; j++) {
              tc_cp_sf(sfa_t + 4 * j, pack64(sfa_lo + 32 * j, kDescHiSF));
#pragma unroll
              for (int h = 0; h < BN / 128; h++)
                tc_cp_sf(sfb_t + (BN / 32) * j + 4 * h, pack64(sfb_lo + 128 * h + 32 * j, kDescHiSF));
            }
            // four MMAs, each 64 FP4 values = 32 bytes further along K inside the 128-byte swizzle row
            tc_mma_nvf4(d_tmem, pack64(a_lo, kDescHiAB), pack64(b_lo, kDescHiAB), idesc, sfa_t, sfb_t, accum);
#pragma unroll
            for (int j = 1; j < 4; j++)
              tc_mma_nvf4(d_tmem, pack64(a_lo + 2 * j, kDescHiAB), pack64(b_lo + 2 * j, kDescHiAB), idesc, sfa_t + 4 * j,
                          sfb_t + (BN / 32) * j, 1u);
          } else {
            const int kchunks = krem >> 6;
            for (int j = 0; j < kchunks; j++) {
              tc_cp_sf(sfa_t + 4 * j, pack64(sfa_lo + 32 * j, kDescHiSF));
#pragma unroll
              for (int h = 0; h < BN / 128; h++)
                tc_cp_sf(sfb_t + (BN / 32) * j + 4 * h, pack64(sfb_lo + 128 * h + 32 * j, kDescHiSF));
            }
            for (int j = 0; j < kchunks; j++)
              tc_mma_nvf4(d_tmem, pack64(a_lo + 2 * j, kDescHiAB), pack64(b_lo + 2 * j, kDescHiAB), idesc, sfa_t + 4 * j,
                          sfb_t + (BN / 32) * j, (j > 0) ? 1u : accum);
          }
          tc_commit(empty0 + 8 * stage);              // frees the stage once these MMAs have read it
        }
        accum = 1u;
        sfa_t += sf_flip; sfb_t += sf_flip; sf_flip = 0u - sf_flip;   // other scale buffer for the next K tile
        a_lo += C::kStageBytes >> 4;
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; a_lo = a_lo0; }
      }
      if (!ok) break;
      if (elect_one()) tc_commit(smem_u32(acc_full + acc));          // accumulator complete
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 2);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Each warp drains kEpiCols columns of its 32-lane quadrant into registers in one go and hands
    // the accumulator back before converting and storing, so the tensor core restarts early.
    constexpr int kEpiCols = BN / 2;
    const int quad = warp & 3;                         // tensor-memory lanes 32*quad .. +31
    const int half = (warp - 2) >> 2;                  // which half of the tile's columns
    int acc = 0; u32 acc_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      const int mt = w % tiles_m;
      const int nt = (w / tiles_m) % tiles_n;
      // the decision must be warp-uniform: the tensor-memory loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(acc_full + acc), acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after();
      u32 r[kEpiCols];
      const u32 t_row = tmem_base + ((u32)(quad * 32) << 16) + (u32)(acc * BN + half * kEpiCols);
#pragma unroll
      for (int c = 0; c < kEpiCols / 32; c++) tc_ld32(t_row + c * 32, *reinterpret_cast<u32(*)[32]>(&r[c * 32]));
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty + acc));
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1u; }

      const long long row = (long long)mt * kBM + quad * 32 + lane;
      float alpha = 1.f;
      if (p.alpha_mode == NVFP4_ALPHA_GS) alpha = ld_cg_f32(p.pa) * ld_cg_f32(p.pb);
      else if (p.alpha_mode == NVFP4_ALPHA_AMAX) alpha = ld_cg_f32(p.pa) * ld_cg_f32(p.pb) * p.kscale;
      else if (p.alpha_mode == NVFP4_ALPHA_ROW) alpha = ld_cg_f32(p.pa + row) * ld_cg_f32(p.pb);   // this lane's row
      const long long col = (long long)nt * BN + half * kEpiCols;
      if (p.c_fp32) {
        float* dst = static_cast<float*>(p.c) + row * p.ldc + col;
        if (p.atomic) {
#pragma unroll
          for (int i = 0; i < kEpiCols; i += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i),
                         "f"(__uint_as_float(r[i]) * alpha), "f"(__uint_as_float(r[i + 1]) * alpha),
                         "f"(__uint_as_float(r[i + 2]) * alpha), "f"(__uint_as_float(r[i + 3]) * alpha) : "memory");
        } else {
#pragma unroll
          for (int i = 0; i < kEpiCols; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(r[i]) * alpha, __uint_as_float(r[i + 1]) * alpha,
                                                              __uint_as_float(r[i + 2]) * alpha, __uint_as_float(r[i + 3]) * alpha);
        }
      } else {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + row * p.ldc + col;
#pragma unroll
        for (int i = 0; i < kEpiCols; i += 8) {
          uint4 o;
          __nv_bfloat162 h;
          h = __floats2bfloat162_rn(__uint_as_float(r[i]) * alpha, __uint_as_float(r[i + 1]) * alpha); o.x = *reinterpret_cast<u32*>(&h);
          h = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * alpha, __uint_as_float(r[i + 3]) * alpha); o.y = *reinterpret_cast<u32*>(&h);
          h = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * alpha, __uint_as_float(r[i + 5]) * alpha); o.z = *reinterpret_cast<u32*>(&h);
          h = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * alpha, __uint_as_float(r[i + 7]) * alpha); o.w = *reinterpret_cast<u32*>(&h);
          *reinterpret_cast<uint4*>(dst + i) = o;
        }
      }
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 3);
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // let bulk copies still in flight land before shared memory is released
    const u64 t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ======================================================================================== CTA-pair kernel
// Two CTAs of one cluster (an SM pair) share every 256x256 output tile: tcgen05.mma.cta_group::2 with
// M = 256 reads A rows 0..127 and B rows 0..127 from the leader CTA's shared memory and rows 128..255
// from its peer's, and leaves each CTA the accumulator of its own 128 rows in its own tensor memory.
// Each CTA therefore loads only half of B per K tile (38 KB a stage instead of 54 KB), which is what
// the operand pipeline -- bound by bytes in flight against the ~1 us load latency -- needs, and the
// shared memory saved holds a fifth stage plus a staging buffer for coalesced output stores.
//   both CTAs   warp 0 loads its A rows, its half of B, its A scales and all B scales with
//               cp.async.bulk.tensor (cta_group::2 form: the bytes are counted on the LEADER's `full`
//               barrier; no multicast), after waiting on its own `empty` barrier
//   leader      warp 1 copies scales to tensor memory (both CTAs at once), issues the MMAs and commits
//               to the `empty` / `acc_full` barriers of both CTAs (one commit per CTA)
//   both CTAs   warps 2..9 drain their accumulator, arrive on the leader's `acc_empty` barrier, then
//               convert and store through a per-warp 4 KB staging area so that every global store
//               instruction writes whole 128-byte (FP32) or 64-byte (bf16) row segments
template <int BN>
struct PairCfg {
  // BN = 256: one 256x256 tile per CTA pair, two accumulators that overlap in 48 tensor-memory columns
  // BN = 192: 256x192 tiles, two disjoint accumulators (the next tile's MMAs never wait for the
  //           previous tile's epilogue); N need not be a multiple of 192 (loads beyond N read zeros,
  //           stores are clipped)
  // BN = 128: 256x128 tiles, two disjoint accumulators, more stages; most operand bytes per FLOP
  static constexpr int kStages = BN == 256 ? 5 : BN == 192 ? 6 : 7;
  static constexpr int kSfbBlocks = BN == 128 ? 1 : 2;     // 128-row scale blocks of B fetched per K tile
  static constexpr int kABytes = 16384;                    // 128 rows x 128 B
  static constexpr int kBBytes = (BN / 2) * 128;           // this CTA's half of the B tile
  static constexpr int kSFABytes = 2048;
  static constexpr int kSFBBytes = kSfbBlocks * 2048;      // all B scales, in both CTAs
  static constexpr int kStageBytes = kABytes + kBBytes + kSFABytes + kSFBBytes;   // multiple of 1024
  static constexpr int kStageRowBytes = BN == 256 ? 128 : 64;                     // staging row of one lane
  static constexpr int kStagingBytes = kEpiWarps * 32 * kStageRowBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 512;   // + alignment + barriers and tile queue
  static constexpr u32 kTxBytes = 2u * kStageBytes;        // both CTAs' loads of one stage
  // Tensor-memory columns.  BN = 256: accumulators at columns 0 and 208 overlap in columns 208..255,
  // which the epilogue drains first and hands back at once; scales behind them at 464 (A: 16 columns,
  // B: 32).  BN = 192 / 128: accumulators at 0 and BN, scales at 2*BN.
  static constexpr int kAccOff1 = BN == 256 ? 208 : BN;
  static constexpr int kSfaCol = BN == 256 ? 464 : 2 * BN;
  static constexpr int kSfbCol = kSfaCol + 16;
  static constexpr int kTmemCols = 512;
  static constexpr int kEpiCols = BN / 2;                  // columns each epilogue warp drains
};


__device__ __forceinline__ u32 cluster_ctarank() { u32 r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ u32 map_to_cta(u32 saddr, u32 rank) {
  u32 r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a (possibly remote) barrier that hands tensor memory back to the MMA warp.  Relaxed on
// purpose: the hand-off is ordered by tcgen05.fence::before_thread_sync; a releasing arrive would
// also wait for this thread's earlier global stores (the previous tile's output) to become visible.
__device__ __forceinline__ void mbar_arrive_cluster(u32 cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(u32 dst, const CUtensorMap* map, int x, int y, u32 bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma2_load_3d(u32 dst, const CUtensorMap* map, int x, int y, int z, u32 bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem2_alloc(u32 smem_dst, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem2_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_dealloc(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc2_commit(u32 cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc2_cp_sf(u32 taddr, u64 sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc2_mma_nvf4(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 sfa_tmem, u32 sfb_tmem,
                                             u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// instruction descriptor of the pair MMA: M = 256 (16 at bit 24), N = n
__host__ __device__ constexpr u32 make_idesc_pair(int n) {
  return (1u << 7) | (1u << 10) | ((u32)(n >> 3) << 17) | ((u32)(256 >> 4) << 24);
}

constexpr int kMaxOwners = 8;

struct PairParams {
  void* c;
  const float* pa;
  const float* pb;
  int* status;
  long long ldc;
  float kscale;
  int M, N, K;
  int alpha_mode;
  int c_fp32;
  int atomic;
  int splitk;
  int ktiles_per_split;
  unsigned* counter;      // this launch's work counter (zero before the launch, zero again after it)
  int dynamic;            // 1: items after a cluster's first are drawn from the counter; 0: dealt out in advance (item = cluster + k * clusters)
  // row-slab scatter (rows_per_owner > 0): rows [r * rows_per_owner, (r + 1) * rows_per_owner) of C are added into
  // owner_c[r] (the same matrix in rank r's memory: a peer mapping, or p.c for this rank) instead of p.c
  float* owner_c[kMaxOwners];
  int rows_per_owner;
};

// ---- dynamic tile scheduler of the pair kernel
// Work items are not dealt out in advance: a cluster takes the next item from a global counter whenever it is ready
// for one.  A grid that finds some SMs occupied (a collective running beside the GEMM) then needs no tuning: the
// clusters that do run share the items, the ones that start late do their first item and find no more.  A warp of
// its own in the leader CTA draws the numbers, decodes them and publishes the tile coordinates to every role of both
// CTAs through a small queue in shared memory: entry k lives in slot k % kSchedSlots as one 64-bit word (coordinates
// and a tag derived from k), written with a single store (to the peer through shared::cluster) and polled by its
// readers.  The drawing warp stays at most kSchedAhead entries ahead of the MMA warp (which posts the entry it is
// working on), the epilogue is at most two entries (accumulators) behind the MMA warp, the producers are ahead of it:
// nobody reads a slot that is being reused.  Why a warp of its own: a draw is a global atomic with a result, and under
// the operand traffic of the GEMM its round trip is long; issued by the producer warp it cost 3-8 % on K = 2048
// shapes (the same queue fed without atomics cost nothing).
// Mode 1: a cluster's first item is its own index (no round trip to the counter before the first load), later ones
// are clusters + draw; a cluster that starts late still has that first item to do.  Mode 2: the first item is drawn
// as well (about half a microsecond more per launch), so a late cluster finds nothing left: the mode for GEMMs that
// run beside a collective.  The counter resets itself: each cluster draws until it misses, so exactly num_work
// (mode 2: num_work + clusters) numbers are drawn per launch and whoever draws the last one stores zero.
constexpr int kSchedAhead = 4;
constexpr int kSchedSlots = 16;
__device__ unsigned g_tile_counters[4096];

// Queue entry: tag (k + 1, 16 bits) | K slice (8 bits) | column tile (20 bits) | row tile (20 bits).  The leader's
// producer decodes the item number once, off everybody's critical path; row tile 0xFFFFF says "no more items".
constexpr u32 kSchedEnd = 0xFFFFFu;
__device__ __forceinline__ u64 sched_pack(u32 k, u32 mt, u32 nt, u32 z) {
  return ((u64)((k + 1u) & 0xFFFFu) << 48) | ((u64)z << 40) | ((u64)nt << 20) | (u64)mt;
}
__device__ __forceinline__ void sched_publish(u32 slot_local, u32 slot_peer, u64 v) {
  asm volatile("st.volatile.shared::cta.u64 [%0], %1;" ::"r"(slot_local), "l"(v) : "memory");
  asm volatile("st.volatile.shared::cluster.u64 [%0], %1;" ::"r"(slot_peer), "l"(v) : "memory");
}
// Entry k of this CTA's queue into (mt, nt, z); false when the CTA is aborting or the bounded wait expired.
__device__ __forceinline__ bool sched_wait(u32 sched0, u32 k, volatile int* abort_flag, int& mt, int& nt, int& z) {
  const u32 addr = sched0 + 8u * (k & (u32)(kSchedSlots - 1));
  const u32 tag = (k + 1u) & 0xFFFFu;
  u64 t0 = 0;
  for (u32 it = 1;; ++it) {
    u64 v;
    asm volatile("ld.volatile.shared::cta.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    if ((u32)(v >> 48) == tag) {
      mt = (int)((u32)v & 0xFFFFFu); nt = (int)((u32)(v >> 20) & 0xFFFFFu); z = (int)((u32)(v >> 40) & 0xFFu);
      return true;
    }
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      const u64 now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) { *abort_flag = 1; return false; }
      __nanosleep(100);
    }
  }
}

// Convert, scale and store the NCOLS accumulator values each lane holds for its row (32 rows per warp,
// starting at `cbase`), through this warp's staging area so that global stores are coalesced: a round
// writes one ROWB-byte row per lane into shared memory (16-byte units XOR-swizzled against bank
// conflicts), then the warp reads it back with consecutive lanes along a row and stores row segments.
template <int NCOLS, int ROWB>
__device__ __forceinline__ void staged_store(const u32 (&r)[NCOLS], float alpha, u32 sw, int lane, void* cbase, long long ldc,
                                             bool fp32, bool atomic, int valid_cols) {
  constexpr int U = ROWB / 16;            // 16-byte units per staging row
  constexpr int RPI = 32 / U;             // rows covered by one read instruction
  const u32 wswz = ROWB == 128 ? (u32)(lane & 7) : (u32)((lane >> 1) & 3);
  const u32 wr = sw + (u32)lane * ROWB;
  const int rrow = lane / U, ru = lane % U;
  if (fp32) {
    constexpr int CPR = ROWB / 4;         // columns per round
    float* cb = static_cast<float*>(cbase);
#pragma unroll
    for (int c = 0; c < NCOLS / CPR; c++) {
      if (c * CPR >= valid_cols) break;               // columns beyond N (multiples of 32): nothing to store
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = c * CPR + u * 4;
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(wr + (((u32)u ^ wswz) << 4)),
                     "f"(__uint_as_float(r[i]) * alpha), "f"(__uint_as_float(r[i + 1]) * alpha),
                     "f"(__uint_as_float(r[i + 2]) * alpha), "f"(__uint_as_float(r[i + 3]) * alpha) : "memory");
      }
      __syncwarp();
#pragma unroll
      for (int it = 0; it < U; it++) {
        const int row = it * RPI + rrow;
        const u32 rswz = ROWB == 128 ? (u32)(row & 7) : (u32)((row >> 1) & 3);
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "r"(sw + (u32)row * ROWB + (((u32)ru ^ rswz) << 4)) : "memory");
        float* dst = cb + (long long)row * ldc + c * CPR + ru * 4;
        if (atomic)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
        else
          *reinterpret_cast<float4*>(dst) = v;
      }
      __syncwarp();
    }
  } else {
    constexpr int CPR = ROWB / 2;
    __nv_bfloat16* cb = static_cast<__nv_bfloat16*>(cbase);
#pragma unroll
    for (int c = 0; c < NCOLS / CPR; c++) {
      if (c * CPR >= valid_cols) break;
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = c * CPR + u * 8;
        uint4 o;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(__uint_as_float(r[i]) * alpha, __uint_as_float(r[i + 1]) * alpha); o.x = *reinterpret_cast<u32*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * alpha, __uint_as_float(r[i + 3]) * alpha); o.y = *reinterpret_cast<u32*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * alpha, __uint_as_float(r[i + 5]) * alpha); o.z = *reinterpret_cast<u32*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * alpha, __uint_as_float(r[i + 7]) * alpha); o.w = *reinterpret_cast<u32*>(&h);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(wr + (((u32)u ^ wswz) << 4)), "r"(o.x), "r"(o.y),
                     "r"(o.z), "r"(o.w) : "memory");
      }
      __syncwarp();
#pragma unroll
      for (int it = 0; it < U; it++) {
        const int row = it * RPI + rrow;
        const u32 rswz = ROWB == 128 ? (u32)(row & 7) : (u32)((row >> 1) & 3);
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(sw + (u32)row * ROWB + (((u32)ru ^ rswz) << 4)) : "memory");
        NVFP4_STORE_C16(cb + (long long)row * ldc + c * CPR + ru * 8, v);
      }
      __syncwarp();
    }
  }
}


// Work item -> (row tile, column tile, K slice) of the pair kernel.  Tiles are walked in bands of
// kBand tile columns, row by row inside a band: the clusters of one wave then cover a roughly square
// patch of C, so every A and B tile they load is shared by about kBand clusters (one HBM read, the
// rest L2 hits) instead of each cluster streaming its own rows of A.
constexpr int kBand = 8;
__device__ __forceinline__ void decode_tile(int w, int tiles_m, int tiles_n, int& mt, int& nt, int& z) {
  const int per_z = tiles_m * tiles_n;
  z = w / per_z;
  const int r = w - z * per_z;
  const int band = r / (kBand * tiles_m);
  const int r2 = r - band * kBand * tiles_m;
  const int width = min(kBand, tiles_n - band * kBand);
  mt = r2 / width;
  nt = band * kBand + (r2 - mt * width);
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_nvf4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                      const PairParams p) {
  using C = PairCfg<BN>;
  constexpr int kStages = C::kStages;
  pdl_trigger();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* staging = smem + kStages * C::kStageBytes;
  unsigned char* bar_mem = staging + C::kStagingBytes;
  u64* full_bar = reinterpret_cast<u64*>(bar_mem);
  u64* empty_bar = full_bar + kStages;
  u64* acc_full = empty_bar + kStages;                // [2]
  u64* acc_empty = acc_full + 2;                      // [2]
  u32* tmem_slot = reinterpret_cast<u32*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  u64* sched = acc_empty + 4;                         // kSchedSlots 64-bit words behind the two 32-bit words above
  volatile u32* mma_at = reinterpret_cast<volatile u32*>(sched + kSchedSlots);   // entry the leader's MMA warp works on

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const u32 rank = cluster_ctarank();                 // 0 = leader (issues the MMAs), 1 = peer
  const int tiles_m = p.M / 256, tiles_n = (p.N + BN - 1) / BN;
  const int ktiles = (p.K + kBK - 1) / kBK;
  const int num_work = tiles_m * tiles_n * p.splitk;
  const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
  const u32 sched0 = smem_u32(sched);
  const u32 smem_base = smem_u32(smem);
  const u32 full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
  const u32 accf0 = smem_u32(acc_full), acce0 = smem_u32(acc_empty);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(accf0 + 8 * a, 1); mbar_init(acce0 + 8 * a, 2 * kEpiWarps); }
    *abort_flag = 0;
    for (int i = 0; i < kSchedSlots; i++) sched[i] = 0ull;      // tag 0 matches no entry
    *mma_at = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem2_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem2_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();                                 // barriers of both CTAs exist before anyone signals them
  tc_fence_after();
  const u32 tmem_base = *tmem_slot;
  pdl_wait();         // operands, scales and alpha words are earlier kernels' results; C may still be read by them

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfa) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfb) : "memory");
    }
    const u32 leader_full0 = map_to_cta(full0, 0);    // the leader's `full` barriers in cluster address space
    int stage = 0; u32 phase = 0;
    u32 st_addr = smem_base;
    bool ok = true;
    for (u32 k = 0; ok; k++) {
      int mt, nt, z;
      if ((k == 0 && p.dynamic != 2) || !p.dynamic) {
        const int w = cid + (int)k * ncl;
        if (w >= num_work) break;
        decode_tile(w, tiles_m, tiles_n, mt, nt, z);
      } else {
        if (!sched_wait(sched0, k, abort_flag, mt, nt, z)) { ok = false; break; }
        if (mt == (int)kSchedEnd) break;
      }
      const int kt0 = z * p.ktiles_per_split;
      const int kt1 = min(ktiles, kt0 + p.ktiles_per_split);
      const int ya = mt * 256 + (int)rank * 128, yb = nt * BN + (int)rank * (BN / 2);
      const int za = mt * 2 + (int)rank, zb = (nt * BN) >> 7;
      for (int kt = kt0; kt < kt1; kt++) {
        if (!__all_sync(0xffffffffu, NVFP4_IDLE_WAIT(empty0 + 8 * stage, phase ^ 1u, abort_flag))) { ok = false; break; }
        if (elect_one()) {
          if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * stage, C::kTxBytes);
          const u32 bar = leader_full0 + 8 * stage;
          tma2_load_2d(st_addr, &map_a, kt * kBKBytes, ya, bar);
          tma2_load_2d(st_addr + C::kABytes, &map_b, kt * kBKBytes, yb, bar);
          tma2_load_3d(st_addr + C::kABytes + C::kBBytes, &map_sfa, 0, kt * 4, za, bar);
          tma2_load_3d(st_addr + C::kABytes + C::kBBytes + C::kSFABytes, &map_sfb, 0, kt * 4, zb, bar);
        }
        st_addr += C::kStageBytes;
        if (++stage == kStages) { stage = 0; phase ^= 1u; st_addr = smem_base; }
      }
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 11);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      constexpr u32 idesc = make_idesc_pair(BN);
      const u32 sfa_t = tmem_base + C::kSfaCol, sfb_t = tmem_base + C::kSfbCol;
      const u32 empty_peer0 = map_to_cta(empty0, 1), accf_peer0 = map_to_cta(accf0, 1);
      int stage = 0; u32 phase = 0;
      const u32 a_lo0 = (smem_base >> 4) | (1u << 16);
      u32 a_lo = a_lo0;
      u32 tile = 0;                                   // tiles done by this cluster
      bool ok = true;
      for (; ok; tile++) {
        int mt, nt, z;
        if ((tile == 0 && p.dynamic != 2) || !p.dynamic) {
          const int w = cid + (int)tile * ncl;
          if (w >= num_work) break;
          decode_tile(w, tiles_m, tiles_n, mt, nt, z);
        } else {
          if (!sched_wait(sched0, tile, abort_flag, mt, nt, z)) { ok = false; break; }
          if (mt == (int)kSchedEnd) break;
        }
        if (lane == 0) *mma_at = tile;                // the drawing warp may go kSchedAhead entries beyond this one
        const int kt0 = z * p.ktiles_per_split;
        const int kt1 = min(ktiles, kt0 + p.ktiles_per_split);
        const u32 acc = tile & 1u;
        // a 192-wide tile starts 0 or 64 rows into its first 128-row scale block: 0 or 2 columns in
        const u32 sfb_m = sfb_t + (BN == 192 ? (u32)(((nt * BN) & 127) >> 5) : 0u);
        // BN = 256: wait until the previous tile's epilogues (both CTAs) have handed back the 48 columns
        // the two accumulators share.  BN = 128: wait until this accumulator's previous tile (two tiles
        // ago) has been drained.
        {
          const u32 bar = BN == 256 ? acce0 : acce0 + 8 * acc;
          const u32 par = BN == 256 ? ((tile & 1u) ^ 1u) : (((tile >> 1) & 1u) ^ 1u);
          if (!__all_sync(0xffffffffu, mbar_wait(bar, par, abort_flag))) { ok = false; break; }
        }
        tc_fence_after();
        const u32 d_tmem = tmem_base + (acc ? C::kAccOff1 : 0);
        u32 accum = 0u;
        for (int kt = kt0; kt < kt1; kt++) {
          if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * stage, phase, abort_flag))) { ok = false; break; }
          const u32 b_lo = a_lo + (C::kABytes >> 4);
          const u32 sfa_lo = (a_lo & 0xFFFFu) + ((C::kABytes + C::kBBytes) >> 4);
          const u32 sfb_lo = sfa_lo + (C::kSFABytes >> 4);
          const int krem = p.K - kt * kBK;
          const int kchunks = krem >= kBK ? 4 : (krem >> 6);
          if (elect_one()) {
            if (kchunks == 4) {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                tc2_cp_sf(sfa_t + 4 * j, pack64(sfa_lo + 32 * j, kDescHiSF));
#pragma unroll
                for (int h = 0; h < C::kSfbBlocks; h++)
                  tc2_cp_sf(sfb_t + (4 * C::kSfbBlocks) * j + 4 * h, pack64(sfb_lo + 128 * h + 32 * j, kDescHiSF));
              }
              tc2_mma_nvf4(d_tmem, pack64(a_lo, kDescHiAB), pack64(b_lo, kDescHiAB), idesc, sfa_t, sfb_m, accum);
#pragma unroll
              for (int j = 1; j < 4; j++)
                tc2_mma_nvf4(d_tmem, pack64(a_lo + 2 * j, kDescHiAB), pack64(b_lo + 2 * j, kDescHiAB), idesc, sfa_t + 4 * j,
                             sfb_m + (4 * C::kSfbBlocks) * j, 1u);
            } else {
              for (int j = 0; j < kchunks; j++) {
                tc2_cp_sf(sfa_t + 4 * j, pack64(sfa_lo + 32 * j, kDescHiSF));
#pragma unroll
                for (int h = 0; h < C::kSfbBlocks; h++)
                  tc2_cp_sf(sfb_t + (4 * C::kSfbBlocks) * j + 4 * h, pack64(sfb_lo + 128 * h + 32 * j, kDescHiSF));
              }
              for (int j = 0; j < kchunks; j++)
                tc2_mma_nvf4(d_tmem, pack64(a_lo + 2 * j, kDescHiAB), pack64(b_lo + 2 * j, kDescHiAB), idesc, sfa_t + 4 * j,
                             sfb_m + (4 * C::kSfbBlocks) * j, (j > 0) ? 1u : accum);
            }
            // free the stage in both CTAs once these MMAs have read it
            tc2_commit(empty0 + 8 * stage);
            tc2_commit(empty_peer0 + 8 * stage);
          }
          accum = 1u;
          a_lo += C::kStageBytes >> 4;
          if (++stage == kStages) { stage = 0; phase ^= 1u; a_lo = a_lo0; }
        }
        if (!ok) break;
        // accumulator complete: tell the epilogues of both CTAs
        const u32 fb = BN == 256 ? 0u : 8u * acc;
        if (elect_one()) { tc2_commit(accf0 + fb); tc2_commit(accf_peer0 + fb); }
      }
      if (!ok && lane == 0 && p.status) atomicExch(p.status, 12);
    }
  } else if (warp == 2 + kEpiWarps) {
    // ------------------------------------------------------------------ work-item draws (leader CTA only, one lane)
    if (p.dynamic && rank == 0 && lane == 0) {
      const u32 sched_peer0 = map_to_cta(sched0, 1);
      // first items dealt out (dynamic == 1): clusters + draw, num_work draws in all; first items drawn too
      // (dynamic == 2): item = draw, num_work + clusters draws in all
      const bool all = p.dynamic == 2;
      const u32 last_draw = (u32)num_work - 1u + (all ? (u32)ncl : 0u);       // the draw that finds the counter complete
      bool fail = false;
      for (u32 k = all ? 0u : 1u;; k++) {
        // flow control against the MMA warp's position, bounded like every wait
        u64 t0 = 0;
        for (u32 it = 1; k > *mma_at + (u32)kSchedAhead; ++it) {
          __nanosleep(200);
          if ((it & 15u) == 0u) {
            if (*abort_flag) { fail = true; break; }
            const u64 now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) { *abort_flag = 1; fail = true; break; }
          }
        }
        if (fail) break;
        const u32 drawn = atomicAdd(p.counter, 1u);
        if (drawn == last_draw) atomicExch(p.counter, 0u);      // every draw of this launch has happened
        const int w = (all ? 0 : ncl) + (int)drawn;
        int mt = (int)kSchedEnd, nt = 0, z = 0;
        if (w < num_work) decode_tile(w, tiles_m, tiles_n, mt, nt, z);
        const u32 slot = 8u * (k & (u32)(kSchedSlots - 1));
        sched_publish(sched0 + slot, sched_peer0 + slot, sched_pack(k, (u32)mt, (u32)nt, (u32)z));
        if (w >= num_work) break;
      }
      if (fail && p.status) atomicExch(p.status, 14);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    constexpr int NC = C::kEpiCols;
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const u32 sw = smem_u32(staging) + (u32)(warp - 2) * (32u * C::kStageRowBytes);   // this warp's staging area
    const u32 acce_leader0 = map_to_cta(acce0, 0);
    u32 tile = 0;
    bool ok = true;
    for (; ok; tile++) {
      int mt, nt, zz;
      if ((tile == 0 && p.dynamic != 2) || !p.dynamic) {
        const int w = cid + (int)tile * ncl;
        if (w >= num_work) break;
        decode_tile(w, tiles_m, tiles_n, mt, nt, zz);
      } else {
        if (!sched_wait(sched0, tile, abort_flag, mt, nt, zz)) { ok = false; break; }
        if (mt == (int)kSchedEnd) break;
      }
      const u32 acc = tile & 1u;
      {
        const u32 bar = BN == 256 ? accf0 : accf0 + 8 * acc;
        const u32 par = BN == 256 ? (tile & 1u) : ((tile >> 1) & 1u);
        // BN = 256: the warps that own the 48 columns the two accumulators share are on the critical path of the
        // next tile's first MMA (it waits for their hand-back), so they poll instead of sleeping
        const bool critical = BN == 256 && ((acc && half == 0) || (!acc && half == 1));
        const bool got = critical ? mbar_wait(bar, par, abort_flag) : NVFP4_IDLE_WAIT(bar, par, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      }
      tc_fence_after();
      u32 r[NC];
      const u32 t_row = tmem_base + ((u32)(quad * 32) << 16) + (acc ? (u32)C::kAccOff1 : 0u) + (u32)(half * NC);
      const u32 rel_bar = BN == 256 ? acce_leader0 : acce_leader0 + 8 * acc;
#define NVFP4_LD32(I) tc_ld32(t_row + (I), *reinterpret_cast<u32(*)[32]>(&r[(I)]))
#define NVFP4_LD16(I) tc_ld16(t_row + (I), *reinterpret_cast<u32(*)[16]>(&r[(I)]))
#define NVFP4_RELEASE_ACC() { tc_wait_ld(); tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive_cluster(rel_bar); }
      if constexpr (BN == 256) {
        if (acc && half == 0) {
          // this warp's first 48 columns are the shared ones: read them, hand them back, read the rest
          NVFP4_LD32(0); NVFP4_LD16(32);
          NVFP4_RELEASE_ACC();
          NVFP4_LD16(48); NVFP4_LD32(64); NVFP4_LD32(96);
          tc_wait_ld();
        } else if (!acc && half == 1) {
          // this warp's last 48 columns are the shared ones
          NVFP4_LD16(80); NVFP4_LD32(96);
          NVFP4_RELEASE_ACC();
          NVFP4_LD32(0); NVFP4_LD32(32); NVFP4_LD16(64);
          tc_wait_ld();
        } else {
          // none of this warp's columns is shared with the other accumulator
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(rel_bar);
          NVFP4_LD32(0); NVFP4_LD32(32); NVFP4_LD32(64); NVFP4_LD32(96);
          tc_wait_ld();
        }
      } else {
        NVFP4_LD32(0); NVFP4_LD32(32);
        if constexpr (NC == 96) NVFP4_LD32(64);
        NVFP4_RELEASE_ACC();
      }
#undef NVFP4_LD32
#undef NVFP4_LD16
#undef NVFP4_RELEASE_ACC

      const long long row0 = (long long)mt * 256 + rank * 128 + quad * 32;      // first row of this warp
      float alpha = 1.f;
      if (p.alpha_mode == NVFP4_ALPHA_GS) alpha = ld_cg_f32(p.pa) * ld_cg_f32(p.pb);
      else if (p.alpha_mode == NVFP4_ALPHA_AMAX) alpha = ld_cg_f32(p.pa) * ld_cg_f32(p.pb) * p.kscale;
      else if (p.alpha_mode == NVFP4_ALPHA_ROW) alpha = ld_cg_f32(p.pa + row0 + lane) * ld_cg_f32(p.pb);   // each lane stages its own row
      const long long col0 = (long long)nt * BN + half * NC;
      // (a warp's 32 rows never straddle two owners: rows_per_owner is a multiple of 128)
      float* cf = p.rows_per_owner ? p.owner_c[(int)row0 / p.rows_per_owner] : static_cast<float*>(p.c);
      void* cbase = p.c_fp32 ? static_cast<void*>(cf + row0 * p.ldc + col0)
                             : static_cast<void*>(static_cast<__nv_bfloat16*>(p.c) + row0 * p.ldc + col0);
      staged_store<NC, C::kStageRowBytes>(r, alpha, sw, lane, cbase, p.ldc, p.c_fp32 != 0, p.atomic != 0,
                                          (int)min((long long)NC, (long long)p.N - col0));
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 13);
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    const u64 t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();                                 // neither CTA frees tensor memory or exits while the other still works
  if (warp == 1) {
    tc_fence_after();
    tmem2_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------- host side
// rows x kbytes byte matrix with row stride ld bytes; box = box_rows x 128 bytes, 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long kbytes, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld};
  const cuuint32_t box[2] = {(cuuint32_t)kBKBytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int g_dynamic_sched = 1;   // pair kernel: 0 = work items dealt out in advance, 1 = drawn at run time after a cluster's first, 2 = all drawn
static int g_sm_budget = 0;  // 0 = all SMs; otherwise the persistent GEMM grids use at most this many (even) SMs
static int g_pair_bn = 0;    // 0 = heuristic, 128 / 192 / 256 = forced tile width of the CTA-pair kernel
static int g_force_bn = 0;   // 0 = heuristic, 128 / 256 = forced one-CTA tile width, 512 = CTA-pair kernel (tuning and tests)

// Swizzled scale bytes of an [R, K/16] operand seen as a 3-D tensor of 32-bit words:
// {128 words of one 512-byte tile, K/64 tiles along K, R/128 row blocks}; box = 4 tiles x `rb_box` row blocks.
static bool make_sf_map(CUtensorMap* map, const void* base, long long rows, long long K, int rb_box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {128, (cuuint64_t)(K / 64), (cuuint64_t)(rows / 128)};
  const cuuint64_t strides[2] = {512, (cuuint64_t)(K / 64) * 512};
  const cuuint32_t box[3] = {128, 4, (cuuint32_t)rb_box};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct DevInfo { int sms; bool attr128, attr256, attr_pair, attr_pair128, attr_pair192; unsigned* counters; };
static DevInfo* dev_info() {
  static DevInfo info[64];
  static bool init[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!init[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return nullptr;
    info[dev].sms = n; info[dev].attr128 = info[dev].attr256 = info[dev].attr_pair = info[dev].attr_pair128 = info[dev].attr_pair192 = false;
    void* ctr = nullptr;
    if (cudaGetSymbolAddress(&ctr, g_tile_counters) != cudaSuccess) return nullptr;
    info[dev].counters = static_cast<unsigned*>(ctr);
    init[dev] = true;
  }
  return &info[dev];
}

template <int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sms, bool& attr_done,
                       cudaStream_t st) {
  using C = Cfg<BN>;
  if (!attr_done) {
    if (cudaFuncSetAttribute(gemm_nvf4_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return NVFP4_ERR_CUDA;
    attr_done = true;
  }
  const long long work = (long long)(p.M / kBM) * (p.N / BN) * p.splitk;
  const unsigned grid = (unsigned)(work < sms ? work : sms);
  if (nvfp4_launch_kernel(gemm_nvf4_kernel<BN>, dim3(grid), dim3(kThreads), C::kSmemBytes, st, ma, mb, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVFP4_ERR_CUDA;
  }
  return NVFP4_OK;
}

}  // namespace nvfp4

using namespace nvfp4;

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// `owners` (null for the plain GEMM): n_owners base addresses of C, one per rank; see PairParams::owner_c
static int gemm_impl(const void* a, const void* sa, long long lda, const void* b, const void* sb, long long ldb,
                     void* c, int c_dtype, long long ldc, int M, int N, int K, int alpha_mode, const float* pa,
                     const float* pb, float ka, float kb, int accumulate, int splitk, int* status, void* stream,
                     void* const* owners, int n_owners, int rows_per_owner) {
  if (!a || !sa || !b || !sb || !c) return NVFP4_ERR_NULL;
  if (alpha_mode < NVFP4_ALPHA_ONE || alpha_mode > NVFP4_ALPHA_ROW) return NVFP4_ERR_ENUM;
  if (alpha_mode != NVFP4_ALPHA_ONE && (!pa || !pb)) return NVFP4_ERR_NULL;
  if (c_dtype != NVFP4_DTYPE_BF16 && c_dtype != NVFP4_DTYPE_FP32) return NVFP4_ERR_ENUM;
  if (M < 0 || N < 0 || K < 0 || (M % 128) || (N % 128) || (K % 64) || splitk < 0) return NVFP4_ERR_SHAPE;
  if (lda < K / 2 || ldb < K / 2 || ldc < N) return NVFP4_ERR_SHAPE;
  if ((accumulate || splitk > 1) && c_dtype != NVFP4_DTYPE_FP32) return NVFP4_ERR_ENUM;
  const bool auto_split = splitk == 0;      // the library picks the number of K slices (FP32 output only)
  if (auto_split) splitk = 1;
  if (!al16(a) || !al16(b) || !al16(sa) || !al16(sb) || !al16(c) || (lda & 15) || (ldb & 15) || (ldc & 7))
    return NVFP4_ERR_ALIGN;
  if (M == 0 || N == 0) return NVFP4_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    // empty contraction: C = 0 unless accumulating
    if (!accumulate) {
      const size_t es = c_dtype == NVFP4_DTYPE_FP32 ? 4 : 2;
      if (cudaMemset2DAsync(c, (size_t)ldc * es, 0, (size_t)N * es, (size_t)M, st) != cudaSuccess) return NVFP4_ERR_CUDA;
    }
    return NVFP4_OK;
  }
  DevInfo* di = dev_info();
  if (!di) return NVFP4_ERR_CUDA;
  int sms = di->sms;
  if (g_sm_budget > 0 && g_sm_budget < sms) sms = g_sm_budget >= 2 ? (g_sm_budget & ~1) : 2;

  const int ktiles = (K + kBK - 1) / kBK;
  if (auto_split && c_dtype == NVFP4_DTYPE_FP32 && (M % 256 == 0) && g_force_bn == 0 && ktiles >= 16) {
    // Weight-gradient shapes have few output tiles and a long contraction: 96 or 176 tiles over 74 SM pairs leave
    // a third of the machine idle in the last round.  Slicing K evens that out; the price is the per-tile fixed
    // cost once more per slice, FP32 atomic adds instead of stores, and a zero fill when the call overwrites C.
    // Same cost model as the tile-width choice below (units of about half a microsecond).
    const long long ncl = sms / 2;
    double best = 0;
    for (int s = 1; s <= 8 && s <= ktiles; s++) {
      const int per_s = (ktiles + s - 1) / s;
      if ((ktiles + per_s - 1) / per_s != s) continue;
      const long long t256 = (N % 256 == 0) ? (long long)(M / 256) * (N / 256) * s : 0;
      const long long t192 = (long long)(M / 256) * ((N + 191) / 192) * s;
      double cost = (double)((t192 + ncl - 1) / ncl) * (1.88 + 0.3255 * per_s);
      if (t256) cost = fmin(cost, (double)((t256 + ncl - 1) / ncl) * (2.98 + 0.346 * per_s));
      if (s > 1) {
        cost *= 1.03;                                                           // atomics in the epilogue
        if (!accumulate) cost += (double)M * (double)N * 4.0 / 1.4e6;           // zero fill first
      }
      if (s == 1 || cost < best * 0.97) { best = cost; splitk = s; }
    }
    if (splitk > 1 && !accumulate) {
      if (cudaMemset2DAsync(c, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, st) != cudaSuccess) return NVFP4_ERR_CUDA;
      accumulate = 1;
    }
  }
  if (splitk > ktiles) splitk = ktiles;
  int per = (ktiles + splitk - 1) / splitk;
  splitk = (ktiles + per - 1) / per;

  // 256-wide tiles move fewer operand bytes per FLOP and need fewer issue slots; fall back to 128
  // when N demands it or when wide tiles would leave SMs without work
  bool wide = (N % 256 == 0) && ((long long)(M / kBM) * (N / 256) * splitk >= sms || (long long)(M / kBM) * (N / 128) * splitk <= sms);
  if (g_force_bn == 128) wide = false;
  if (g_force_bn == 256 && N % 256 == 0) wide = true;
  const int bn = wide ? 256 : 128;

  // CTA-pair kernels (an SM pair per 256-row tile): the fast path whenever M allows it
  bool use_pair = (M % 256 == 0) && g_force_bn != 128 && g_force_bn != 256;
  if (g_force_bn == 0 && (long long)(M / 256) * ((N + 255) / 256) * splitk < sms / 4) use_pair = false;   // too few tiles: finer tiles fill more SMs
  if (owners) use_pair = true;                    // the scatter lives in the pair kernel's epilogue only
  if (use_pair) {
    // tile width: 256 moves the fewest operand bytes per FLOP but consecutive tiles wait for each other's
    // epilogue hand-off; 192 has two independent accumulators and handles any N; 128 as well, more bytes
    int pbn = 192;
    if (N % 256 == 0) {
      // relative per-tile cost of a CTA pair fitted to measurements: 256-wide 2.98 + 0.346 per K tile, 192-wide
      // 1.88 + 0.3255 (0.78 of the 256-wide tile at K = 2048, 0.89 at K = 11264); what decides is mostly how
      // evenly the tile count divides over the SM pairs
      const long long ncl = sms / 2;
      const long long r256 = ((long long)(M / 256) * (N / 256) * splitk + ncl - 1) / ncl;
      const long long r192 = ((long long)(M / 256) * ((N + 191) / 192) * splitk + ncl - 1) / ncl;
      if (r256 * (2.98 + 0.346 * per) <= r192 * (1.88 + 0.3255 * per)) pbn = 256;
    }
    if (g_pair_bn == 128 || g_pair_bn == 192 || (g_pair_bn == 256 && N % 256 == 0)) pbn = g_pair_bn;   // forced (tuning and tests)
    CUtensorMap ma, mb, msa, msb;
    if (!make_map(&ma, a, M, K / 2, lda, 128) || !make_sf_map(&msa, sa, M, K, 1) ||
        !make_map(&mb, b, N, K / 2, ldb, pbn / 2) || !make_sf_map(&msb, sb, N, K, pbn == 128 ? 1 : 2))
      return NVFP4_ERR_CUDA;
    PairParams pp;
    pp.c = c; pp.pa = pa; pp.pb = pb; pp.status = status; pp.ldc = ldc;
    pp.kscale = ka * kb * (1.f / (kFp4E4m3 * kFp4E4m3));
    pp.M = M; pp.N = N; pp.K = K;
    pp.alpha_mode = alpha_mode;
    pp.c_fp32 = c_dtype == NVFP4_DTYPE_FP32;
    pp.atomic = (accumulate || splitk > 1) ? 1 : 0;
    pp.splitk = splitk;
    pp.ktiles_per_split = per;
    pp.rows_per_owner = owners ? rows_per_owner : 0;
    for (int r = 0; r < kMaxOwners; r++) pp.owner_c[r] = (owners && r < n_owners) ? static_cast<float*>(owners[r]) : nullptr;
    // a counter of its own for every launch in flight: consecutive launches take consecutive slots, a slot comes
    // round again 4096 launches later
    static std::atomic<unsigned> launch_seq{0};
    pp.counter = di->counters + (launch_seq.fetch_add(1u, std::memory_order_relaxed) & 4095u);
    // (items shorter than four K tiles stay dealt out in advance: one draw takes about as long as such an item)
    pp.dynamic = (g_dynamic_sched && per >= 4 && splitk <= 255 && (M / 256) < (int)kSchedEnd && (N + pbn - 1) / pbn <= (int)kSchedEnd) ? g_dynamic_sched : 0;
    const long long work = (long long)(M / 256) * ((N + pbn - 1) / pbn) * splitk;
    const long long clusters = work < sms / 2 ? work : sms / 2;
    const unsigned grid = (unsigned)(2 * clusters);
#define NVFP4_LAUNCH_PAIR(BN_, FLAG)                                                                                      \
    {                                                                                                                      \
      if (!di->FLAG) {                                                                                                     \
        if (cudaFuncSetAttribute(gemm_nvf4_pair_kernel<BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                 PairCfg<BN_>::kSmemBytes) != cudaSuccess)                                                 \
          return NVFP4_ERR_CUDA;                                                                                           \
        di->FLAG = true;                                                                                                   \
      }                                                                                                                    \
      if (nvfp4_launch_kernel(gemm_nvf4_pair_kernel<BN_>, dim3(grid), dim3(kPairThreads), PairCfg<BN_>::kSmemBytes, st, ma, mb,\
                              msa, msb, pp) != cudaSuccess) {                                                               \
        (void)cudaGetLastError();                                                                                          \
        return NVFP4_ERR_CUDA;                                                                                             \
      }                                                                                                                    \
    }
    if (pbn == 256) NVFP4_LAUNCH_PAIR(256, attr_pair)
    else if (pbn == 192) NVFP4_LAUNCH_PAIR(192, attr_pair192)
    else NVFP4_LAUNCH_PAIR(128, attr_pair128)
#undef NVFP4_LAUNCH_PAIR
    NVFP4_LAUNCH_CHECK();
    return NVFP4_OK;
  }

  CUtensorMap ma, mb;
  if (!make_map(&ma, a, M, K / 2, lda, kBM) || !make_map(&mb, b, N, K / 2, ldb, bn)) return NVFP4_ERR_CUDA;

  GemmParams p;
  p.sfa = static_cast<const unsigned char*>(sa);
  p.sfb = static_cast<const unsigned char*>(sb);
  p.c = c; p.pa = pa; p.pb = pb; p.status = status; p.ldc = ldc;
  p.kscale = ka * kb * (1.f / (kFp4E4m3 * kFp4E4m3));
  p.M = M; p.N = N; p.K = K;
  p.alpha_mode = alpha_mode;
  p.c_fp32 = c_dtype == NVFP4_DTYPE_FP32;
  p.atomic = (accumulate || splitk > 1) ? 1 : 0;
  p.splitk = splitk;
  p.ktiles_per_split = per;
  if (wide) return launch_gemm<256>(ma, mb, p, sms, di->attr256, st);
  return launch_gemm<128>(ma, mb, p, sms, di->attr128, st);
}

extern "C" int nvfp4_gemm(const void* a, const void* sa, long long lda, const void* b, const void* sb, long long ldb,
                          void* c, int c_dtype, long long ldc, int M, int N, int K, int alpha_mode, const float* pa,
                          const float* pb, float ka, float kb, int accumulate, int splitk, int* status, void* stream) {
  return gemm_impl(a, sa, lda, b, sb, ldb, c, c_dtype, ldc, M, N, K, alpha_mode, pa, pb, ka, kb, accumulate, splitk,
                   status, stream, nullptr, 0, 0);
}

// The weight-gradient GEMM of a data-parallel rank with the reduce-scatter in its epilogue: C is [M, N] FP32 with the
// same layout on every rank, rank r owns rows [r * M / n_owners, (r + 1) * M / n_owners), and this rank's product is
// ADDED (red.global.add.v4.f32, through the peer mapping for r != this rank) into each owner's rows.  The caller has
// cleared the owned rows on every rank and synchronised the ranks before the first launch of a step, and synchronises
// them again (after this stream's work) before an owner reads its rows.
extern "C" int nvfp4_gemm_scatter_rows(const void* a, const void* sa, long long lda, const void* b, const void* sb,
                                       long long ldb, void* const* owners, int n_owners, long long ldc, int M, int N,
                                       int K, int alpha_mode, const float* pa, const float* pb, float ka, float kb,
                                       int splitk, int* status, void* stream) {
  if (!owners) return NVFP4_ERR_NULL;
  if (n_owners < 1 || n_owners > kMaxOwners || M <= 0 || (M % 256) || (M % n_owners) || ((M / n_owners) % 128))
    return NVFP4_ERR_SHAPE;
  for (int r = 0; r < n_owners; r++) {
    if (!owners[r]) return NVFP4_ERR_NULL;
    if (!al16(owners[r])) return NVFP4_ERR_ALIGN;
  }
  return gemm_impl(a, sa, lda, b, sb, ldb, owners[0], NVFP4_DTYPE_FP32, ldc, M, N, K, alpha_mode, pa, pb, ka, kb, 1,
                   splitk, status, stream, owners, n_owners, M / n_owners);
}

extern "C" size_t nvfp4_gemm_linear_workspace_bytes(int M, int N, int K) {
  if (M < 0 || N < 0 || K < 0) return 0;
  return ((size_t)M + (size_t)N) * (size_t)(K / 16);
}

extern "C" int nvfp4_gemm_linear(const void* a, const void* sa, long long lda, long long ldsa, const void* b, const void* sb,
                                 long long ldb, long long ldsb, void* c, int c_dtype, long long ldc, int M, int N, int K,
                                 int alpha_mode, const float* pa, const float* pb, float ka, float kb, int accumulate,
                                 int splitk, void* workspace, size_t workspace_bytes, int* status, void* stream) {
  if (!sa || !sb) return NVFP4_ERR_NULL;
  if (M < 0 || N < 0 || K < 0 || (M % 128) || (N % 128) || (K % 64)) return NVFP4_ERR_SHAPE;
  if (!workspace || workspace_bytes < nvfp4_gemm_linear_workspace_bytes(M, N, K)) return NVFP4_ERR_WORKSPACE;
  if (!al16(workspace)) return NVFP4_ERR_ALIGN;
  unsigned char* wsa = static_cast<unsigned char*>(workspace);
  unsigned char* wsb = wsa + (size_t)M * (size_t)(K / 16);      // M % 128 == 0 keeps this 16-byte aligned
  int rc = nvfp4_swizzle_scales(sa, ldsa, M, K / 16, wsa, stream);
  if (rc != NVFP4_OK) return rc;
  rc = nvfp4_swizzle_scales(sb, ldsb, N, K / 16, wsb, stream);
  if (rc != NVFP4_OK) return rc;
  return nvfp4_gemm(a, wsa, lda, b, wsb, ldb, c, c_dtype, ldc, M, N, K, alpha_mode, pa, pb, ka, kb, accumulate, splitk,
                    status, stream);
}

extern "C" int nvfp4_gemm_set_scheduler(int dynamic) {
  g_dynamic_sched = dynamic < 0 ? 0 : dynamic > 2 ? 2 : dynamic;
  return NVFP4_OK;
}

// Clears the work counters of the pair kernel's scheduler on the current device: needed only after a launch was
// abandoned (a bounded wait expired and the status word was set), which can leave a counter half-way.
extern "C" int nvfp4_gemm_reset_scheduler(void) {
  DevInfo* di = dev_info();
  if (!di) return NVFP4_ERR_CUDA;
  if (cudaMemset(di->counters, 0, sizeof(unsigned) * 4096) != cudaSuccess) return NVFP4_ERR_CUDA;
  return NVFP4_OK;
}

// The budget as the persistent quantizer / emitter grids read it (0 = none).
int nvfp4_sm_budget_value() { return g_sm_budget; }

extern "C" int nvfp4_gemm_set_sm_budget(int sms) {
  if (sms < 0 || sms == 1) return NVFP4_ERR_SHAPE;   // the CTA-pair grids need at least one SM pair
  g_sm_budget = sms;
  return NVFP4_OK;
}

extern "C" int nvfp4_gemm_force_tile_n(int bn) {
  if (bn != 0 && bn != 128 && bn != 256 && bn != 512 && bn != 384 && bn != 448) return NVFP4_ERR_ENUM;
  g_pair_bn = bn == 512 ? 256 : bn == 448 ? 192 : bn == 384 ? 128 : 0;
  g_force_bn = bn >= 384 ? 512 : bn;
  return NVFP4_OK;
}

extern "C" int nvfp4_version(void) { return 100; }

extern "C" const char* nvfp4_error_string(int status) {
  switch (status) {
    case NVFP4_OK: return "ok";
    case NVFP4_ERR_NULL: return "a required pointer is null";
    case NVFP4_ERR_SHAPE: return "a size violates the divisibility rules of the entry point";
    case NVFP4_ERR_ALIGN: return "a pointer or stride is not aligned as required";
    case NVFP4_ERR_ENUM: return "unknown or unsupported layout / dtype / mode value";
    case NVFP4_ERR_CUDA: return "a CUDA runtime or driver call failed";
    case NVFP4_ERR_WORKSPACE: return "workspace missing or too small";
    case NVFP4_ERR_TOO_LARGE: return "a size exceeds a documented maximum";
    default: return "unknown status";
  }
}

