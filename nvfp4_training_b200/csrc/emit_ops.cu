// Row-operand emitter with an exact per-row FP32 scale (sm_100a): one launch, no tensor-wide amax
// pass.  Reference: `row_emit` of llm-1b/emit.cu:263-285 and, for 11264-column rows, `row_emit_11264`
// (llm-1b/emit.cu:228-260), as the launcher llm-1b/emit.py:62-68 dispatches them; the arithmetic
// (multiplications by reciprocals, IEEE here) and both random sequences are reproduced bit for bit.
//
// One warp per row.  Lane l owns the 8-column chunks 256 j + 8 l of its row: that is the unit the
// reference's per-lane random sequence is defined on, and a warp-wide load of one chunk index j
// is 512 contiguous bytes.  Rows of up to 5632 columns stay in registers between the row-max pass
// and the quantization pass (packed bf16, 4 registers per chunk); longer rows are read a second
// time, which L2 serves.
#include "emit_chunk.cuh"

namespace nvfp4 {

// KEEP = number of chunks per lane held in registers (C == 256 * KEEP), or 0 for rows of any
// length that are read twice.  SUBS = 4 reproduces the random sequence of the kernel the reference's launcher
// picks for 11264-column rows (`row_emit_11264` = row_reg<4, 11>, llm-1b/emit.cu:228-260, llm-1b/emit.py:64-67): four
// sequences per lane, sequence s seeded with hash32(seed ^ salt ^ hash32(r*128 + s*32 + lane)) and walking the
// chunks 4 j + s in order; SUBS = 1 is the generic `row_emit` sequence (one per lane, seeded with r*32 + lane).
template <int KEEP, int SR, int SUBS = 1>
__global__ void __launch_bounds__(256) emit_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int C,
                                                        u32* __restrict__ codes, unsigned char* __restrict__ scales,
                                                        float* __restrict__ rs_out, int T, const u32* __restrict__ rng,
                                                        u32 salt) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const __nv_bfloat16* row = x + r * ldx + lane * 8;
  constexpr int NK = KEEP > 0 ? KEEP : 1;
  uint4 kept[NK];
  u32 mm = 0u;
  if (KEEP > 0) {
#pragma unroll
    for (int j = 0; j < NK; j++) kept[j] = ld_chunk(row + j * 256);
#pragma unroll
    for (int j = 0; j < NK; j++) mm = absmax_packed(mm, kept[j]);
  } else {
    for (int c = 0; c < C; c += 256) mm = absmax_packed(mm, ld_chunk(row + c));
  }
  mm = max(mm & 0xFFFFu, mm >> 16);
#pragma unroll
  for (int o = 16; o; o >>= 1) mm = max(mm, __shfl_xor_sync(0xffffffffu, mm, o));
  const float am = __uint_as_float(mm << 16);
  const float inv = am > 0.f ? __fdiv_rn(kFp4E4m3, am) : 0.f;
  if (lane == 0) rs_out[r] = __fmul_rn(am, 1.f / kFp4E4m3);
  const u32 seed = (SR ? __ldg(rng) : 0u) ^ salt;
  if (SUBS == 4) {
    u32 lcg4[4];
#pragma unroll
    for (int sidx = 0; sidx < 4; sidx++) lcg4[sidx] = hash32(seed ^ hash32((u32)(r * 128 + sidx * 32 + lane)));
    for (int c = 0; c < C; c += 1024)
#pragma unroll
      for (int sidx = 0; sidx < 4; sidx++)
        emit_chunk<SR>(ld_chunk(row + c + sidx * 256), inv, lcg4[sidx], r, c + sidx * 256 + lane * 8, C, codes, scales, lane);
    return;
  }
  u32 lcg = SR == 2 ? seed : hash32(seed ^ hash32((u32)(r * 32 + lane)));
  if (KEEP > 0) {
#pragma unroll
    for (int j = 0; j < NK; j++) emit_chunk<SR>(kept[j], inv, lcg, r, j * 256 + lane * 8, C, codes, scales, lane);
  } else {
    for (int c = 0; c < C; c += 256) emit_chunk<SR>(ld_chunk(row + c), inv, lcg, r, c + lane * 8, C, codes, scales, lane);
  }
}

template <int KEEP>
static void launch_rows(int sr, unsigned blocks, cudaStream_t st, const __nv_bfloat16* x, long long ldx, int C, u32* codes,
                        unsigned char* scales, float* rs, int T, const u32* rng, u32 salt) {
  if (sr == 2) emit_rows_kernel<KEEP, 2><<<blocks, 256, 0, st>>>(x, ldx, C, codes, scales, rs, T, rng, salt);
  else if (sr) emit_rows_kernel<KEEP, 1><<<blocks, 256, 0, st>>>(x, ldx, C, codes, scales, rs, T, rng, salt);
  else emit_rows_kernel<KEEP, 0><<<blocks, 256, 0, st>>>(x, ldx, C, codes, scales, rs, T, rng, salt);
}

}  // namespace nvfp4

using namespace nvfp4;

// the TMA-fed kernel (emit_rows_ring.cu)
bool nvfp4_emit_rows_ring_accepts(const void* x, long long ldx, int T, int C, const void* codes);
int nvfp4_emit_rows_ring_launch(const void* x, long long ldx, int T, int C, void* codes, void* scales, float* rs_out,
                                int sr, const unsigned* rng, unsigned salt, void* stream);

static int g_emit_rows_path = 0;   // 0 = TMA-fed kernel where it applies, 1 = always the warp-per-row kernel

extern "C" int nvfp4_emit_rows_set_path(int path) {
  if (path != 0 && path != 1) return NVFP4_ERR_ENUM;
  g_emit_rows_path = path;
  return NVFP4_OK;
}

extern "C" int nvfp4_emit_rows(const void* x, long long ldx, int T, int C, void* codes, void* scales, float* rs_out,
                               int sr, const unsigned* rng, unsigned salt, void* stream) {
  if (!x || !codes || !scales || !rs_out || (sr && !rng)) return NVFP4_ERR_NULL;
  if (T < 0 || C < 0 || (C & 255) || ldx < C || (T & 127)) return NVFP4_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (ldx & 7) || (reinterpret_cast<uintptr_t>(codes) & 3u)) return NVFP4_ERR_ALIGN;
  if (sr < 0 || sr > 2) return NVFP4_ERR_ENUM;
  if (T == 0 || C == 0) return NVFP4_OK;
  if (g_emit_rows_path == 0 && nvfp4_emit_rows_ring_accepts(x, ldx, T, C, codes))
    return nvfp4_emit_rows_ring_launch(x, ldx, T, C, codes, scales, rs_out, sr, rng, salt, stream);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((T + 7) / 8);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  u32* cp = static_cast<u32*>(codes);
  unsigned char* sp = static_cast<unsigned char*>(scales);
  switch (C / 256) {
    case 8: launch_rows<8>(sr, blocks, st, xp, ldx, C, cp, sp, rs_out, T, rng, salt); break;
    case 12: launch_rows<12>(sr, blocks, st, xp, ldx, C, cp, sp, rs_out, T, rng, salt); break;
    case 22: launch_rows<22>(sr, blocks, st, xp, ldx, C, cp, sp, rs_out, T, rng, salt); break;
    case 44:   // 11264 columns: the reference's launcher switches to its four-sequence kernel here
      if (sr == 1) emit_rows_kernel<0, 1, 4><<<blocks, 256, 0, st>>>(xp, ldx, C, cp, sp, rs_out, T, rng, salt);
      else launch_rows<0>(sr, blocks, st, xp, ldx, C, cp, sp, rs_out, T, rng, salt);
      break;
    default: launch_rows<0>(sr, blocks, st, xp, ldx, C, cp, sp, rs_out, T, rng, salt); break;
  }
  NVFP4_LAUNCH_CHECK();
  return NVFP4_OK;
}
