/*
 * nvfp4_b200 -- C ABI of the B200 (sm_100a) NVFP4 linear-layer kernels.
 *
 * Drop-in boundary: these entry points take the place of the CUDA kernels the reference
 * (Not4right/nvfp4-training) compiles at run time with NVRTC and launches through CuPy
 * (llm-1b/nvrtc_util.py:53-67).  Each declaration names the reference kernel/launcher it replaces.
 *
 * Conventions (inherited from the reference launcher):
 *   - every pointer is a DEVICE pointer unless stated otherwise; the caller owns all memory;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns at once:
 *     no host synchronisation, no device-scalar read-back, no allocation;
 *   - device scalars (amax, gs) stay on the device;
 *   - return value: 0 = enqueued, negative = rejected before any launch (see nvfp4_error_string).
 *
 * Data formats (llm-1b/nvq.cu:1-7):
 *   codes   E2M1, two per byte, low nibble = lower index, rows contiguous along the contraction dim
 *   scales  one unsigned E4M3 byte per 16 values along the contraction dim, either
 *           NVFP4_SCALES_SWIZZLED: 128-row x 4-column tiles of 512 bytes, tiles row-block-major,
 *                                  byte (r%32)*16 + ((r%128)/32)*4 + (c%4) inside a tile
 *                                  (llm-1b/nvq.cu:40-42; the layout tcgen05 block-scaled MMA and
 *                                  cuBLASLt consume), or
 *           NVFP4_SCALES_LINEAR:   row-major [R, C/16] (llm-1b/fp4k.cu:66-87)
 *   tensor scale  gs = amax / 2688, FP32, not folded into the scales
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_OK               0
#define NVFP4_ERR_NULL        -1   /* a required pointer is null */
#define NVFP4_ERR_SHAPE       -2   /* a size violates the divisibility rules of the entry point */
#define NVFP4_ERR_ALIGN       -3   /* a pointer or stride is not aligned as required */
#define NVFP4_ERR_ENUM        -4   /* unknown layout / dtype / mode value */
#define NVFP4_ERR_CUDA        -5   /* a CUDA runtime or driver call failed (launch, attribute, tensor map) */
#define NVFP4_ERR_WORKSPACE   -6   /* workspace missing or too small */
#define NVFP4_ERR_TOO_LARGE   -7   /* a size exceeds a documented maximum */

#define NVFP4_SCALES_SWIZZLED  0
#define NVFP4_SCALES_LINEAR    1

#define NVFP4_DTYPE_BF16       0
#define NVFP4_DTYPE_FP32       1

/* rounding of the codes */
#define NVFP4_ROUND_NEAREST     0  /* round to nearest even (cvt.rn.satfinite.e2m1x2.f32)               */
#define NVFP4_ROUND_SR_DITHER   1  /* mantissa-dither SR + random stream of llm-1b/nvq.cu:32-39,52-59   */
#define NVFP4_ROUND_SR_DITHER_K 2  /* same rounding, random stream of llm-1b/fp4k.cu:53-58              */
#define NVFP4_ROUND_SR_HW       3  /* cvt.rs.satfinite.e2m1x4.f32, counter-based stream of this library */

/* how nvfp4_gemm forms the output scale alpha */
#define NVFP4_ALPHA_ONE         0  /* alpha = 1                       (llm-1b/nvq.py:94 scale=False)    */
#define NVFP4_ALPHA_GS          1  /* alpha = *pa * *pb               (llm-1b/nvq.py:93: gsA*gsB)       */
#define NVFP4_ALPHA_AMAX        2  /* alpha = *pa * *pb * ka*kb/2688^2 (llm-1b/fp4k.cu:261)             */
#define NVFP4_ALPHA_ROW         3  /* alpha[row] = pa[row] * *pb: per-row scale of the A operand times the
                                      tensor scale of B, the separate `scale_rows` pass of llm-1b/model2.py:152-154
                                      done in the epilogue; pa = device FP32 [M] */

/* Library version, major*10000 + minor*100 + patch. */
int nvfp4_version(void);

/* Static text for a status code returned by this library. */
const char* nvfp4_error_string(int status);

/*
 * Per-tensor max|x| of a contiguous bf16 tensor into *out (FP32).  *out is set to 0 first.
 * Replaces kernel `amax_bf16` (llm-1b/nvq.cu:69-90) and launcher `nvq.amax` (llm-1b/nvq.py:32-40).
 * Requires n % 8 == 0, x 16-byte aligned.  n == 0 gives 0.
 */
int nvfp4_amax_bf16(const void* x, long long n, float* out, void* stream);

/*
 * out[0] = max(out[0], max|x|): nvfp4_amax_bf16 without the clearing of out[0], for callers that clear a batch of
 * amax words with one fill (out[0] must hold a non-negative finite value or +0).  No reference counterpart.  Without
 * the fill the amax kernel follows the previous kernel of the stream directly (one graph node less per call).
 */
int nvfp4_amax_bf16_update(const void* x, long long n, float* out, void* stream);

/*
 * Programmatic dependent launch of this library's amax, one-read quantizer and GEMM kernels: when on, such a kernel
 * may become resident and run its set-up (barriers, tensor-memory allocation, constant tables) while the previous
 * kernel of the stream drains; it waits for that kernel's completion before it touches global memory, and reads
 * global memory past L1 only.  Off by default (measured gain on the 81-linear step: 0.2-0.6 %); the environment
 * variable NVFP4_PDL=1 or this call switch it on.  Process-wide; no reference counterpart.
 */
int nvfp4_set_pdl(int on);

/*
 * 1x16 block quantization of x [R, C] bf16 (row stride ldx elements) along C.
 * Replaces kernel `quant_rows` (llm-1b/nvq.cu:93-116, llm-1b/fp4k.cu:66-87) and launchers
 * `nvq.quant_rows` (llm-1b/nvq.py:47-57), `fp4ops.quant_rows` (llm-1b/fp4ops.py:30-38).
 * codes [R, C/2] bytes, contiguous.  scales: R*C/16 bytes in `scale_layout`.
 * amax: device FP32 scalar, max|x| of the whole tensor (or a larger bound).
 * gs_out: optional device FP32 scalar that receives the tensor scale gs (`nvq._gs`, llm-1b/nvq.py:43-44).
 * seed / seed_dev: stochastic-rounding seed; when seed_dev (a device word) is given it replaces
 * `seed`, so a captured CUDA graph can be replayed with a fresh seed per microbatch
 * (the reference changes `LinCtx.seed` on the host every microbatch, llm-1b/model.py:36-39,59).
 * Requires C % 16 == 0, ldx % 8 == 0, x 16-byte aligned; SWIZZLED also R % 128 == 0, C % 64 == 0.
 * Arithmetic: gs = max(amax/2688, 1e-30); bs = e4m3(min((max16|x|/gs)/6, 448));
 * code = round((x/gs)/bs) -- the operation order of small-model/model_ref.py:39-47, IEEE FP32.
 */
int nvfp4_quant_rows(const void* x, long long ldx, int R, int C, void* codes, void* scales,
                     int scale_layout, const float* amax, float* gs_out, int rounding, unsigned seed,
                     const unsigned* seed_dev, void* stream);

/*
 * Quantization of x^T along the token dim after a 16-point random Hadamard transform:
 * x [M, C] bf16 contiguous -> codes [C, M/2], scales for [C, M/16]; tensor scale uses 4*amax.
 * Bit i of `signs` negates token i of every 16-token block; butterflies of strides 1,2,4,8 in FP32,
 * then x0.25; gs_out (optional) receives gs = 4*amax/2688.  Replaces kernel `quant_cols_rht` (llm-1b/nvq.cu:122-158, llm-1b/fp4k.cu:92-117) and
 * launchers `nvq.quant_cols_rht` (llm-1b/nvq.py:60-70), `fp4ops.quant_cols_rht` (llm-1b/fp4ops.py:41-49).
 * Requires M % 16 == 0, C % 8 == 0, x 16-byte aligned; SWIZZLED also C % 128 == 0, M % 64 == 0.
 */
int nvfp4_quant_cols_rht(const void* x, int M, int C, void* codes, void* scales, int scale_layout,
                         const float* amax, float* gs_out, unsigned signs, int rounding, unsigned seed,
                         const unsigned* seed_dev, void* stream);

/*
 * One pass over x [M, C] bf16 (row stride ldx elements) producing BOTH operands the linear layer
 * needs from an activation or a gradient: the row operand of `nvfp4_quant_rows` (codes_r, scales_r,
 * gs_r_out) and the transposed RHT16 operand of `nvfp4_quant_cols_rht` (codes_c, scales_c, gs_c_out),
 * bit-identical to those two calls with seeds seed_r / seed_c (seed_*_dev: device words that
 * replace them).  Either output pair may be null to skip it.  The tensor is read from HBM once.
 * Fuses the reference's pair of launches `quant_rows(gy)` + `quant_cols_rht(gy)` (llm-1b/model.py:62-66,
 * llm-1b/nvq.py:46-70).  Two kernels stand behind it:
 *   - tensor-core fed (M % 128 == 0, C % 128 == 0, codes 16-byte and scales 4-byte aligned): TMA tiles of
 *     128 x 128, tcgen05.mma with 0/+-1 matrices converts / transposes / sign-flips the tile exactly into
 *     tensor memory, the quantizing warps read it with tcgen05.ld.  One documented difference: an input
 *     that is exactly -0 gives code 0x0 (the scalar kernels and the reference's convert give 0x8);
 *   - scalar (any other accepted shape): TMA tiles of 128 x 64 in a shared-memory ring, read by the
 *     quantizing warps.
 * Requires M % 128 == 0, C % 64 == 0 (C % 128 == 0 with SWIZZLED scales and codes_c), ldx % 8 == 0,
 * x and codes_c 16-byte aligned, codes_r and scales_c 8-byte aligned.  A wait that expires inside the kernel (1 s) is reported by nvfp4_quant_tile_status.
 */
int nvfp4_quant_tile(const void* x, long long ldx, int M, int C, void* codes_r, void* scales_r, void* codes_c,
                     void* scales_c, int scale_layout, const float* amax, float* gs_r_out, float* gs_c_out,
                     unsigned signs, int rounding, unsigned seed_r, unsigned seed_c,
                     const unsigned* seed_r_dev, const unsigned* seed_c_dev, void* stream);

/* Tuning / test hook: 0 = nvfp4_quant_tile picks the tensor-core-fed kernel where it applies (default),
 * 1 = always the scalar tile kernel, 2 = the tensor-core-fed kernel with the 16-point Hadamard transform of the
 * transposed operand computed by the MMA itself (B operand = rows of H diag(signs)) instead of FP32 butterflies, as
 * the reference's fused backward does on mma.sync (small-model/fused_bwd.cu:33-64 `emit_wg`, small-model/wg16.cu:41-103).
 * Mode 2 is not bit-exact: the tensor core sums a block's 16 signed values in its own order; results equal the
 * butterflies' whenever every partial sum is representable in FP32 and may differ in the last bit otherwise.
 * Process-wide. */
int nvfp4_quant_tile_set_path(int path);

/* Reads (synchronously) the status word of nvfp4_quant_tile launches on the current device:
 * 0, or the role whose wait expired first (scalar kernel: 1 producer, 2 consumer; tensor-core-fed kernel:
 * 17 / 19 the loading and MMA-issuing warp waiting for a tile / for a free stage, 18 a consumer; row emitter's ring
 * kernel: 33 producer, 34 consumer); `reset` != 0 clears it. */
int nvfp4_quant_tile_status(int* out, int reset);

/*
 * Row operand with an exact per-row FP32 scale, produced in one launch without a tensor-wide amax
 * pass: x [T, C] bf16 (row stride ldx) -> codes [T, C/2], swizzled block scales for [T, C/16] and
 * rs_out[t] = rowmax * (1/2688); a consumer multiplies the raw GEMM result by rs[t] * (weight scale).
 * Replaces launcher `emit.row_emit` (llm-1b/emit.py:62-68) with the kernels it dispatches: `row_emit`
 * (llm-1b/emit.cu:263-285) and, for C == 11264, `row_emit_11264` (llm-1b/emit.cu:228-260).  Arithmetic per row, IEEE FP32: inv = 2688/rowmax;
 * per 16 values sb = e4m3((max*inv)*(1/6)), k = inv/dec(sb), code = rn(x*k).  sr != 0: stochastic
 * rounding by 11-bit mantissa dither (llm-1b/emit.cu:38-43) with the reference's random sequence:
 * lane l = (column/8) % 32 of row r runs s <- s*1664525+1013904223 from hash32(rng[0] ^ salt ^
 * hash32(r*32+l)) over its 8-column chunks in column order, one step per pair of values; for C == 11264 the
 * sequence of `row_emit_11264`: four per lane, sequence s from hash32(rng[0] ^ salt ^ hash32(r*128+s*32+l)) over
 * the chunks 4 j + s.  sr == 2: hardware stochastic convert (cvt.rs.satfinite.e2m1x4.f32) with this library's
 * counter-based words, key from rng[0] ^ salt and the block index r*(C/16) + block (no reference
 * counterpart).  rng: device words (rng[0] = seed), required when sr != 0.  Requires C % 256 == 0,
 * T % 128 == 0, ldx % 8 == 0, x 16-byte aligned.  Two kernels stand behind it: rows of at most 11776 columns travel
 * as whole rows through a shared-memory ring fed by bulk copies (cp.async.bulk) and are quantized from there;
 * longer rows take a warp-per-row kernel that re-reads them through L2.  Same bytes from both.
 */
int nvfp4_emit_rows(const void* x, long long ldx, int T, int C, void* codes, void* scales, float* rs_out,
                    int sr, const unsigned* rng, unsigned salt, void* stream);

/* Tuning / test hook: 0 = nvfp4_emit_rows picks the ring kernel where it applies (default), 1 = always the
 * warp-per-row kernel.  Process-wide.  No reference counterpart. */
int nvfp4_emit_rows_set_path(int path);

/*
 * Column operand with a delayed per-tensor scale: x [M, C] bf16 (row stride ldx) -> x^T quantized
 * along the tokens after the 16-point random Hadamard transform, codes [C, M/2], swizzled scales for
 * [C, M/16].  The scale comes from *amax_use, an RHT-domain amax observed earlier (inv = 2688/amax_use);
 * the RHT-domain amax of THIS tensor is recorded into *amax_cur with atomicMax on float bits (the
 * caller zeroes it).  No amax pass over x is needed.  Replaces kernel `col_emit` (llm-1b/emit.cu:287-341)
 * and launcher `emit.col_emit` (llm-1b/emit.py:82-85).  rng: device words, rng[0] = SR seed, rng[1] =
 * Hadamard sign bits (required).  sr != 0: 11-bit mantissa dither with the reference's random
 * sequence (the thread of column c and 64-token group g starts at hash32(rng[0] ^ salt ^ hash32(c*4099+g))
 * and takes its four 16-token blocks in order, one LCG step per pair of values).  sr == 2: hardware stochastic convert
 * with this library's counter-based words (key from rng[0] ^ salt and the block index c*(M/16) + block; no reference
 * counterpart).
 * Requires M % 128 == 0, C % 128 == 0, ldx % 8 == 0, x and codes 16-byte aligned, scales 8-byte aligned.
 */
int nvfp4_emit_cols(const void* x, long long ldx, int M, int C, void* codes, void* scales,
                    const float* amax_use, unsigned* amax_cur, int sr, const unsigned* rng, unsigned salt,
                    void* stream);

/*
 * Producer-fused emitters of the reference's trainer: the row operand (codes, swizzled scales, per-row FP32 scale
 * rs_out, as nvfp4_emit_rows writes them) straight from the FP32 values a normalisation / activation computes.
 *
 * nvfp4_rms_emit replaces `rms_emit` (llm-1b/emit.cu:97-147, launcher llm-1b/emit.py:40-47): per row t of x [T, D]
 * bf16, x_new = x + y * (ys[t] * ygw[0]) when y is given (stored to xout as bf16 and continued from the stored
 * value), rstd = rsqrt(mean(x_new^2) + eps), h = (x_new * rstd) * w.  Optional outputs: h (bf16 [T, D]), rstd_out
 * (FP32 [T]), and the row operand of the FP32 h when codes is non-null (then T % 128 == 0).  D in {1024, 2048, 4096}
 * (the reference: 2048).  y non-null requires ys, ygw and xout.
 *
 * nvfp4_swiglu_emit replaces `swiglu_emit` / `swiglu_emit_5632` (llm-1b/emit.cu:149-222, launcher
 * llm-1b/emit.py:50-58): gu [T, 2F] bf16 = raw gate | up GEMM output, true value = raw * (rs_in[t] * gw[0]);
 * a = silu(g) * u.  Optional outputs: a_out (bf16 [T, F]), a_f32 (FP32 [T, F], for tests: the value that is
 * quantized), the row operand of a when codes is non-null (then T % 128 == 0).  F % 256 == 0.
 *
 * Arithmetic: FP32; fused multiply-adds for x + y*s, the sum of squares (lane l = (column/16) % 32 sums the even and
 * the odd elements of its 16-value blocks separately in column order, adds the two, then a butterfly over the 32
 * lanes) and mean + eps; round-to-nearest multiplications elsewhere; rsqrtf, __expf and the division of
 * the sigmoid are the hardware approximations, everything after them is exact IEEE arithmetic on their results.
 *
 * nvfp4_mom_acc replaces `mom_acc` (llm-1b/emit.cu:343-363): m (bf16, n values, n % 8 == 0) <- m + (alpha[0] * scale)
 * * g, rounded stochastically to bf16 (16 random bits added below the bf16 mantissa, then truncation); thread
 * i = element / 8 runs s <- s*1664525 + 1013904223 from hash32(rng[0] ^ salt ^ hash32(i)), one step per pair of values.
 */
int nvfp4_rms_emit(const void* x, const void* y, const float* ys, const float* ygw, void* xout, const void* w, void* h,
                   void* codes, void* scales, float* rs_out, float* rstd_out, int T, int D, float eps, void* stream);
int nvfp4_swiglu_emit(const void* gu, const float* rs_in, const float* gw, int F, void* a_out, float* a_f32, void* codes,
                      void* scales, float* rs_out, int T, void* stream);
int nvfp4_mom_acc(void* m, const void* g, const float* alpha, float scale, long long n, const unsigned* rng,
                  unsigned salt, void* stream);

/*
 * 16x16-block quantization of a weight w [N, K] (bf16 or fp32, contiguous): one scale per block,
 * emitting W (q [N, K/2], s for [N, K/16]) and W^T (qt [K, N/2], st for [K, N/16]) with identical
 * code values.  Either output pair may be null to skip it.
 * Replaces kernel `quant_w2d` (llm-1b/nvq.cu:162-196 bf16; llm-1b/fp4k.cu:121-158 fp32) and
 * launchers `nvq.quant_w2d` (llm-1b/nvq.py:73-87), `fp4ops.quant_w2d` (llm-1b/fp4ops.py:52-61).
 * Requires N % 16 == 0, K % 16 == 0; SWIZZLED also N % 128 == 0, K % 128 == 0; w 16-byte, q / qt / st 4-byte aligned.
 */
int nvfp4_quant_w2d(const void* w, int w_dtype, int N, int K, void* q, void* s, void* qt, void* st,
                    int scale_layout, const float* amax, float* gs_out, void* stream);

/*
 * The stochastic-rounding convert on its own, with caller-supplied random bits: group i turns
 * y[4i..4i+3] (FP32, already divided by the scales) into 16 bits of E2M1 codes, y[4i] in the lowest
 * nibble, using `cvt.rs.satfinite.e2m1x4.f32` with the random word rbits[i].  It exists so that the
 * rounding function can be checked bit-for-bit against a CPU model on identical random bits.
 * No reference counterpart (sm_120 has no cvt.rs: llm-1b/nvq.cu:31).  y 16-byte aligned.
 */
int nvfp4_e2m1x4_sr(const float* y, const unsigned* rbits, void* codes, long long n4, void* stream);

/*
 * Row-major scale bytes [R, C16] (row stride lds bytes) -> the swizzled layout.
 * No reference kernel: it converts the llm-1b/fp4k.cu scale layout into the llm-1b/nvq.cu one
 * (inverse of `nvq.unswizzle`, llm-1b/nvq.py:103-107).  Requires R % 128 == 0, C16 % 4 == 0.
 */
int nvfp4_swizzle_scales(const void* s_linear, long long lds, int R, int C16, void* s_swizzled, void* stream);

/*
 * Block-scaled FP4 GEMM  C[M,N] (+)= alpha * A[M,K] * B[N,K]^T  on tcgen05 tensor cores.
 * Replaces kernel `gemm_fp4` (llm-1b/fp4k.cu:181-280) / launcher `fp4ops.gemm`
 * (llm-1b/fp4ops.py:64-80) and the cuBLASLt call behind `nvq.mm` (llm-1b/nvq.py:90-96).
 *   a, b      packed codes, row strides lda / ldb BYTES (multiples of 16), 16-byte aligned
 *   sa, sb    scales in the SWIZZLED layout for [M, K/16] and [N, K/16], 16-byte aligned
 *   c         bf16 or fp32 [M, N], row stride ldc ELEMENTS (multiple of 8), 16-byte aligned
 *   pa, pb    device FP32 scalars used by alpha_mode (may be null for NVFP4_ALPHA_ONE); NVFP4_ALPHA_ROW: pa = FP32 [M]
 *   accumulate  0: C = result; 1: C += result (fp32 only, atomic adds)
 *   splitk    >= 1: the K range is cut into that many slices of whole 256-element tiles, each
 *             added atomically into C; needs accumulate = 1 or C zeroed by the caller when > 1.
 *             0 (fp32 C only; bf16 C runs unsliced): the library picks the slice count from its tile cost model --
 *             weight-gradient shapes with few output tiles and a long K fill the SMs better in slices -- and, when it
 *             slices a call with accumulate = 0, zero-fills C itself first.  Slices add in no fixed order, so the
 *             last bits of C may differ from run to run, as in the reference's split-K (llm-1b/fp4k.cu:272-278)
 *   status    optional device int; a CTA whose bounded pipeline wait expires writes a non-zero
 *             code there and leaves the kernel without completing its tiles (never expected)
 * Requires M % 128 == 0, N % 128 == 0, K % 64 == 0.
 */
int nvfp4_gemm(const void* a, const void* sa, long long lda, const void* b, const void* sb, long long ldb,
               void* c, int c_dtype, long long ldc, int M, int N, int K,
               int alpha_mode, const float* pa, const float* pb, float ka, float kb,
               int accumulate, int splitk, int* status, void* stream);

/*
 * Tuning hook: force the kernel variant of nvfp4_gemm: 128 or 256 = one-CTA tiles of that many columns,
 * 512 / 448 / 384 = the CTA-pair kernel with 256x256 / 256x192 / 256x128 tiles over an SM pair (needs M a
 * multiple of 256; 512 also N), 0 restores the built-in choice.  Process-wide; a variant the shape does not allow is ignored.  No reference
 * counterpart (the reference kernel has one fixed 128x128 tile, llm-1b/fp4k.cu:164-167).
 */
int nvfp4_gemm_force_tile_n(int bn);

/*
 * Cap the number of SMs the persistent grids occupy (0 = all): the GEMM, and the one-read quantizer, the tile
 * kernel and the ring emitter, whose CTAs each own a fixed share of the tiles or rows (a CTA that finds its SM taken
 * and starts late would finish a whole share late).  Meant for data-parallel runs: leaving a few SMs free lets the
 * NCCL all-reduce kernels of the weight gradients run beside them.  Process-wide; takes effect for later calls (a captured
 * CUDA graph keeps the grid it was captured with).  No reference counterpart (single GPU).
 */
int nvfp4_gemm_set_sm_budget(int sms);

/*
 * The CTA-pair GEMM hands out its work items at run time from a per-launch counter in device memory (a grid that finds
 * SMs occupied by another kernel shares the items among the CTAs that do run); the counter returns to zero when a
 * launch completes.  After a launch that was abandoned (status word set by an expired wait) call this once to clear
 * the counters of the current device.  Synchronises the device.  No reference counterpart.
 */
int nvfp4_gemm_reset_scheduler(void);
/* 1 (default): a cluster's first item is its own index, later ones are drawn at run time; 2: the first one is drawn
 * too (half a microsecond more per launch; for GEMMs that run beside another kernel: a cluster that starts late then
 * leaves no item waiting for it); 0: dealt out in advance, cluster c takes items c, c + clusters, ...  Process-wide. */
int nvfp4_gemm_set_scheduler(int dynamic);

/*
 * The weight-gradient GEMM of a data-parallel rank with the gradient reduce-scatter in its epilogue (no reference
 * counterpart: the reference's trainers are single-GPU; this replaces the reduce half of the dW all-reduce that a
 * data-parallel wrapper around llm-1b/model.py:85 would issue).  C = A B^T is [M, N] FP32 with leading dimension
 * ldc, laid out the same on every rank; rank r owns rows [r * M / n_owners, (r + 1) * M / n_owners) and owners[r] is
 * the address of C in rank r's memory as this process sees it (a peer mapping; this rank's own buffer for itself).
 * The product is ADDED into each owner's rows (FP32 reductions that commute: no ordering between ranks is needed).
 * Protocol kept by the caller: every rank clears its owned rows, the ranks synchronise, any number of these calls
 * run, the ranks synchronise again behind them, then each owner's rows hold the sum over ranks (an all-gather
 * of the row slabs completes the all-reduce).  owners is a HOST array, read during the call.
 * M % 256 == 0, (M / n_owners) % 128 == 0, 1 <= n_owners <= 8; other arguments as nvfp4_gemm (splitk 0 = library's
 * choice).
 */
int nvfp4_gemm_scatter_rows(const void* a, const void* sa, long long lda, const void* b, const void* sb,
                            long long ldb, void* const* owners, int n_owners, long long ldc, int M, int N, int K,
                            int alpha_mode, const float* pa, const float* pb, float ka, float kb, int splitk,
                            int* status, void* stream);

/*
 * Same product for operands whose scales are in the LINEAR layout (row strides ldsa / ldsb bytes):
 * the scales are first rewritten into the swizzled layout inside `workspace`, then nvfp4_gemm runs.
 * This is the `fp4ops.gemm` contract (llm-1b/fp4ops.py:64-80: strided d and s views allowed).
 * workspace: device memory of at least nvfp4_gemm_linear_workspace_bytes(M, N, K) bytes, 16-byte
 * aligned, owned by the caller and free for reuse once the stream has passed this call.
 */
size_t nvfp4_gemm_linear_workspace_bytes(int M, int N, int K);
int nvfp4_gemm_linear(const void* a, const void* sa, long long lda, long long ldsa,
                      const void* b, const void* sb, long long ldb, long long ldsb,
                      void* c, int c_dtype, long long ldc, int M, int N, int K,
                      int alpha_mode, const float* pa, const float* pb, float ka, float kb,
                      int accumulate, int splitk, void* workspace, size_t workspace_bytes,
                      int* status, void* stream);

/*
 * nvfp4_gemm_linear without a workspace argument, for callers that cannot obtain device memory at
 * call time (no counterpart in the reference, whose launcher always allocates with torch:
 * llm-1b/fp4ops.py:67-72).  The re-swizzled scales go into a fixed array inside the library, so the
 * call allocates nothing -- no cudaMalloc/cudaFree, no allocating library routine.
 *   limit    (M + N) * K / 16 <= nvfp4_gemm_linear_noalloc_max_scratch() (8 MiB); larger problems are
 *            rejected with NVFP4_ERR_TOO_LARGE before anything is launched
 *   cost     every GPU on which the library is loaded holds those 8 MiB until the process exits
 *   first call on a device: looks up the array's device address (cudaGetSymbolAddress) with that
 *            device current; make this first call outside any stream capture.  The first launch of
 *            each kernel variant a shape selects also makes the CUDA runtime load that kernel and set
 *            its shared-memory attribute, which may reserve driver memory once: the guarantee of no
 *            allocation holds from the second call with a given shape class on
 *   sharing  all calls on a device use the same array, which keeps the previous call's bytes (each
 *            call overwrites what it reads, nothing has to start at zero); two calls whose kernels
 *            can overlap on the GPU -- different streams without ordering -- race on it
 * Everything else (arguments, results, status codes) is exactly nvfp4_gemm_linear.
 */
size_t nvfp4_gemm_linear_noalloc_max_scratch(void);
int nvfp4_gemm_linear_noalloc(const void* a, const void* sa, long long lda, long long ldsa,
                              const void* b, const void* sb, long long ldb, long long ldsb,
                              void* c, int c_dtype, long long ldc, int M, int N, int K,
                              int alpha_mode, const float* pa, const float* pb, float ka, float kb,
                              int accumulate, int splitk, int* status, void* stream);

/*
 * Self-test of the bounded waits: launches one CTA that waits on a barrier nobody arrives on, with a
 * limit of limit_us microseconds (1..1000), and ORs into *status (device int, zeroed by the caller)
 * bit 0 when the limited wait gave up, bit 1 when the CTA's second warp left through the abort flag,
 * and in bits 8.. the microseconds the first warp waited.  parked != 0 exercises the sleeping form of
 * the wait.  The kernel has no copies in flight and always terminates.  No reference counterpart (the
 * reference kernels have no waits).
 */
int nvfp4_selftest_wait_timeout(unsigned limit_us, int parked, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
