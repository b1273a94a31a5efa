/*
 * altob200 -- C ABI of the B200 (sm_100a) low-precision linear path.
 *
 * The reference (AMD-AGI/ALTO) has no FFI for this path: its seam is a set of
 * Python callables backed by Triton kernels.  Each entry point below names the
 * reference callable whose device work it replaces (path inside the reference
 * project : line).  All pointers are DEVICE pointers unless stated otherwise,
 * all sizes are in elements unless stated otherwise, `stream` is a
 * cudaStream_t passed as void*, and every function returns 0 on success or a
 * negative ALTOB200_E* code.  Nothing here allocates device memory unless the
 * comment of the function says so; outputs are owned by the caller.
 *
 * Quantised data layouts
 * ----------------------
 *  codes (FP4)  : uint8, two E2M1 codes per byte, the element with the even
 *                 index along the quantisation axis in the low nibble
 *                 (alto/kernels/fp4/mxfp4/mxfp_quantization.py:184-186).
 *  codes (FP8)  : one byte per element (float8_e4m3fn or float8_e5m2).
 *  plain scales : row-major [rows, cols/block] (1D) or [rows/block, cols/block]
 *                 (2D); MXFP4/MXFP8: uint8 E8M0 exponent, NVFP4: float32 value
 *                 on the E4M3 grid (alto/kernels/fp4/nvfp4/nvfp_quantization.py:558).
 *  packed scales: the layout the tcgen05 block-scaled MMA reads from tensor
 *                 memory: uint8 (E8M0 or E4M3), tiles of 128 rows x 4 scale
 *                 columns = 512 bytes, tile (rb, cb) at ((rb * ceil(ncols/4)) + cb) * 512,
 *                 element (r, c) of a tile at (r % 32) * 16 + (r / 32) * 4 + c.
 *                 Rows and columns are padded to multiples of 128 and 4; padded
 *                 entries are written as zero.  Size: altob200_packed_scale_bytes().
 */
#ifndef ALTOB200_H_
#define ALTOB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define ALTOB200_OK 0
#define ALTOB200_EINVAL_SHAPE (-1)   /* a size/divisibility contract is violated      */
#define ALTOB200_EINVAL_ALIGN (-2)   /* a pointer or leading dimension is misaligned  */
#define ALTOB200_ETIMEOUT_DEVICE (-3) /* a bounded device-side wait gave up           */
#define ALTOB200_ECUDA (-4)          /* a CUDA runtime/driver call failed             */
#define ALTOB200_EUNSUPPORTED (-5)   /* valid request this build does not implement   */
#define ALTOB200_ELIMIT (-6)         /* a size exceeds a stated fixed maximum         */

/* ---- enums (plain ints in the ABI) ------------------------------------- */
/* element formats */
#define ALTOB200_FMT_NVFP4 0      /* E2M1, block 16, E4M3 inner scale (+fp32 outer) */
#define ALTOB200_FMT_MXFP4 1      /* E2M1, block 32, E8M0 scale                     */
#define ALTOB200_FMT_MXFP8_E4M3 2 /* E4M3, block 32, E8M0 scale                     */
#define ALTOB200_FMT_MXFP8_E5M2 3 /* E5M2, block 32, E8M0 scale                     */
/* high-precision dtypes */
#define ALTOB200_DT_BF16 0
#define ALTOB200_DT_F32 1
/* scale output layouts */
#define ALTOB200_SCALE_PLAIN 1
#define ALTOB200_SCALE_PACKED 2
/* rounding */
#define ALTOB200_ROUND_RTN 0
#define ALTOB200_ROUND_SR_BITS 1   /* stochastic rounding, caller supplies 32 random bits per element */
#define ALTOB200_ROUND_SR_PHILOX 2 /* stochastic rounding, Philox-4x32-10 generated in the kernel     */

int altob200_version(void);
const char* altob200_status_string(int status);

/* Bytes of a packed scale buffer for `rows` x `ncols` scale entries. */
size_t altob200_packed_scale_bytes(int64_t rows, int64_t ncols);

/* Reads (and clears) the sticky device-side status word written by kernels
 * whose bounded waits gave up.  Synchronises `stream`.  Returns 0 or
 * ALTOB200_ETIMEOUT_DEVICE; `detail` (host, may be NULL) receives
 * {kernel id, block id, wait site, 0}. */
int altob200_status_read(void* stream, int32_t detail[4]);

#define ALTOB200_CLIP_NONE 0
#define ALTOB200_CLIP_STATIC 1
#define ALTOB200_CLIP_DYNAMIC 2

/* ---- quantizer parameters ---------------------------------------------- */
typedef struct altob200_quant_params {
  int32_t format;      /* ALTOB200_FMT_*                                             */
  int32_t in_dtype;    /* ALTOB200_DT_*                                              */
  int32_t rounding;    /* ALTOB200_ROUND_*                                           */
  int32_t scale_flags; /* ALTOB200_SCALE_PLAIN | ALTOB200_SCALE_PACKED               */
  /* NVFP4 tensorwise outer scale (device float[1]) or NULL when outer scaling is off
   * (alto/kernels/fp4/nvfp4/nvfp_quantization.py:273-287).                         */
  const float* outer_scale;
  /* ROUND_SR_BITS: device uint32 [2][rows_q][cols_q/2] in the quantisation-axis-last
   * view; plane 0 feeds even elements, plane 1 odd elements
   * (alto/kernels/fp4/fp4_common/triton_fp4_ops.py:13-19,
   *  alto/kernels/fp4/mxfp4/mxfp_quantization.py:128-132,184-186).                  */
  const uint32_t* rand_bits;
  /* ROUND_SR_PHILOX: Philox-4x32-10 with key = (seed lo, seed hi) and counter =
   * (c lo, c hi, 0, 0), c = philox_offset + q, where q = (pair index) / 2 and the pair
   * index is r * (cols_q / 2) + c / 2 in the quantisation-axis-last view.  The four
   * output words feed, in order, the even and odd element of pair 2q and the even and
   * odd element of pair 2q+1.  (The generator is the one triton.language.randint4x uses,
   * alto/kernels/fp4/fp4_common/triton_fp4_ops.py:13-19; the word-to-element mapping is
   * this library's own and uses all four words of a call.)                            */
  uint64_t philox_seed;
  uint64_t philox_offset;
  /* Randomised Hadamard transform applied along the row axis before an axis-0
   * quantisation (alto/kernels/hadamard_transform/transform.py:115-142).  0 = off,
   * else the block size n (16).  The n x n matrix is W = (diag(sign) H_n)[perm][:, perm]
   * with H_n the Sylvester matrix; `rht_perm[i]` and `rht_sign[i]` (+1/-1) are HOST
   * arrays of length n.                                                              */
  int32_t rht_n;
  const int32_t* rht_perm;
  const int32_t* rht_sign;
  /* MXFP4 only (alto/kernels/fp4/mxfp4/mxfp_quantization.py:29-95, 321-322, 420-438):
   * clip_mode STATIC multiplies the elements by 3/4 before encoding (scale unchanged);
   * DYNAMIC takes the scale from 2.92247856/6 * std(block) + 1e-8 with target exponent 0
   * (1-D blocks only); use_uos != 0 computes the scale as ceil(log2(amax / 7.25)) + 127.
   * Arithmetic is done in the input dtype, as in the reference's emulation
   * (tests/unittest/mxfp4/utils.py:320-358).                                          */
  int32_t clip_mode;
  int32_t use_uos;
  /* ROUND_SR_BITS with a periodic table: when both are non-zero, rand_bits is
   * [2][rand_tile_rows][rand_tile_pairs] and element pair (r, p) of the quantisation-axis-last
   * view reads entry (r % rand_tile_rows, p % rand_tile_pairs).  With the table written by
   * altob200_philox_tile this reproduces the reference kernels' stochastic rounding for a given
   * (philox_seed, philox_offset) bit for bit.  rand_tile_pairs must be a multiple of 8 for the
   * row-wise quantizer.                                                                  */
  int64_t rand_tile_rows;
  int64_t rand_tile_pairs;
} altob200_quant_params;

/*
 * Absolute maximum of a [rows, cols] matrix with leading dimension `ld`
 * (elements).  Replaces the three eager kernels of compute_dynamic_outer_scale
 * (alto/kernels/fp4/nvfp4/nvfp_quantization.py:460-487).
 *
 *  amax_bits[0] <- max |x|            (fp32 bit pattern, NaN elements ignored)
 *  amax_bits[1] <- max |bf16(W x/sqrt(n))| over row blocks of n when p->rht_n != 0
 *  outer_scale[i] <- max(amax_i / (448 * 6), 1e-30) for i in {0,1} when non-NULL
 *
 * `scratch` is device memory of at least ALTOB200_AMAX_SCRATCH_BYTES that must be
 * zero before the first call; the kernel leaves it zeroed again (a ticket counter and the
 * running maxima live there, so amax_bits need not be cleared and no launch precedes the
 * kernel; amax_bits[1] is written as 0 without a transform).  Calls that share a scratch
 * buffer must be ordered on one stream.
 */
#define ALTOB200_AMAX_SCRATCH_BYTES 16
int altob200_amax(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, int64_t ld,
                  int32_t rht_n, const int32_t* rht_perm, const int32_t* rht_sign,
                  uint32_t* amax_bits, float* outer_scale, void* scratch, void* stream);

/*
 * Absolute maximum of a [rows, cols] matrix (and the NVFP4 outer scale derived from
 * it) for callers that must not allocate device memory and cannot hand over a
 * scratch buffer of their own -- for example a step that runs inside a memory pool
 * which is already fully planned, a plugin living in another runtime's address
 * space, or an inference server whose allocator is frozen after start-up.  This
 * entry point has no counterpart in the reference; it computes what altob200_amax
 * computes without a Hadamard transform:
 *
 *  amax_bits[0]   <- max |x| as an fp32 bit pattern
 *  outer_scale[0] <- max(amax / (448 * 6), 1e-30) when non-NULL
 *
 * It calls no cudaMalloc / cudaFree and no allocating library routine.  Its working
 * memory (one partial maximum per thread block and a completion counter, about
 * 33 KiB) is a fixed array inside the library's device image; every GPU that loads
 * the library keeps those bytes until the process exits.  Consequences:
 *  - the input is limited to ALTOB200_NOALLOC_MAX_BYTES (one array slot per 64 KiB
 *    of input); larger inputs are refused with ALTOB200_ELIMIT before any launch;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and keeps it; make that first
 *    call before starting any stream capture, and do not call again on a device
 *    after cudaDeviceReset in the same process (the kept address is then stale);
 *  - all calls on one device share the array: two calls whose kernels may overlap on
 *    the GPU (different streams, no dependency between them) race and give wrong
 *    results; calls on one stream are safe, and each call resets what it needs.
 */
#define ALTOB200_NOALLOC_MAX_BYTES (512ll << 20)
int altob200_amax_noalloc(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, int64_t ld,
                          uint32_t* amax_bits, float* outer_scale, void* stream);

/*
 * 1D block quantisation along the last (contiguous) axis of x[rows, cols].
 * Replaces convert_to_mxfp4 / convert_to_nvfp4 / convert_to_mxfp8 with axis=-1,
 * is_2d_block=False (alto/kernels/fp4/mxfp4/mxfp_quantization.py:411-484,
 * alto/kernels/fp4/nvfp4/nvfp_quantization.py:491-630,
 * alto/kernels/mxfp8/mxfp8_quantization.py:483-586).
 *   codes       : [rows, cols/2] (FP4) or [rows, cols] (FP8), row-major
 *   scale_plain : [rows, cols/block] (uint8 or float32), may be NULL
 *   scale_packed: packed layout with rows=rows, ncols=cols/block, may be NULL
 */
int altob200_quantize_rowwise(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              const altob200_quant_params* p, void* codes, void* scale_plain,
                              void* scale_packed, void* stream);

/*
 * 1D block quantisation along axis 0 (blocks of consecutive ROWS) of
 * x[rows, cols], optionally preceded by the randomised Hadamard transform over
 * row blocks of p->rht_n.  Replaces the axis=0 calls of the same reference
 * functions, whose physical output is the transposed matrix
 * (alto/kernels/fp4/mxfp4/mxfp_quantization.py:439-443,484):
 *   codes       : [cols, rows/2] (FP4) or [cols, rows] (FP8), row-major
 *   scale_plain : [cols, rows/block]
 *   scale_packed: packed layout with rows=cols, ncols=rows/block
 */
int altob200_quantize_colwise(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              const altob200_quant_params* p, void* codes, void* scale_plain,
                              void* scale_packed, void* stream);

/*
 * 2D block quantisation (block x block tiles share one scale) of w[rows, cols].
 * Replaces the is_2d_block=True calls of the same reference functions (scale
 * derivation: alto/kernels/fp4/mxfp4/mxfp_quantization.py:44-57,
 * alto/kernels/fp4/nvfp4/nvfp_quantization.py:246-251,
 * alto/kernels/mxfp8/mxfp8_quantization.py:36-78).  2D scales do
 * not depend on the axis, so one read of w produces both operand packings:
 *   codes_k       : [rows, cols/2]  (packed along cols; forward operand)
 *   codes_t       : [cols, rows/2]  (packed along rows; dgrad operand), may be NULL
 *   scale_plain   : [rows/block, cols/block], may be NULL
 *   scale_packed_k: packed layout rows=rows, ncols=cols/block (2D scale broadcast per row), may be NULL
 *   scale_packed_t: packed layout rows=cols, ncols=rows/block, may be NULL
 * Rounding: ALTOB200_ROUND_RTN, or (FP4 formats) ALTOB200_ROUND_SR_BITS with rand_bits indexed by
 * (row, column pair) exactly as in altob200_quantize_rowwise - full planes [2][rows][cols/2] or the
 * periodic table [2][rand_tile_rows][rand_tile_pairs], rand_tile_pairs a multiple of 4; both packings
 * then hold the same stochastically rounded codes (the 2-D-block gradient of a use_2dblock_x linear is
 * quantised once, alto/kernels/fp4/nvfp4/nvfp_linear.py:176-186).  No Hadamard transform.
 */
int altob200_quantize_2d(const void* w, int64_t rows, int64_t cols, int64_t ld,
                         const altob200_quant_params* p, void* codes_k, void* codes_t,
                         void* scale_plain, void* scale_packed_k, void* scale_packed_t,
                         void* stream);

/*
 * The same for `batch` equally shaped matrices in one launch (the experts of a MoE weight [E, N, K],
 * alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:633-652): matrix b starts batch_stride
 * elements after matrix b - 1; every output holds the per-matrix outputs of altob200_quantize_2d one
 * after the other (codes_k [batch][rows][cols/2], codes_t [batch][cols][rows/2], scale_plain
 * [batch][rows/block][cols/block], packed scales batch x altob200_packed_scale_bytes(..)).  With
 * stochastic rounding the rows of the random-word view are the rows of all matrices in sequence,
 * as in the reference's flattened view.
 */
int altob200_quantize_2d_batched(const void* w, int64_t batch, int64_t batch_stride, int64_t rows, int64_t cols,
                                 int64_t ld, const altob200_quant_params* p, void* codes_k, void* codes_t,
                                 void* scale_plain, void* scale_packed_k, void* scale_packed_t, void* stream);

/*
 * The reference's table of stochastic-rounding words: out[0][m][n], out[1][m][n] = first and second
 * word of Philox-4x32-10 with key (seed lo, seed hi) and counter (uint32(offset + m * tile_pairs + n),
 * 0, 0, 0), which is `r1, r2, _, _ = tl.randint4x(seed, offset + m * n_pairs + n)` of
 * alto/kernels/fp4/fp4_common/triton_fp4_ops.py:13-19.  The reference draws this same table in every
 * BLOCK_M x BLOCK_N tile (BLOCK = min(64, extent), alto/kernels/fp4/mxfp4/mxfp_quantization.py:452-459,
 * alto/kernels/fp4/nvfp4/nvfp_quantization.py:591-598): tile_rows = BLOCK_M, tile_pairs = BLOCK_N / 2.
 * out: device uint32 [2][tile_rows][tile_pairs], 16-byte aligned.
 */
int altob200_philox_tile(uint64_t seed, uint64_t offset, int64_t tile_rows, int64_t tile_pairs, uint32_t* out,
                         void* stream);

/*
 * Dequantisation of row-major codes[rows, cols(/2)] with plain scales.
 * Replaces convert_from_mxfp4 / convert_from_nvfp4 / convert_from_mxfp8
 * (alto/kernels/fp4/mxfp4/mxfp_quantization.py:488-545,
 *  alto/kernels/fp4/nvfp4/nvfp_quantization.py:634-711,
 *  alto/kernels/mxfp8/mxfp8_quantization.py:590-663) for the axis-last view;
 * `is_2d`: bit 0 selects [rows/block, cols/block] scales; bit 1 (MXFP4 only) is the static
 * clip of the reference's dequantizer: decoded values times 4/3 in the output dtype before the
 * scale (alto/kernels/fp4/mxfp4/mxfp_quantization.py:404-405).
 */
int altob200_dequantize(const void* codes, const void* scale_plain, const float* outer_scale,
                        int32_t format, int32_t is_2d, int64_t rows, int64_t cols,
                        int32_t out_dtype, void* out, int64_t ld_out, void* stream);

/*
 * Randomised Hadamard transform alone: y = bf16/f32( (W x_block) / sqrt(n) ) over
 * row blocks of n (alto/kernels/hadamard_transform/transform.py:115-142, left_mul=True).
 */
int altob200_rht(const void* x, int32_t dtype, int64_t rows, int64_t cols, int64_t ld,
                 int32_t rht_n, const int32_t* rht_perm, const int32_t* rht_sign, void* y,
                 int64_t ld_y, void* stream);

/*
 * The same transform with an arbitrary n x n matrix W = weight[perm][:, perm] given on the
 * device (fp32, row-major), n in {16, 32, 64}: y = cast((W x_block) * fp32(1 / sqrt(n))), the
 * way PyTorch evaluates the reference's division by the 0-dim sqrt(n) tensor on CUDA
 * (alto/kernels/hadamard_transform/transform.py:115-142; matrix construction
 * alto/kernels/hadamard_transform/hadamard.py:63-161, whose table matrices, e.g. the default
 * n = 32, are not of Sylvester type).  rows must be a multiple of n.
 */
int altob200_rht_dense(const void* x, int32_t dtype, int64_t rows, int64_t cols, int64_t ld, int32_t n,
                       const float* w, void* y, int64_t ld_y, void* stream);

/*
 * Macro-block two-level scaling for MXFP4: before the E8M0 quantiser, each block of 128
 * elements is multiplied by a factor in [1, 2) whose top 8 mantissa bits are those of
 * 6 / amax(block); the 8 bits are stored as one uint8 per block.  Replaces macro_block_scaling
 * (alto/kernels/fp4/mxfp4/macro_block_scaling.py:35-96, host wrapper :236-288, public
 * op :423-428).  x and y are contiguous [batch, rows, cols] of `dtype`; any cols (4-wide
 * accesses are used when cols is a multiple of 4 and both pointers are 16-byte aligned).
 *   mode 0: blocks along the last axis;   scale [batch, rows, ceil(cols/128)]
 *   mode 1: 128 x 128 tiles;              scale [batch, ceil(rows/128), ceil(cols/128)]
 *   mode 2: blocks down the row axis (the reference's axis=0 on a matrix, which it reaches
 *           through a transposed view);   scale [batch, cols, ceil(rows/128)]
 * Ragged last blocks take their amax over the elements that exist.
 */
int altob200_macro_block_scaling(const void* x, int32_t dtype, int64_t batch, int64_t rows, int64_t cols,
                                 int32_t mode, void* y, uint8_t* scale, void* stream);

/*
 * Inverse of the above: x = y / factor(scale).  Replaces macro_block_descaling
 * (alto/kernels/fp4/mxfp4/macro_block_scaling.py:100-146, host wrapper :345-420, public
 * op :431-437).
 */
int altob200_macro_block_descaling(const void* y, const uint8_t* scale, int32_t dtype, int64_t batch, int64_t rows,
                                   int64_t cols, int32_t mode, void* x, void* stream);

/*
 * DGE factor on a weight gradient, in place: dw[n, k] = cast(float(dw[n, k]) * lut[code(W[n, k])]).
 * Replaces `grad_weights * dge_bwd(w_fp4_values, float4_e2m1fn_x2)` (alto/kernels/dge/dge.py:81-93;
 * alto/kernels/fp4/nvfp4/nvfp_linear.py:250-268, alto/kernels/fp4/mxfp4/mxfp_linear.py:546-566):
 * the bin value of a weight element is one of sixteen numbers, so the factor is a table over its
 * E2M1 code.  `codes_t` is the packed weight operand of the dgrad GEMM, [K, N/2] with element n in
 * nibble n & 1; `lut16` is a HOST array of 16 floats indexed by the 4-bit code.
 */
int altob200_dge_scale(void* dw, int32_t dtype, int64_t N, int64_t K, int64_t ld, const void* codes_t,
                       const float* lut16, void* stream);

/*
 * Weight de-oscillation bookkeeping after an optimizer step, in one pass over n elements:
 * dist_w += |w - prev|, dist_qdq += |w_qdq - prev_qdq|, prev = w, where w_qdq / prev_qdq are the
 * quantise-dequantise round trips of w and prev on the forward pass's grid.  Replaces the five
 * tensor ops of _DeOscillationHook._step_param (alto/components/optimizer.py:381-386).  All arrays
 * have `dtype`; with bf16 every intermediate is rounded to bf16 as the tensor ops round.
 */
int altob200_deosc_accumulate(const void* w, void* prev, const void* w_qdq, const void* prev_qdq, void* dist_w,
                              void* dist_qdq, int64_t n, int32_t dtype, void* stream);

/*
 * Row gather with zero fill: dst[i] = index[i] >= 0 ? src[index[i]] : zeros, rows of row_bytes
 * (a multiple of 16; both pointers 16-byte aligned).  The MoE token path around the grouped
 * GEMMs: sort routed rows by expert and pad each expert's run to a multiple of 128 rows (index
 * -1), and the inverse.  The reference leaves this to its TorchTitan fork's token dispatcher
 * (call sites alto/modifiers/lpt/base.py:194-201, alto/kernels/dispatch/tensor.py:224-263); the
 * grouped kernels fix the result's form (alto/kernels/fp4/fp4_common/grouped_utils.py:81-94).
 * `index` is device int32 [out_rows]; entries outside [0, src_rows) give zero rows.
 */
int altob200_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes, const int32_t* index,
                         int64_t out_rows, void* dst, void* stream);

/*
 * Weighted combine of the k routed rows of every token, bf16 (the end of the MoE token path, same
 * call sites as altob200_gather_rows):
 *   out[t] = bf16( sum_j f32( bf16( rows[index[t k + j]] * scores[t k + j] ) ) ),  j = 0 .. k-1
 * i.e. a row gather, the multiplication by the routing scores and the sum over k in one pass, with
 * the roundings of the tensor-op form.  index: device int32 [tokens * k], entries outside
 * [0, n_rows) contribute nothing; scores: device bf16 [tokens * k] or NULL (weights of one).
 * altob200_spread_rows is its gradient with respect to the rows:
 *   grad_rows[r] = bf16( grad_out[position[r] / k] * scores[position[r]] ),  zero rows where position[r] < 0,
 * with position: device int32 [n_rows], the routed slot t k + j that row r feeds.
 * row_bytes a multiple of 16, pointers 16-byte aligned.
 */
int altob200_combine_rows(const void* rows, int64_t n_rows, int64_t row_bytes, const int32_t* index,
                          const void* scores, int64_t tokens, int32_t k, void* out, void* stream);
int altob200_spread_rows(const void* grad_out, int64_t tokens, int32_t k, int64_t row_bytes,
                         const int32_t* position, const void* scores, int64_t n_rows, void* grad_rows,
                         void* stream);

/*
 * SwiGLU between the two grouped GEMMs of an expert MLP, bf16.  h is [rows, 2H] with row stride
 * ld_h elements (gate in columns [0, H), up in [H, 2H)); forward writes out [rows, H] =
 * bf16(bf16(silu(gate)) * up); backward takes grad_out [rows, H] and writes grad_h [rows, 2H]
 * (same row stride) with the roundings of the tensor-op form silu(h[:, :H]) * h[:, H:] and its
 * autograd.  The module that holds this activation in the reference's setting is the
 * GroupedExperts of its TorchTitan fork (converted at alto/modifiers/lpt/base.py:186-187).
 * H and ld_h multiples of 8, pointers 16-byte aligned.
 */
int altob200_swiglu_forward(const void* h, int64_t rows, int64_t H, int64_t ld_h, void* out, void* stream);
int altob200_swiglu_backward(const void* h, const void* grad_out, int64_t rows, int64_t H, int64_t ld_h,
                             void* grad_h, void* stream);

/*
 * Block-scaled GEMM on tcgen05:  D[m, n] = alpha * sum_k A[m, k] * B[n, k]
 * with A and B both stored reduction-axis-contiguous ("NT"), packed scales, fp32
 * accumulation in tensor memory.  Replaces blockwise_mxfp4_gemm
 * (alto/kernels/fp4/mxfp4/mxfp_linear.py:143-255), blockwise_mxfp8_gemm
 * (alto/kernels/mxfp8/mxfp8_linear.py:153-296) and the dequantise + bf16 matmul of
 * the NVFP4 path (alto/kernels/fp4/nvfp4/nvfp_linear.py:90,247-248).
 *   a_codes [M, K/2 or K], a_scales packed(rows=M, ncols=K/block)
 *   b_codes [N, K/2 or K], b_scales packed(rows=N, ncols=K/block)
 *   alpha   : device float pointers multiplied together (either may be NULL = 1.0);
 *             NVFP4 passes the two tensorwise outer scales.
 *   d       : [M, N] row-major, out_dtype bf16 or f32, leading dimension ldd.
 * K must be a multiple of the format block; M, N arbitrary (multiples of 8).
 */
int altob200_gemm_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N, int64_t K,
                              const void* a_codes, const void* a_scales, const void* b_codes,
                              const void* b_scales, const float* alpha_a, const float* alpha_b,
                              int32_t out_dtype, void* d, int64_t ldd, void* stream);

/*
 * Grouped (MoE) variant: rows of A are grouped in runs of 128 that share one
 * expert; `group_expert[g]` (device int32, length ceil(M/128), -1 = padding rows that
 * produce zeros) selects B[e] of shape [N, K].  Replaces
 * mxfp4_grouped_gemm_forward / backward_inputs
 * (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_forward.py:201,
 *  alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:399).
 */
int altob200_grouped_gemm_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N,
                                      int64_t K, int32_t num_experts, const void* a_codes,
                                      const void* a_scales, const void* b_codes,
                                      const void* b_scales, const int32_t* group_expert,
                                      const float* alpha_a, const float* alpha_b,
                                      int32_t out_dtype, void* d, int64_t ldd, void* stream);

/*
 * Grouped weight gradient: dW[e][m, n] = alpha * sum over k in [k_offs[e-1], k_offs[e]) of
 * A[m, k] * B[n, k], for e in [0, num_experts) (k_offs[-1] = 0).  A and B are the
 * axis-0 quantised gradient and activation ([N_out, tokens] and [K_in, tokens], token
 * axis contiguous); `k_offs` (device int32, cumulative, every entry a multiple of 128)
 * gives each expert's token range; experts with an empty range receive zeros.  Replaces
 * mxfp4_grouped_gemm_backward_weights (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:501)
 * and the per-expert loop of the NVFP4 path
 * (alto/kernels/fp4/nvfp4/nvfp_grouped_gemm/cg_backward.py:126-141).
 *   d : [num_experts, M, N] row-major, leading dimension ldd (elements).
 * K here is the total number of tokens (the length of the shared reduction axis).
 */
int altob200_grouped_gemm_wgrad_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N, int64_t K,
                                            int32_t num_experts, const void* a_codes, const void* a_scales,
                                            const void* b_codes, const void* b_scales, const int32_t* k_offs,
                                            const float* alpha_a, const float* alpha_b, int32_t out_dtype,
                                            void* d, int64_t ldd, void* stream);

/*
 * Macro-block factors of one MXFP4 operand [rows, K] of the two-level GEMMs below: the uint8 codes
 * altob200_macro_block_scaling wrote (factor = 1 + code / 256 in [1, 2), one per 128 elements of K).
 * The code of (row r, chunk c = k / 128) sits at
 *     codes[(r >> row_shift) * row_stride + c * chunk_stride  (+ expert * expert_stride)]
 * so that every scale tensor of the reference can be passed as it is, without a transposed copy:
 *   blocks along the operand's K axis, one per row   [rows, ceil(K/128)]             -> shift 0, strides (ceil(K/128), 1)
 *   128 x 128 tiles of an operand stored [rows, K]   [ceil(rows/128), ceil(K/128)]   -> shift 7, strides (ceil(K/128), 1)
 *   128 x 128 tiles of the TRANSPOSED operand (W along N for dgrad: rows = in-features,
 *   K = out-features, tiles indexed [out/128, in/128])                               -> shift 7, strides (1, ceil(rows/128))
 * `expert_stride` (B operand of the row-grouped form only) is the distance between two experts' code
 * matrices.
 */
typedef struct altob200_macro_scale {
  const uint8_t* codes;
  int64_t row_stride;
  int64_t chunk_stride;
  int64_t expert_stride;
  int32_t row_shift; /* 0 or 7 */
} altob200_macro_scale;

/*
 * MXFP4 GEMM with two-level ("blockwise" macro-block) scaling on tcgen05:
 *   D[m, n] = out_scale * sum over chunks c of 128 along K of
 *             (sum_{k in c} A[m, k] * B[n, k]) / (fa[m, c] * fb[n, c])
 * Operand layouts as altob200_gemm_blockscaled (format MXFP4 on both sides).  Each chunk is
 * accumulated by the block-scaled MMA in tensor memory and folded into an fp32 result in registers
 * with the reciprocal factors.  Replaces the flow the reference uses where no matrix core takes the
 * macro factors: macro_block_descaling of the de-quantised operands followed by a bf16 matmul
 * (alto/kernels/fp4/mxfp4/mxfp_linear.py:337-356 forward, :496-547 backward;
 * alto/kernels/fp4/mxfp4/macro_block_scaling.py:100-146).  `out_scale` is a host float (1, or 16/9
 * for a weight gradient whose two operands were clipped statically, mxfp_linear.py:543-544).
 * K must be a multiple of 32; a last chunk shorter than 128 takes the factor of its own code.
 */
int altob200_gemm_mxfp4_two_level(int64_t M, int64_t N, int64_t K, const void* a_codes, const void* a_scales,
                                  const altob200_macro_scale* a_macro, const void* b_codes, const void* b_scales,
                                  const altob200_macro_scale* b_macro, float out_scale, int32_t out_dtype, void* d,
                                  int64_t ldd, void* stream);

/*
 * Row-grouped (MoE forward / dgrad) form of the above: `group_expert` as in
 * altob200_grouped_gemm_blockscaled, B and its scales stacked per expert, `b_macro->expert_stride`
 * between the experts' factor codes.  Replaces cg_grouped_gemm_forward / cg_grouped_gemm_backward_inputs
 * on de-scaled operands (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:668-690, 897-901).
 */
int altob200_grouped_gemm_mxfp4_two_level(int64_t M, int64_t N, int64_t K, int32_t num_experts, const void* a_codes,
                                          const void* a_scales, const altob200_macro_scale* a_macro,
                                          const void* b_codes, const void* b_scales,
                                          const altob200_macro_scale* b_macro, const int32_t* group_expert,
                                          float out_scale, int32_t out_dtype, void* d, int64_t ldd, void* stream);

/*
 * Grouped weight gradient with two-level scaling: as altob200_grouped_gemm_wgrad_blockscaled, the
 * shared reduction axis (tokens, length K) cut into per-expert ranges by `k_offs`; chunk c of the
 * factor codes is the absolute 128-token block c of the buffer.  Replaces
 * cg_grouped_gemm_backward_weights on de-scaled operands
 * (alto/kernels/fp4/mxfp4/mxfp_grouped_gemm/cg_backward.py:902-909).
 */
int altob200_grouped_gemm_wgrad_mxfp4_two_level(int64_t M, int64_t N, int64_t K, int32_t num_experts,
                                                const void* a_codes, const void* a_scales,
                                                const altob200_macro_scale* a_macro, const void* b_codes,
                                                const void* b_scales, const altob200_macro_scale* b_macro,
                                                const int32_t* k_offs, float out_scale, int32_t out_dtype, void* d,
                                                int64_t ldd, void* stream);

/*
 * Failure detection of the GEMM kernels.  Every mbarrier wait inside them is bounded by a wall-clock
 * limit (default 4 s); a wait that runs out records {kernel, block, site} in the status word that
 * altob200_status_read returns, and the kernel leaves through its normal teardown.
 * altob200_set_wait_limit_ns changes the limit for later launches of this process.  The reference
 * has no counterpart (its Triton kernels do not wait on one another).
 */
int altob200_set_wait_limit_ns(uint64_t limit_ns);

/*
 * Launches one small kernel whose single wait can never be satisfied (an mbarrier on which nobody
 * arrives) with the given limit (at most 1e9 ns).  Nothing faults and nothing is left running: the
 * wait gives up after `limit_ns`, and the next altob200_status_read on the stream returns
 * ALTOB200_ETIMEOUT_DEVICE with detail {9, 0, 99, 0}, the one after that 0.  For tests of the
 * host-side handling of a device timeout.  No counterpart in the reference.
 */
int altob200_selftest_wait_timeout(uint64_t limit_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ALTOB200_H_ */
