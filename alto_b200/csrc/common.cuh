// Device-side arithmetic shared by the quantizer kernels: scale derivation, E2M1 / FP8
// encode and decode, exact division, packed-scale addressing.
//
// Every function restates arithmetic of the reference so that codes and scales are
// bit-identical to it; the citation next to each function names the reference lines.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/altob200.h"

namespace altob200 {

// ---------------------------------------------------------------------------------------
// host helpers
// ---------------------------------------------------------------------------------------
#define ALTOB200_CUDA_CHECK(expr)                 \
  do {                                            \
    cudaError_t _e = (expr);                      \
    if (_e != cudaSuccess) return ALTOB200_ECUDA; \
  } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel launched through launch_after() may be scheduled while the
// kernel before it in the stream is still draining (its launch latency and the start-up of its CTAs
// then overlap that tail); it must call grid_dependency_wait() before it touches global memory, which
// blocks until the earlier kernel has completed and its writes are visible.  Launched any other way,
// the wait is a no-op.  ALTOB200_PDL=0 in the environment launches everything the plain way.
static inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ALTOB200_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}
template <class... KArgs, class... Args>
static inline cudaError_t launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// bit casts
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }

// bf16 pair (little endian: element 0 in the low half) -> two floats, exact.
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return u2f(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return u2f(w & 0xFFFF0000u); }

// float -> bf16 bits, round to nearest even (what Tensor.to(torch.bfloat16) does).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// ---------------------------------------------------------------------------------------
// packed scale layout (tiles of 128 rows x 4 scale columns, 512 bytes each)
// ---------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int64_t packed_scale_offset(int64_t r, int64_t c,
                                                                int64_t ncol_tiles) {
  const int64_t tile = (r >> 7) * ncol_tiles + (c >> 2);
  return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

// ---------------------------------------------------------------------------------------
// E8M0 scale from a block amax, computed on the BITS of the amax in the input dtype.
//   alto/kernels/fp4/mxfp4/mxfp_quantization.py:79-95  (mbits=1, target_max_pow2=2)
//   alto/kernels/mxfp8/mxfp8_quantization.py:70-78      (e4m3: 3/8, e5m2: 2/15)
// `amax_bits` is the non-negative amax as bf16 bits (IS_BF16) or fp32 bits.
// ---------------------------------------------------------------------------------------
template <bool IS_BF16>
__device__ __forceinline__ uint32_t e8m0_from_amax_bits(uint32_t amax_bits, int mbits,
                                                        int target_max_pow2) {
  int e;
  if (IS_BF16) {
    // int16 arithmetic in the reference: wrap to 16 bits, arithmetic shift.
    const int32_t v = (int32_t)(int16_t)(((amax_bits + (1u << (7 - mbits - 1))) & 0xFF80u));
    e = (v >> 7) - target_max_pow2;
  } else {
    const int32_t v = (int32_t)((amax_bits + (1u << (23 - mbits - 1))) & 0xFF800000u);
    e = (v >> 23) - target_max_pow2;
  }
  e = e < 1 ? 1 : e;
  return (uint32_t)e & 0xFFu;  // .to(uint8)
}

// ---------------------------------------------------------------------------------------
// float -> E4M3 (float8_e4m3fn) round-to-nearest-even for inputs already clamped to
// [2^-6, 448] (all normal in E4M3), returned both as the byte and as the fp32 value.
//   alto/kernels/fp4/nvfp4/nvfp_quantization.py:278-282
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float round_to_e4m3_grid(float x, uint32_t* code) {
  uint32_t b = f2u(x);
  b += 0x7FFFFu + ((b >> 20) & 1u);  // RNE on the 20 dropped mantissa bits
  b &= 0xFFF00000u;
  // E4M3 bias 7: exponent field = e32 - 127 + 7
  const uint32_t e8 = (b >> 23) - 120u;
  *code = (e8 << 3) | ((b >> 20) & 7u);
  return u2f(b);
}

// NVFP4 block scales (inner on the E4M3 grid, quant = inner * outer).
//   alto/kernels/fp4/nvfp4/nvfp_quantization.py:255-289
// `raw` = amax / outer / 6 (or amax / 6), correctly rounded.
__device__ __forceinline__ void nvfp4_block_scale_from_raw(float raw, bool use_outer, float outer,
                                                           float* inner, float* quant, uint32_t* code) {
  raw = fminf(fmaxf(raw, 0.015625f), 448.0f);
  const float in = round_to_e4m3_grid(raw, code);
  *inner = in;
  *quant = use_outer ? __fmul_rn(in, outer) : in;
}
__device__ __forceinline__ void nvfp4_block_scale(float amax, bool use_outer, float outer,
                                                  float* inner, float* quant, uint32_t* code) {
  if (amax != amax) amax = 0.0f;  // NaN amax -> 0
  const float raw = use_outer ? __fdiv_rn(__fdiv_rn(amax, outer), 6.0f) : __fdiv_rn(amax, 6.0f);
  nvfp4_block_scale_from_raw(raw, use_outer, outer, inner, quant, code);
}

// ---------------------------------------------------------------------------------------
// Exact fp32 division x / q.
//
// For a bf16-valued numerator the sequence  y = x*r; e = fma(-y, q, x); y' = fma(e, r, y)
// with r = RN(1/q) returns the correctly rounded quotient (checked exhaustively over all
// 2^7 numerator and 2^23 denominator mantissas); it needs q and the quotient to stay away
// from the subnormal range, which callers guarantee by testing q once per block
// (`div_fast_ok`).  The sign of x is copied so that -0.0 keeps its sign bit as IEEE
// division does (the reference ORs that sign into the code, triton_fp4_ops.py:40-41,90-92).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ bool div_fast_ok(float q) {
  const uint32_t e = (f2u(q) >> 23) & 0xFFu;
  return e >= 67u && e <= 187u;  // 2^-60 <= q < 2^61
}
__device__ __forceinline__ float div_bf16_num(float x, float q, float r) {
  const float y = __fmul_rn(x, r);
  const float e = __fmaf_rn(-y, q, x);
  const float y2 = __fmaf_rn(e, r, y);
  return u2f((f2u(y2) & 0x7FFFFFFFu) | (f2u(x) & 0x80000000u));
}
// The same quotient up to the sign of a zero (for callers that take the sign from x).
__device__ __forceinline__ float div_bf16_num_mag(float x, float q, float r) {
  const float y = __fmul_rn(x, r);
  const float e = __fmaf_rn(-y, q, x);
  return __fmaf_rn(e, r, y);
}

// x / 6 for a normal x whose quotient and residual stay normal (callers keep |x| in [2^-91, 2^120) or
// zero): y = x * r, e = fma(-y, 6, x), y' = fma(e, r, y) with r = RN(1/6) is the correctly rounded
// quotient for every one of the 2^23 mantissas of x (checked exhaustively in integer arithmetic).
__device__ __forceinline__ float div_by_6(float x) {
  const float r = 0.16666667163372040f;
  const float y = __fmul_rn(x, r);
  const float e = __fmaf_rn(-y, 6.0f, x);
  return __fmaf_rn(e, r, y);
}

// ---------------------------------------------------------------------------------------
// E2M1 encode, round to nearest even, saturating:
//   alto/kernels/fp4/fp4_common/triton_fp4_ops.py:26-93 with USE_SR=False.
// Two floats -> one byte of E2M1 codes (v0 in the low nibble) with the hardware converter, which
// computes what the reference's bit arithmetic computes for every finite input: round to nearest
// even on the E2M1 grid including its subnormal 0.5, saturation to 6, sign of zero kept (checked
// against the oracle on the golden vectors and on random data in the GPU tests).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e2m1x2_rtn_hw(float v0, float v1) {
  uint16_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }"
      : "=h"(r)
      : "f"(v1), "f"(v0));
  return (uint32_t)r;
}

// ---------------------------------------------------------------------------------------
// E2M1 encode with stochastic rounding from 32 random bits.  Restatement of
//   alto/kernels/fp4/fp4_common/triton_fp4_ops.py:26-93 with USE_SR=True.
// ---------------------------------------------------------------------------------------
// Arranged for instruction count (the stochastic-rounding quantizers are bound by instruction
// issue, not by memory).  The reference rounds the normal range [1, 6) by adding 22 random bits
// below the kept mantissa bit and truncating; in the E2M1-subnormal range [0, 1), with 2a = k + frac,
// it compares the random word with uint32(a * fp32(2^33 - 2)) for a < 0.5 and with
// uint32((2a - 1) * fp32(2^32 - 1)) otherwise; both constants round to powers of two in fp32, so
// both thresholds are trunc(frac * 2^32) and the code is k + [rnd <= threshold].
// `v` is the scaled value up to the sign of a zero; the sign
// bit of the code is taken from `sign_bits` (the bits of the unscaled element: scales are positive).
// With a = min(|v|, 6):
//   normal range   code = (bits(a) + (rnd & (2^22 - 1)) - (126 << 23)) >> 22: the carry out of the low
//                  22 mantissa bits rounds up, and 6.0 itself maps to 7, so saturation needs no
//                  separate test;
//   a < 1          with T = trunc(a * 2^33) = k * 2^32 + threshold (k = [a >= 0.5]),
//                  code = hi32(T + 1 + ~rnd) = k + [rnd <= threshold].
// A NaN saturates to 7 (the reference's code for a NaN element is an accident of its payload).
// COMPARE selects how the sub-one threshold is evaluated (same value): the 64-bit carry form above, or
// T.hi + [T.lo >= rnd]; the row-wise kernel is faster with the compare, the column-wise one with the carry.
template <bool COMPARE = false>
__device__ __forceinline__ uint32_t e2m1_sr_code(float v, uint32_t sign_bits, uint32_t rnd) {
  const float a = fminf(fabsf(v), 6.0f);
  const uint32_t ab = f2u(a);
  const uint32_t cn = (ab + (rnd & 0x3FFFFFu) - (126u << 23)) >> 22;
  const uint64_t t = __float2ull_rz(__fmul_rn(a, 8589934592.0f));
  // hi32(T + 1 + ~rnd) = hi32(T + 2^32 - rnd) = T.hi + [T.lo >= rnd]
  const uint32_t cd = COMPARE ? (uint32_t)(t >> 32) + ((uint32_t)t >= rnd ? 1u : 0u)
                              : (uint32_t)((t + 1ull + (uint64_t)(~rnd)) >> 32);
  const uint32_t mag = a < 1.0f ? cd : cn;
  // sign into bit 3 with one shift and one multiply-add (disjoint bits): the ALU pipe is the busy one
  uint32_t r;
  asm("mad.lo.u32 %0, %1, 8, %2;" : "=r"(r) : "r"(sign_bits >> 31), "r"(mag));
  return r;
}

// E2M1 decode to fp32 (alto/kernels/fp4/fp4_common/triton_fp4_ops.py:100-132).
__device__ __forceinline__ float e2m1_decode(uint32_t c) {
  const uint32_t s = (c & 8u) << 28;
  const uint32_t m = c & 7u;
  uint32_t bits;
  if (m == 0u) bits = 0u;
  else if (m == 1u) bits = 0x3F000000u;
  else bits = (((m >> 1) - 1u + 127u) << 23) | ((m & 1u) << 22);
  return u2f(bits | s);
}

// ---------------------------------------------------------------------------------------
// FP8 encode: saturating round-to-nearest-even (the emulation clamps to +-max and then
// casts, tests/unittest/mxfp8/utils.py:126-132; the Triton cast saturates natively,
// alto/kernels/mxfp8/mxfp8_quantization.py:263-281).  v0 goes to the low byte.
// ---------------------------------------------------------------------------------------
template <bool E5M2>
__device__ __forceinline__ uint32_t fp8x2_rtn_hw(float v0, float v1) {
  uint16_t r;
  if (E5M2) {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(v1), "f"(v0));
  } else {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(v1), "f"(v0));
  }
  return (uint32_t)r;
}

// Two FP8 bytes (low byte first) -> two floats; exact (both formats embed in fp16).
template <bool E5M2>
__device__ __forceinline__ float2 fp8x2_decode(uint32_t c) {
  uint32_t h2;
  const uint16_t c16 = (uint16_t)c;
  if (E5M2) {
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(c16));
  } else {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c16));
  }
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  return __half22float2(h);
}

// ---------------------------------------------------------------------------------------
// Philox-4x32-10 with the counter/key convention of triton.language.randint4x(seed, offset):
// counter = (offset_lo, offset_hi, 0, 0), key = (seed_lo, seed_hi); each of the ten rounds is
//   c0' = hi(B * c2) ^ c1 ^ k0,  c2' = hi(A * c0) ^ c3 ^ k1,  c1' = lo(B * c2),  c3' = lo(A * c0)
// with A = 0xD2511F53, B = 0xCD9E8D57 and the key advanced by (0x9E3779B9, 0xBB67AE85) per round.
// The ten round keys are precomputed on the host (they depend on the seed only), so that each round
// is two wide multiplies and two three-input XORs.
// ---------------------------------------------------------------------------------------
struct PhiloxKeys {
  uint32_t k[20];  // k[2i], k[2i+1]: key of round i
};
static inline void philox_make_keys(uint64_t seed, PhiloxKeys* pk) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int i = 0; i < 10; ++i) {
    pk->k[2 * i] = k0;
    pk->k[2 * i + 1] = k1;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}
__device__ __forceinline__ void philox4x32_10_keys(uint32_t c0, uint32_t c1, const PhiloxKeys& pk, uint32_t out[4]) {
  const uint32_t A = 0xD2511F53u, B = 0xCD9E8D57u;
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint64_t pb = (uint64_t)B * c2, pa = (uint64_t)A * c0;
    c0 = (uint32_t)(pb >> 32) ^ c1 ^ pk.k[2 * i];
    c2 = (uint32_t)(pa >> 32) ^ c3 ^ pk.k[2 * i + 1];
    c1 = (uint32_t)pb;
    c3 = (uint32_t)pa;
  }
  out[0] = c0;
  out[1] = c1;
  out[2] = c2;
  out[3] = c3;
}

}  // namespace altob200
