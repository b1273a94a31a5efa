// Bandwidth kernels of the low-precision linear path: block quantizers (row-wise,
// column-wise with the optional randomised Hadamard transform, 2D with dual packing),
// tensor amax, dequantizers and the standalone Hadamard transform.
//
// Work layout (every global access is a full 32-byte sector or better, and every thread keeps one
// quantisation block or a fixed part of it in registers; the counters show all of these kernels
// bound by instruction issue rather than by HBM):
//   row-wise  : a warp task is 4 rows x 512 contiguous elements, a lane 16 elements of each row
//               (two 128-bit loads per row for bf16, all issued first).  NVFP4 blocks (16) live in
//               one lane, MX blocks (32) in a lane pair.
//   col-wise  : a CTA owns a 128-row x 64-column tile; a lane owns two adjacent columns of one
//               block of rows, so the Hadamard butterfly and the block amax need no shuffles.
//               Codes are transposed through shared memory so that every output row receives 64
//               (FP4) or 128 (FP8) contiguous bytes.
//   2D        : a warp owns 4 block columns x 64 (or 32) rows, a thread 16 rows x 8 columns in
//               registers; block maxima by shuffles, the second packing by an in-register
//               transpose; no shared memory.
#include <type_traits>

#include <atomic>

#include "common.cuh"

namespace altob200 {

// ---------------------------------------------------------------------------------------
// format traits
// ---------------------------------------------------------------------------------------
template <int FMT>
struct Fmt;
template <>
struct Fmt<ALTOB200_FMT_NVFP4> {
  static constexpr int B = 16;
  static constexpr bool FP4 = true, MX = false, E5M2 = false;
  static constexpr int MBITS = 0, TMAX = 0;
};
template <>
struct Fmt<ALTOB200_FMT_MXFP4> {
  static constexpr int B = 32;
  static constexpr bool FP4 = true, MX = true, E5M2 = false;
  static constexpr int MBITS = 1, TMAX = 2;
};
template <>
struct Fmt<ALTOB200_FMT_MXFP8_E4M3> {
  static constexpr int B = 32;
  static constexpr bool FP4 = false, MX = true, E5M2 = false;
  static constexpr int MBITS = 3, TMAX = 8;
};
template <>
struct Fmt<ALTOB200_FMT_MXFP8_E5M2> {
  static constexpr int B = 32;
  static constexpr bool FP4 = false, MX = true, E5M2 = true;
  static constexpr int MBITS = 2, TMAX = 15;
};

// Scale of one quantisation block, in the forms the element loop needs.
struct BlockScale {
  float q;        // divisor applied to the elements
  float r;        // reciprocal used by the fast paths
  bool fast;      // fast path valid
  uint32_t byte;  // stored scale byte (E8M0 exponent or E4M3 code)
  float plain;    // NVFP4: inner scale as fp32 (plain layout)
};

// The tensor-wide outer scale of NVFP4 in the forms the block-scale arithmetic needs (per thread, once).
struct OuterScale {
  bool use;    // an outer scale is applied
  float v;     // its value (1 when unused)
  float r;     // RN(1 / v)
  bool fast;   // v allows the reciprocal form of amax / v
};
__device__ __forceinline__ OuterScale make_outer_scale(bool use, const float* p) {
  OuterScale o;
  o.use = use;
  o.v = use ? __ldg(p) : 1.0f;
  o.r = __frcp_rn(o.v);
  o.fast = div_fast_ok(o.v);
  return o;
}

// amax_abs_bits: max over the block of (bits & 0x7FFF..) in the input dtype's bit width
// (bf16 bits or fp32 bits); integer max propagates NaN like torch.amax does.
template <int FMT, bool IN_BF16>
__device__ __forceinline__ BlockScale make_block_scale(uint32_t amax_abs_bits, const OuterScale& os) {
  using F = Fmt<FMT>;
  BlockScale s;
  if (F::MX) {
    const uint32_t e = e8m0_from_amax_bits<IN_BF16>(amax_abs_bits, F::MBITS, F::TMAX);
    s.byte = e;
    s.q = u2f(e << 23);
    s.fast = e <= 253u;
    s.r = u2f((254u - e) << 23);
    s.plain = 0.0f;
  } else {
    const float amax = IN_BF16 ? u2f(amax_abs_bits << 16) : u2f(amax_abs_bits);
    // bf16 amax of 0 or in [2^-30, 2^60): amax / outer / 6 by reciprocals with one correction step each
    // (exact, see div_bf16_num and div_by_6); everything else divides
    const uint32_t e8 = amax_abs_bits >> 7;
    if (IN_BF16 && (amax_abs_bits == 0u || (e8 >= 97u && e8 < 187u)) && (!os.use || os.fast)) {
      const float t = os.use ? div_bf16_num_mag(amax, os.v, os.r) : amax;
      nvfp4_block_scale_from_raw(div_by_6(t), os.use, os.v, &s.plain, &s.q, &s.byte);
    } else {
      nvfp4_block_scale(amax, os.use, os.v, &s.plain, &s.q, &s.byte);
    }
    s.fast = IN_BF16 && div_fast_ok(s.q);
    s.r = __frcp_rn(s.q);
  }
  return s;
}

// ---------------------------------------------------------------------------------------
// Options of the MXFP4 quantizer (alto/kernels/fp4/mxfp4/mxfp_quantization.py:29-95, 321-322;
// arithmetic as in the reference's emulation, tests/unittest/mxfp4/utils.py:320-358, which works
// in the input dtype: with bf16 inputs every intermediate is rounded to bf16).
//   clip 1 (static) : elements are multiplied by 3/4 before encoding; the scale is unchanged
//   clip 2 (dynamic): the scale is taken from 2.92247856/6 * std(block) + 1e-8 instead of the amax,
//                     with target exponent 0 instead of 2
//   uos             : scale = ceil(log2(amax / 7.25)) + 127 (128 for an all-zero block)
// ---------------------------------------------------------------------------------------
struct MxOpts {
  int clip;
  int uos;
};

template <bool IN_BF16>
__device__ __forceinline__ float round_in(float v) {
  return IN_BF16 ? u2f(f32_to_bf16_bits(v) << 16) : v;
}

// E8M0 byte of an MX block from its statistics.  `amax_abs_bits` as in make_block_scale; `sum` and
// `sumsq` (of the squares rounded to the input dtype) over the n elements are used by clip 2 only.
template <int FMT, bool IN_BF16>
__device__ __forceinline__ BlockScale make_block_scale_opts(uint32_t amax_abs_bits, float sum, float sumsq, int n,
                                                            MxOpts o) {
  using F = Fmt<FMT>;
  float max_abs = IN_BF16 ? u2f(amax_abs_bits << 16) : u2f(amax_abs_bits);
  int tmax = F::TMAX;
  if (o.clip == 2) {
    const float inv_n = 1.0f / (float)n;
    const float mean_sq = round_in<IN_BF16>(__fmul_rn(sumsq, inv_n));
    const float mean = round_in<IN_BF16>(__fmul_rn(sum, inv_n));
    const float var = round_in<IN_BF16>(__fsub_rn(mean_sq, round_in<IN_BF16>(__fmul_rn(mean, mean))));
    const float sd = round_in<IN_BF16>(__fsqrt_rn(var));
    max_abs = round_in<IN_BF16>(__fadd_rn(round_in<IN_BF16>(__fmul_rn(sd, (float)(2.92247856 / 6.0))), 1e-8f));
    tmax = 0;
  }
  uint32_t e;
  if (o.uos) {
    const float r = round_in<IN_BF16>(__fdiv_rn(max_abs, 7.25f));
    float s = ceilf(round_in<IN_BF16>(log2f(r)));
    if (max_abs == 0.0f) s = 1.0f;
    s += 127.0f;
    // NaN compares false everywhere and converts to 0, which the clamp turns into 1
    e = s < 1.0f ? 1u : (s > 255.0f ? 255u : (uint32_t)s);
    if (!(s == s)) e = 1u;
  } else {
    const uint32_t bits = IN_BF16 ? (f2u(max_abs) >> 16) : f2u(max_abs);
    e = e8m0_from_amax_bits<IN_BF16>(bits, F::MBITS, tmax);
  }
  BlockScale s;
  s.byte = e;
  s.q = u2f(e << 23);
  s.fast = e <= 253u;
  s.r = u2f((254u - e) << 23);
  s.plain = 0.0f;
  return s;
}

// One element divided by its block scale.  FAST is decided once per warp (every lane's block scale
// allows the reciprocal forms), so that the element loops carry no per-element branch; the other
// variant divides.  Both give the correctly rounded quotient.
template <int FMT, bool IN_BF16, bool FAST>
__device__ __forceinline__ float scale_elem(float x, const BlockScale& s) {
  if (!FAST) return __fdiv_rn(x, s.q);
  if (Fmt<FMT>::MX) return __fmul_rn(x, s.r);
  return div_bf16_num(x, s.q, s.r);
}

// acc | (x << sh) for disjoint bits, as one integer multiply-add.
__device__ __forceinline__ uint32_t merge_shifted(uint32_t x, int sh, uint32_t acc) {
  uint32_t r;
  asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(1u << sh), "r"(acc));
  return r;
}

// The scaled element up to the sign of a zero (the stochastic-rounding encoder takes the sign from x).
template <int FMT, bool IN_BF16, bool FAST>
__device__ __forceinline__ float scale_elem_mag(float x, const BlockScale& s) {
  if (!FAST) return __fdiv_rn(x, s.q);
  if (Fmt<FMT>::MX) return __fmul_rn(x, s.r);
  return div_bf16_num_mag(x, s.q, s.r);
}

// Two elements of two different blocks divided by their block scales at once (reciprocal forms only;
// magnitudes up to the sign of a zero, as scale_elem_mag): x * r for the power-of-two scales of the MX
// formats, else y = x r, e = fma(y, -q, x), y + e r - the three roundings of div_bf16_num_mag per element.
template <int FMT>
__device__ __forceinline__ float2 scale_pair_mag(float2 x, const BlockScale& s0, const BlockScale& s1) {
  const float2 r = make_float2(s0.r, s1.r);
  const float2 y = __fmul2_rn(x, r);
  if (Fmt<FMT>::MX) return y;
  const float2 e = __ffma2_rn(y, make_float2(-s0.q, -s1.q), x);
  return __ffma2_rn(e, r, y);
}

// Scale and quantise 2 elements into one FP4 byte (x0 in the low nibble).
template <int FMT, bool IN_BF16, int ROUND, bool FAST>
__device__ __forceinline__ uint32_t fp4_pair(float x0, float x1, const BlockScale& s, uint32_t r0, uint32_t r1) {
  if (ROUND == ALTOB200_ROUND_RTN)
    return e2m1x2_rtn_hw(scale_elem<FMT, IN_BF16, FAST>(x0, s), scale_elem<FMT, IN_BF16, FAST>(x1, s));
  // codes are merged with multiply-adds (disjoint bits: adding is or-ing): the integer ALU is the
  // busiest pipe of these kernels and the multiply-add pipe has room
  const uint32_t c0 = e2m1_sr_code<true>(scale_elem_mag<FMT, IN_BF16, FAST>(x0, s), f2u(x0), r0);
  const uint32_t c1 = e2m1_sr_code<true>(scale_elem_mag<FMT, IN_BF16, FAST>(x1, s), f2u(x1), r1);
  return merge_shifted(c1, 4, c0);
}

// Runs body(std::true_type) when every lane of the warp may use the reciprocal forms, else
// body(std::false_type); must be reached by the whole warp.
template <class Body>
__device__ __forceinline__ void with_uniform_fast(bool lane_fast, Body body) {
  if (__all_sync(0xFFFFFFFFu, lane_fast)) body(std::true_type{});
  else body(std::false_type{});
}

// Quotient and remainder with a 32-bit divide whenever the operands fit (a 64-bit divide costs
// several dozen instructions per task).
__device__ __forceinline__ void divmod_fast(int64_t t, int64_t d, int64_t* q, int64_t* r) {
  if ((((uint64_t)t | (uint64_t)d) >> 32) == 0) {
    const uint32_t qq = (uint32_t)t / (uint32_t)d;
    *q = qq;
    *r = (uint32_t)t - qq * (uint32_t)d;
  } else {
    *q = t / d;
    *r = t - *q * d;
  }
}

__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t w) {
  return __vmaxu2(acc, w & 0x7FFF7FFFu);
}
__device__ __forceinline__ uint32_t fold_bf16x2(uint32_t acc) {
  const uint32_t lo = acc & 0xFFFFu, hi = acc >> 16;
  return lo > hi ? lo : hi;
}

// =======================================================================================
// Row-wise quantizer
// =======================================================================================
struct RowwiseArgs {
  const void* x;
  int64_t rows, cols, ld;
  uint8_t* codes;
  void* scale_plain;
  uint8_t* scale_packed;
  int64_t ncol_tiles;  // ceil(cols / B / 4)
  const float* outer;
  const uint32_t* rand_bits;
  // rand_bits as a periodic tile [2][tile_rows][tile_pairs] (0 = full planes [2][rows][cols/2])
  int64_t tile_rows, tile_pairs;
  uint64_t philox_seed, philox_offset;
  PhiloxKeys pk;
  MxOpts mx;
};

// A warp task is 4 consecutive rows x 512 contiguous columns (a lane: 16 columns of each row).  The
// loads of all four rows are issued before the first is consumed (128 bytes per lane in flight), and
// the index arithmetic of a task (row and chunk, pointers, position in the periodic random table) is
// paid once per 64 elements of a lane.
// Three resident blocks per SM (at most 85 registers per thread) measured fastest: fewer registers
// spill, more leave too few warps to cover the issue slots.
constexpr int ROW_R = 4;

template <int FMT, bool IN_BF16, int ROUND>
__global__ void __launch_bounds__(256, 3) quantize_rowwise_kernel(RowwiseArgs a) {
  grid_dependency_wait();
  using F = Fmt<FMT>;
  constexpr int LPB = F::B / 16;  // lanes per block
  constexpr int ESZ = IN_BF16 ? 2 : 4;
  constexpr int NV = IN_BF16 ? 2 : 4;  // 16-byte vectors per lane and row
  const int lane = threadIdx.x & 31;
  const int64_t chunks_per_row = (a.cols + 511) >> 9;
  const int64_t n_tasks = ((a.rows + ROW_R - 1) / ROW_R) * chunks_per_row;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const OuterScale os = make_outer_scale((!F::MX) && a.outer != nullptr, a.outer);
  const int64_t half_cols = a.cols >> 1;
  const int64_t nkb = a.cols / F::B;
  const bool tiled = a.tile_rows != 0;
  const uint32_t t_rows = (uint32_t)a.tile_rows, t_pairs = (uint32_t)a.tile_pairs;

  for (int64_t task = warp0; task < n_tasks; task += n_warps) {
    int64_t rg, chunk;
    divmod_fast(task, chunks_per_row, &rg, &chunk);
    const int64_t row0 = rg * ROW_R;
    const int64_t col = (chunk << 9) + lane * 16;
    const bool col_ok = col < a.cols;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.x) + (row0 * a.ld + col) * ESZ;
    const int64_t pitch = a.ld * ESZ;

    // ---- all loads of the task ----
    uint4 raw[ROW_R][NV];
#pragma unroll
    for (int i = 0; i < ROW_R; ++i) {
      const bool ok = col_ok && row0 + i < a.rows;
#pragma unroll
      for (int q = 0; q < NV; ++q)
        raw[i][q] = ok ? __ldg(reinterpret_cast<const uint4*>(src + i * pitch) + q) : make_uint4(0u, 0u, 0u, 0u);
    }
    // position of the task in the periodic random table (32-bit: the host refuses larger extents)
    uint32_t rr0 = 0, pp = 0;
    if (ROUND == ALTOB200_ROUND_SR_BITS && tiled) {
      rr0 = (uint32_t)row0 % t_rows;
      pp = (uint32_t)(col >> 1) % t_pairs;
    }
    const int64_t kb = (chunk << 9) / F::B + lane / LPB;  // scale column of this lane
    const bool holder = col_ok && (lane % LPB == 0);

#pragma unroll
    for (int i = 0; i < ROW_R; ++i) {
      const int64_t row = row0 + i;
      const bool active = col_ok && row < a.rows;
      // random words first: their (cache-resident) loads overlap the scale arithmetic below
      uint32_t r0[8], r1[8];
      if (ROUND == ALTOB200_ROUND_SR_BITS) {
        // full planes [2][rows][cols/2], or a [2][tile_rows][tile_pairs] table repeated over the matrix
        // (the 8 pairs of a lane never straddle a tile: tile_pairs is a multiple of 8)
        uint32_t rr = rr0 + (uint32_t)i;
        while (tiled && rr >= t_rows) rr -= t_rows;
        const int64_t off = tiled ? (int64_t)(rr * t_pairs + pp) : row * half_cols + (col >> 1);
        const int64_t plane = tiled ? (int64_t)(t_rows * t_pairs) : a.rows * half_cols;
        uint4 a0 = make_uint4(0u, 0u, 0u, 0u), a1 = a0, b0 = a0, b1 = a0;
        if (active) {
          const uint4* p0 = reinterpret_cast<const uint4*>(a.rand_bits + off);
          const uint4* p1 = reinterpret_cast<const uint4*>(a.rand_bits + plane + off);
          a0 = __ldg(p0); a1 = __ldg(p0 + 1); b0 = __ldg(p1); b1 = __ldg(p1 + 1);
        }
        r0[0] = a0.x; r0[1] = a0.y; r0[2] = a0.z; r0[3] = a0.w;
        r0[4] = a1.x; r0[5] = a1.y; r0[6] = a1.z; r0[7] = a1.w;
        r1[0] = b0.x; r1[1] = b0.y; r1[2] = b0.z; r1[3] = b0.w;
        r1[4] = b1.x; r1[5] = b1.y; r1[6] = b1.z; r1[7] = b1.w;
      } else if (ROUND == ALTOB200_ROUND_SR_PHILOX) {
        // one Philox call feeds two element pairs: call index = pair index / 2
        const uint64_t q0 = a.philox_offset + (uint64_t)((row * half_cols + (col >> 1)) >> 1);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[4];
          const uint64_t ctr = q0 + c;
          philox4x32_10_keys((uint32_t)ctr, (uint32_t)(ctr >> 32), a.pk, o);
          r0[2 * c] = o[0]; r1[2 * c] = o[1]; r0[2 * c + 1] = o[2]; r1[2 * c + 1] = o[3];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) r0[j] = r1[j] = 0;
      }

      // ---- unpack, block maximum ----
      float v[16];
      uint32_t amax_bits = 0;
      if (IN_BF16) {
        const uint32_t w[8] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w,
                               raw[i][1].x, raw[i][1].y, raw[i][1].z, raw[i][1].w};
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc = absmax_bf16x2(acc, w[j]);
          v[2 * j] = bf16lo_to_f32(w[j]);
          v[2 * j + 1] = bf16hi_to_f32(w[j]);
        }
        amax_bits = fold_bf16x2(acc);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          v[4 * q] = u2f(raw[i][q % NV].x); v[4 * q + 1] = u2f(raw[i][q % NV].y);
          v[4 * q + 2] = u2f(raw[i][q % NV].z); v[4 * q + 3] = u2f(raw[i][q % NV].w);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t b = f2u(v[j]) & 0x7FFFFFFFu;
          amax_bits = b > amax_bits ? b : amax_bits;
        }
      }
      if (LPB == 2) {
        const uint32_t o = __shfl_xor_sync(0xFFFFFFFFu, amax_bits, 1);
        amax_bits = o > amax_bits ? o : amax_bits;
      }
      BlockScale s;
      if (F::MX && (a.mx.clip | a.mx.uos)) {
        float sum = 0.0f, sumsq = 0.0f;
        if (a.mx.clip == 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            sum = __fadd_rn(sum, v[j]);
            sumsq = __fadd_rn(sumsq, round_in<IN_BF16>(__fmul_rn(v[j], v[j])));
          }
          if (LPB == 2) {
            sum = __fadd_rn(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, 1));
            sumsq = __fadd_rn(sumsq, __shfl_xor_sync(0xFFFFFFFFu, sumsq, 1));
          }
        }
        s = make_block_scale_opts<FMT, IN_BF16>(amax_bits, sum, sumsq, F::B, a.mx);
        if (a.mx.clip == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = round_in<IN_BF16>(__fmul_rn(v[j], 0.75f));
        }
      } else {
        s = make_block_scale<FMT, IN_BF16>(amax_bits, os);
      }

      // ---- encode and store ----
      with_uniform_fast(s.fast, [&](auto fast_tag) {
        constexpr bool FAST = decltype(fast_tag)::value;
        if (F::FP4) {
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            lo = merge_shifted(fp4_pair<FMT, IN_BF16, ROUND, FAST>(v[2 * j], v[2 * j + 1], s, r0[j], r1[j]), 8 * j, lo);
            hi = merge_shifted(fp4_pair<FMT, IN_BF16, ROUND, FAST>(v[8 + 2 * j], v[9 + 2 * j], s, r0[4 + j], r1[4 + j]),
                               8 * j, hi);
          }
          if (active) *reinterpret_cast<uint2*>(a.codes + row * half_cols + (col >> 1)) = make_uint2(lo, hi);
        } else {
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float q[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) q[c] = scale_elem<FMT, IN_BF16, FAST>(v[4 * j + c], s);
            o[j] = fp8x2_rtn_hw<F::E5M2>(q[0], q[1]) | (fp8x2_rtn_hw<F::E5M2>(q[2], q[3]) << 16);
          }
          if (active) *reinterpret_cast<uint4*>(a.codes + row * a.cols + col) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      });

      // ---- scales ----
      if (a.scale_plain != nullptr && holder && row < a.rows) {
        if (F::MX) reinterpret_cast<uint8_t*>(a.scale_plain)[row * nkb + kb] = (uint8_t)s.byte;
        else reinterpret_cast<float*>(a.scale_plain)[row * nkb + kb] = s.plain;
      }
      if (a.scale_packed != nullptr) {
        uint32_t word = (holder && row < a.rows) ? s.byte : 0u;
        word |= __shfl_down_sync(0xFFFFFFFFu, word, LPB) << 8;
        word |= __shfl_down_sync(0xFFFFFFFFu, word, 2 * LPB) << 16;
        if ((lane % (4 * LPB) == 0) && (kb < a.ncol_tiles * 4) && row < a.rows)
          *reinterpret_cast<uint32_t*>(a.scale_packed + packed_scale_offset(row, kb, a.ncol_tiles)) = word;
      }
    }
  }
}

// =======================================================================================
// Hadamard helpers (n = 16, Sylvester ordering, in registers)
// =======================================================================================
struct RhtParams {
  int n;           // 0 or 16
  int8_t pinv[16]; // slot k reads row pinv[k] of the block
  int8_t perm[16]; // output position i takes slot perm[i]
  float sign[16];  // sign applied to slot k after the butterfly
  int64_t row_off[16];  // byte offset of row pinv[k] from the first row of a 16-row group (column passes)
  float qsign[16];      // sign[k] / sqrt(16): the factor applied to slot k
  int perm_off[16];     // pinv[k] * 8: byte offset of slot k's row in the shared-memory position table, per thread of the CTA
};

__device__ __forceinline__ void hadamard16(float* z) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float a = z[i], b = z[i + h];
        z[i] = __fadd_rn(a, b);
        z[i + h] = __fsub_rn(a, b);
      }
    }
  }
}

// The same butterfly on the two columns of a lane at once, as packed fp32 operations (one instruction
// per pair of sums): a - b is fma(b, -1, a), which rounds once like the subtraction.
__device__ __forceinline__ void hadamard16_pair(float* za, float* zb) {
  float2 z[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) z[i] = make_float2(za[i], zb[i]);
  const float2 neg = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float2 a = z[i], b = z[i + h];
        z[i] = __fadd2_rn(a, b);
        z[i + h] = __ffma2_rn(b, neg, a);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    za[i] = z[i].x;
    zb[i] = z[i].y;
  }
}

// =======================================================================================
// Column-wise quantizer (axis 0) with optional Hadamard transform
// =======================================================================================
struct ColwiseArgs {
  const void* x;
  int64_t rows, cols, ld;
  uint8_t* codes;       // [cols, rows/2] or [cols, rows]
  void* scale_plain;    // [cols, rows/B]
  uint8_t* scale_packed;
  int64_t ncol_tiles;   // ceil(rows / B / 4)
  const float* outer;
  const uint32_t* rand_bits;  // [2][cols][rows/2], or a periodic tile [2][tile_rows][tile_pairs]
  int64_t tile_rows, tile_pairs;
  uint64_t philox_seed, philox_offset;
  PhiloxKeys pk;
  RhtParams rht;
  MxOpts mx;
};

// Threads per CTA = rows per CTA tile.  128 rather than 256: more, smaller CTAs per SM (four of the
// 128-register stochastic-rounding variant instead of two), so that the start-up loads and the
// barrier of one overlap the arithmetic of the others (measured 5-6 % on the bench's launches).
constexpr int COL_NT = 128;
constexpr int COL_TN = 64;   // columns per CTA tile

template <int FMT, bool IN_BF16, int ROUND, bool RHT>
__global__ void __launch_bounds__(COL_NT) quantize_colwise_kernel(ColwiseArgs a) {
  grid_dependency_wait();
  using F = Fmt<FMT>;
  constexpr int B = F::B;
  constexpr int NT = COL_NT;   // threads per CTA
  constexpr int COL_TM = NT;               // rows per CTA tile
  constexpr int NBLK = COL_TM / B;          // row blocks per tile (16 or 8)
  constexpr int ITERS = NBLK / (NT / 32);   // per warp
  constexpr int ROW_BYTES = F::FP4 ? COL_TM / 2 : COL_TM;  // bytes per output row per tile
  constexpr int BLK_BYTES = F::FP4 ? B / 2 : B;            // bytes per block per column
  // codes staged as [block][column][BLK_BYTES]; scales as [column][NBLK]
  __shared__ __align__(16) uint8_t s_codes[COL_TN * ROW_BYTES];
  __shared__ __align__(16) uint8_t s_sf[COL_TN * NBLK];
  __shared__ float s_sf_plain[Fmt<FMT>::MX ? 1 : COL_TN * NBLK];
  __shared__ float2 s_perm[(RHT && ROUND != ALTOB200_ROUND_RTN) ? 16 : 1][NT];   // (column c, column c + 1) per thread

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.y * COL_TM;
  const int64_t n0 = (int64_t)blockIdx.x * COL_TN;
  const int64_t c = n0 + 2 * lane;  // first of this lane's two columns
  const bool col_ok = c < a.cols;   // cols is even, so c+1 is valid too
  const OuterScale os = make_outer_scale((!F::MX) && a.outer != nullptr, a.outer);
  const int64_t half_rows = a.rows >> 1;
  // rows of the periodic random table for this lane's two columns (rows of the axis-last view)
  // (32-bit arithmetic: with a periodic table the host refuses extents of 2^32 and more; a 64-bit
  // modulo is ~70 instructions, several per thread of a CTA that handles 64 elements per thread)
  const uint32_t tile_row0 = a.tile_rows != 0 ? (uint32_t)c % (uint32_t)a.tile_rows : 0u;
  const uint32_t tile_row1 = a.tile_rows != 0 ? (tile_row0 + 1u == (uint32_t)a.tile_rows ? 0u : tile_row0 + 1u) : 0u;

  // bf16: the words of every iteration are requested before the first is used (slot k <- row pinv[k]
  // when the transform is on; the identity otherwise), so the second block's loads fly under the
  // first block's arithmetic
  constexpr int ESZ = IN_BF16 ? 2 : 4;
  const int64_t half_blk = 16 * a.ld * ESZ;  // second 16-row group of a 32-row block
  uint32_t pre[IN_BF16 ? ITERS : 1][IN_BF16 ? B : 1];
  if (IN_BF16) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int64_t mb = m0 + (int64_t)(warp * ITERS + it) * B;
      const bool ok = col_ok && mb < a.rows;
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.x) + (mb * a.ld + c) * ESZ;
#pragma unroll
      for (int k = 0; k < B; ++k)
        pre[it % (IN_BF16 ? ITERS : 1)][k % (IN_BF16 ? B : 1)] =
            ok ? __ldg(reinterpret_cast<const uint32_t*>(base + a.rht.row_off[k & 15] + (k >= 16 ? half_blk : 0))) : 0u;
    }
  }

#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int blk = warp * ITERS + it;
    const int64_t mb = m0 + (int64_t)blk * B;
    const bool ok = col_ok && mb < a.rows;  // rows % B == 0
    float v0[B], v1[B];
    if (IN_BF16) {
#pragma unroll
      for (int k = 0; k < B; ++k) {
        const uint32_t w = pre[it % (IN_BF16 ? ITERS : 1)][k % (IN_BF16 ? B : 1)];
        v0[k] = bf16lo_to_f32(w);
        v1[k] = bf16hi_to_f32(w);
      }
    } else {
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.x) + (mb * a.ld + c) * ESZ;
#pragma unroll
      for (int k = 0; k < B; ++k) {
        float2 f = make_float2(0.f, 0.f);
        if (ok) f = __ldg(reinterpret_cast<const float2*>(base + a.rht.row_off[k & 15] + (k >= 16 ? half_blk : 0)));
        v0[k] = f.x;
        v1[k] = f.y;
      }
    }
    // ---- transform: y = (H z) / sqrt(16), rounded to the input dtype ----
    if (RHT) {
#pragma unroll
      for (int g = 0; g < B; g += 16) {
        hadamard16_pair(v0 + g, v1 + g);
      }
    }
    // ---- scale by +-1/sqrt(16) (exact), round to the input dtype, block amax on the rounded bits ----
    uint32_t am0 = 0, am1 = 0;
    if (RHT && IN_BF16) {
      // both columns of a lane travel as one packed bf16 pair: one conversion and one packed maximum
      uint32_t acc = 0;
#pragma unroll
      for (int k = 0; k < B; ++k) {
        // the fused +0 turns a -0 product into the +0 that a dot product yields
        const float sg = a.rht.qsign[k & 15];
        const float2 sc = __ffma2_rn(make_float2(v0[k], v1[k]), make_float2(sg, sg), make_float2(0.0f, 0.0f));
        const __nv_bfloat162 p2 = __floats2bfloat162_rn(sc.x, sc.y);
        const uint32_t pw = *reinterpret_cast<const uint32_t*>(&p2);
        acc = absmax_bf16x2(acc, pw);
        v0[k] = bf16lo_to_f32(pw);
        v1[k] = bf16hi_to_f32(pw);
      }
      am0 = acc & 0xFFFFu;
      am1 = acc >> 16;
    } else {
      if (RHT) {
#pragma unroll
        for (int k = 0; k < B; ++k) {
          const float sg = a.rht.qsign[k & 15];
          v0[k] = __fmaf_rn(v0[k], sg, 0.0f);
          v1[k] = __fmaf_rn(v1[k], sg, 0.0f);
        }
      }
#pragma unroll
      for (int k = 0; k < B; ++k) {
        const uint32_t b0 = f2u(v0[k]) & 0x7FFFFFFFu, b1 = f2u(v1[k]) & 0x7FFFFFFFu;
        am0 = b0 > am0 ? b0 : am0;
        am1 = b1 > am1 ? b1 : am1;
      }
      if (IN_BF16) {
        am0 >>= 16;
        am1 >>= 16;
      }
    }
    BlockScale s0, s1;
    if (F::MX && (a.mx.clip | a.mx.uos)) {
      float sum0 = 0.0f, sq0 = 0.0f, sum1 = 0.0f, sq1 = 0.0f;
      if (a.mx.clip == 2) {
#pragma unroll
        for (int k = 0; k < B; ++k) {
          sum0 = __fadd_rn(sum0, v0[k]);
          sq0 = __fadd_rn(sq0, round_in<IN_BF16>(__fmul_rn(v0[k], v0[k])));
          sum1 = __fadd_rn(sum1, v1[k]);
          sq1 = __fadd_rn(sq1, round_in<IN_BF16>(__fmul_rn(v1[k], v1[k])));
        }
      }
      s0 = make_block_scale_opts<FMT, IN_BF16>(am0, sum0, sq0, B, a.mx);
      s1 = make_block_scale_opts<FMT, IN_BF16>(am1, sum1, sq1, B, a.mx);
      if (a.mx.clip == 1) {
#pragma unroll
        for (int k = 0; k < B; ++k) {
          v0[k] = round_in<IN_BF16>(__fmul_rn(v0[k], 0.75f));
          v1[k] = round_in<IN_BF16>(__fmul_rn(v1[k], 0.75f));
        }
      }
    } else {
      s0 = make_block_scale<FMT, IN_BF16>(am0, os);
      s1 = make_block_scale<FMT, IN_BF16>(am1, os);
    }

    // ---- quantise in slot order ----
    if (F::FP4) {
#pragma unroll
      for (int h = 0; h < B / 16; ++h) {
        // With stochastic rounding the random word belongs to the OUTPUT position, so the
        // transformed values are first moved from slot order to position order through a
        // private shared-memory column (static register index, dynamic address).
        constexpr bool TO_POS = RHT && ROUND != ALTOB200_ROUND_RTN;
        float y0[16], y1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          y0[j] = v0[16 * h + j];
          y1[j] = v1[16 * h + j];
        }
        if (TO_POS) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // row pinv[j] of the table (NT pairs of 8 bytes per row): both columns in one 8-byte access
            float2* dst = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(&s_perm[0][threadIdx.x]) +
                                                    a.rht.perm_off[j] * NT);
            *dst = make_float2(y0[j], y1[j]);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 t = s_perm[j][threadIdx.x];
            y0[j] = t.x;
            y1[j] = t.y;
          }
        }
        // random words by position: r0[i]/r1[i] for column c / c+1
        uint32_t r0[16], r1[16];
        if (ROUND == ALTOB200_ROUND_SR_BITS) {
          if (a.tile_rows != 0 && (a.tile_pairs & 7) == 0) {
            // periodic table: the 8 pairs of these 16 rows are 8 consecutive, 32-byte aligned words of
            // one table row in each plane (tile_pairs is a multiple of 8) -> four 16-byte loads per column
            const uint32_t tp = (uint32_t)a.tile_pairs;
            const uint32_t base = (uint32_t)((mb + 16 * h) >> 1) % tp;
            const uint32_t plane = (uint32_t)a.tile_rows * tp;
            const uint32_t* t0 = a.rand_bits + tile_row0 * tp + base;
            const uint32_t* t1 = a.rand_bits + tile_row1 * tp + base;
            uint4 e0[2], o0[2], e1[2], o1[2];  // even / odd planes of column c and c + 1
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              e0[q] = o0[q] = e1[q] = o1[q] = make_uint4(0u, 0u, 0u, 0u);
              if (ok) {
                e0[q] = __ldg(reinterpret_cast<const uint4*>(t0) + q);
                o0[q] = __ldg(reinterpret_cast<const uint4*>(t0 + plane) + q);
                e1[q] = __ldg(reinterpret_cast<const uint4*>(t1) + q);
                o1[q] = __ldg(reinterpret_cast<const uint4*>(t1 + plane) + q);
              }
            }
            const uint32_t ev0[8] = {e0[0].x, e0[0].y, e0[0].z, e0[0].w, e0[1].x, e0[1].y, e0[1].z, e0[1].w};
            const uint32_t od0[8] = {o0[0].x, o0[0].y, o0[0].z, o0[0].w, o0[1].x, o0[1].y, o0[1].z, o0[1].w};
            const uint32_t ev1[8] = {e1[0].x, e1[0].y, e1[0].z, e1[0].w, e1[1].x, e1[1].y, e1[1].z, e1[1].w};
            const uint32_t od1[8] = {o1[0].x, o1[0].y, o1[0].z, o1[0].w, o1[1].x, o1[1].y, o1[1].z, o1[1].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              r0[2 * j] = ev0[j]; r0[2 * j + 1] = od0[j];
              r1[2 * j] = ev1[j]; r1[2 * j + 1] = od1[j];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              r0[i] = r1[i] = 0;
              if (ok) {
                const int64_t idx = (mb + 16 * h + i) >> 1;
                if (a.tile_rows != 0) {
                  const int64_t plane = (int64_t)(i & 1) * a.tile_rows * a.tile_pairs;
                  const int64_t pi = idx % a.tile_pairs;
                  r0[i] = __ldg(a.rand_bits + plane + (int64_t)tile_row0 * a.tile_pairs + pi);
                  r1[i] = __ldg(a.rand_bits + plane + (int64_t)tile_row1 * a.tile_pairs + pi);
                } else {
                  const int64_t plane = (int64_t)(i & 1) * a.cols * half_rows;
                  r0[i] = __ldg(a.rand_bits + plane + c * half_rows + idx);
                  r1[i] = __ldg(a.rand_bits + plane + (c + 1) * half_rows + idx);
                }
              }
            }
          }
        } else if (ROUND == ALTOB200_ROUND_SR_PHILOX) {
          const uint64_t p0 = (uint64_t)(c * half_rows + ((mb + 16 * h) >> 1));        // pair index, column c
          const uint64_t p1 = (uint64_t)((c + 1) * half_rows + ((mb + 16 * h) >> 1));  // column c + 1
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t o[4];
            uint64_t ctr = a.philox_offset + (p0 >> 1) + i;
            philox4x32_10_keys((uint32_t)ctr, (uint32_t)(ctr >> 32), a.pk, o);
            r0[4 * i] = o[0]; r0[4 * i + 1] = o[1]; r0[4 * i + 2] = o[2]; r0[4 * i + 3] = o[3];
            ctr = a.philox_offset + (p1 >> 1) + i;
            philox4x32_10_keys((uint32_t)ctr, (uint32_t)(ctr >> 32), a.pk, o);
            r1[4 * i] = o[0]; r1[4 * i + 1] = o[1]; r1[4 * i + 2] = o[2]; r1[4 * i + 3] = o[3];
          }
        }
        // nibble j = code of entry j (slot order, or position order if TO_POS), in two 32-bit halves
        uint32_t w0h[2] = {0u, 0u}, w1h[2] = {0u, 0u};
        with_uniform_fast(s0.fast && s1.fast, [&](auto fast_tag) {
          constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            uint32_t c0, c1;
            if (ROUND == ALTOB200_ROUND_RTN) {
              // the hardware converter takes one value of each column per call
              const uint32_t b = e2m1x2_rtn_hw(scale_elem<FMT, IN_BF16, FAST>(y0[j], s0),
                                               scale_elem<FMT, IN_BF16, FAST>(y1[j], s1));
              c0 = b & 0xFu;
              c1 = b >> 4;
            } else if (FAST) {
              // both columns' quotients with packed operations (the same three roundings per element)
              const float2 q = scale_pair_mag<FMT>(make_float2(y0[j], y1[j]), s0, s1);
              c0 = e2m1_sr_code(q.x, f2u(y0[j]), r0[j]);
              c1 = e2m1_sr_code(q.y, f2u(y1[j]), r1[j]);
            } else {
              c0 = e2m1_sr_code(scale_elem_mag<FMT, IN_BF16, FAST>(y0[j], s0), f2u(y0[j]), r0[j]);
              c1 = e2m1_sr_code(scale_elem_mag<FMT, IN_BF16, FAST>(y1[j], s1), f2u(y1[j]), r1[j]);
            }
            // disjoint bits: adding is or-ing, and the multiply-add pipe has room where the ALU pipe has not
            w0h[j >> 3] = merge_shifted(c0, 4 * (j & 7), w0h[j >> 3]);
            w1h[j >> 3] = merge_shifted(c1, 4 * (j & 7), w1h[j >> 3]);
          }
        });
        const uint64_t w0 = ((uint64_t)w0h[1] << 32) | w0h[0], w1 = ((uint64_t)w1h[1] << 32) | w1h[0];
        uint64_t o0 = w0, o1 = w1;
        if (RHT && !TO_POS) {  // output position i takes slot perm[i]
          o0 = o1 = 0;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            o0 |= ((w0 >> (4 * a.rht.perm[i])) & 0xFull) << (4 * i);
            o1 |= ((w1 >> (4 * a.rht.perm[i])) & 0xFull) << (4 * i);
          }
        }
        uint8_t* d = s_codes + ((size_t)blk * COL_TN + 2 * lane) * BLK_BYTES + 8 * h;
        *reinterpret_cast<uint2*>(d) = make_uint2((uint32_t)o0, (uint32_t)(o0 >> 32));
        *reinterpret_cast<uint2*>(d + BLK_BYTES) = make_uint2((uint32_t)o1, (uint32_t)(o1 >> 32));
      }
    } else {
      // FP8: one byte per element, no transform (the reference asserts that MXFP8 runs
      // without Hadamard, alto/kernels/dispatch/tensor.py:448-454)
      uint8_t* d = s_codes + ((size_t)blk * COL_TN + 2 * lane) * BLK_BYTES;
      with_uniform_fast(s0.fast && s1.fast, [&](auto fast_tag) {
        constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
        for (int k = 0; k < B; k += 4) {
          float q0[4], q1[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            q0[j] = scale_elem<FMT, IN_BF16, FAST>(v0[k + j], s0);
            q1[j] = scale_elem<FMT, IN_BF16, FAST>(v1[k + j], s1);
          }
          *reinterpret_cast<uint32_t*>(d + k) = fp8x2_rtn_hw<F::E5M2>(q0[0], q0[1]) |
                                                (fp8x2_rtn_hw<F::E5M2>(q0[2], q0[3]) << 16);
          *reinterpret_cast<uint32_t*>(d + BLK_BYTES + k) =
              fp8x2_rtn_hw<F::E5M2>(q1[0], q1[1]) | (fp8x2_rtn_hw<F::E5M2>(q1[2], q1[3]) << 16);
        }
      });
    }
    s_sf[(2 * lane) * NBLK + blk] = ok ? (uint8_t)s0.byte : 0;
    s_sf[(2 * lane + 1) * NBLK + blk] = ok ? (uint8_t)s1.byte : 0;
    if (!F::MX) {
      s_sf_plain[(2 * lane) * NBLK + blk] = s0.plain;
      s_sf_plain[(2 * lane + 1) * NBLK + blk] = s1.plain;
    }
  }
  __syncthreads();

  // ---- write codes: output row n gets ROW_BYTES contiguous bytes, 16 bytes per thread ----
  constexpr int CHUNKS = ROW_BYTES / 16;  // 8 (FP4) or 16 (FP8) per output row
  for (int t = threadIdx.x; t < COL_TN * CHUNKS; t += NT) {
    const int n = t / CHUNKS, ch = t - n * CHUNKS;
    const int64_t col = n0 + n;
    const int64_t mrow = m0 + (int64_t)ch * (F::FP4 ? 32 : 16);  // first row covered by this chunk
    if (col >= a.cols || mrow >= a.rows) continue;
    // a 16-byte chunk covers 32 rows (FP4) or 16 rows (FP8)
    uint4 o;
    if (BLK_BYTES >= 16) {
      const int blk = (ch * 16) / BLK_BYTES, off = (ch * 16) % BLK_BYTES;
      o = *reinterpret_cast<const uint4*>(s_codes + ((size_t)blk * COL_TN + n) * BLK_BYTES + off);
    } else {  // BLK_BYTES == 8: two blocks per chunk
      const uint2 lo = *reinterpret_cast<const uint2*>(s_codes + ((size_t)(2 * ch) * COL_TN + n) * 8);
      const uint2 hi = *reinterpret_cast<const uint2*>(s_codes + ((size_t)(2 * ch + 1) * COL_TN + n) * 8);
      o = make_uint4(lo.x, lo.y, hi.x, hi.y);
    }
    uint8_t* dst = a.codes + col * (F::FP4 ? half_rows : a.rows) + (F::FP4 ? (m0 >> 1) : m0) + ch * 16;
    const int64_t rows_left = a.rows - mrow;
    if (rows_left >= (F::FP4 ? 32 : 16)) {
      *reinterpret_cast<uint4*>(dst) = o;
    } else {  // ragged tail: rows_left is a multiple of B = 16 here (NVFP4 only)
      *reinterpret_cast<uint2*>(dst) = make_uint2(o.x, o.y);
    }
  }
  // ---- write scales ----
  const int64_t nkb = a.rows / B;
  if (a.scale_plain != nullptr) {
    for (int t = threadIdx.x; t < COL_TN * NBLK; t += NT) {
      const int n = t / NBLK, b = t - n * NBLK;
      const int64_t col = n0 + n, kb = m0 / B + b;
      if (col < a.cols && kb < nkb) {
        if (F::MX) reinterpret_cast<uint8_t*>(a.scale_plain)[col * nkb + kb] = s_sf[n * NBLK + b];
        else reinterpret_cast<float*>(a.scale_plain)[col * nkb + kb] = s_sf_plain[n * NBLK + b];
      }
    }
  }
  if (a.scale_packed != nullptr) {
    for (int t = threadIdx.x; t < COL_TN * (NBLK / 4); t += NT) {
      const int n = t / (NBLK / 4), qd = t - n * (NBLK / 4);
      const int64_t col = n0 + n, kb = m0 / B + qd * 4;
      if (col < a.cols && kb < a.ncol_tiles * 4) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (kb + j < nkb) word |= (uint32_t)s_sf[n * NBLK + qd * 4 + j] << (8 * j);
        *reinterpret_cast<uint32_t*>(a.scale_packed + packed_scale_offset(col, kb, a.ncol_tiles)) = word;
      }
    }
  }
}

// =======================================================================================
// 2D block quantizer with dual packing
// =======================================================================================
struct Quant2dArgs {
  const void* w;
  int64_t rows, cols, ld;
  uint8_t* codes_k;   // [rows, cols/2] or [rows, cols]
  uint8_t* codes_t;   // [cols, rows/2] or [cols, rows]
  void* scale_plain;  // [rows/B, cols/B]
  uint8_t* packed_k;  // rows=rows, ncols=cols/B
  uint8_t* packed_t;  // rows=cols, ncols=rows/B
  int64_t nct_k, nct_t;
  const float* outer;
  MxOpts mx;          // clip 0/1/2 and uos
  // stochastic rounding (FP4): words by (row, pair of columns) as in the row-wise quantizer: full planes
  // [2][rows][cols/2], or a periodic table [2][tile_rows][tile_pairs]
  const uint32_t* rand_bits;
  int64_t tile_rows, tile_pairs;
  // batch of equally shaped matrices: input stride in elements, outputs stacked contiguously; the
  // rows of the stochastic-rounding view are the rows of all matrices, one after the other
  int64_t batch, batch_stride, packed_k_bytes, packed_t_bytes;
};

// 4 x 4 byte transpose: out[b] = (in[0].byte b, in[1].byte b, in[2].byte b, in[3].byte b)
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t* in, uint32_t* out) {
  const uint32_t t0 = __byte_perm(in[0], in[1], 0x5140);  // a0 b0 a1 b1
  const uint32_t t1 = __byte_perm(in[2], in[3], 0x5140);  // c0 d0 c1 d1
  const uint32_t t2 = __byte_perm(in[0], in[1], 0x7362);  // a2 b2 a3 b3
  const uint32_t t3 = __byte_perm(in[2], in[3], 0x7362);  // c2 d2 c3 d3
  out[0] = __byte_perm(t0, t1, 0x5410);
  out[1] = __byte_perm(t0, t1, 0x7632);
  out[2] = __byte_perm(t2, t3, 0x5410);
  out[3] = __byte_perm(t2, t3, 0x7632);
}

// A thread owns 16 rows x 8 columns, kept in registers from the load to both stores; a warp owns
// 4 block columns (LC lanes) x 16 * LR rows, so block maxima need shuffles only and the kernel uses
// no shared memory.  The K packing is written row by row (4 or 8 bytes per row per lane, 32 or 128
// contiguous bytes per row per warp); for the transposed packing the thread's 16 x 8 codes are
// transposed in registers (nibble merge of row pairs, then 4 x 4 byte transposes) and every column
// receives 8 (FP4) or 16 (FP8) contiguous bytes per lane, 32 contiguous bytes per warp and column.
template <int FMT, bool IN_BF16, int ROUND, bool BATCHED>
__global__ void __launch_bounds__(256) quantize_2d_kernel(Quant2dArgs a) {
  grid_dependency_wait();
  using F = Fmt<FMT>;
  constexpr int B = F::B;
  constexpr int LC = B / 2;          // lanes across columns: 8 columns each, 4 block columns per warp
  constexpr int LR = 32 / LC;        // 16-row groups per warp: 4 (B = 16) or 2 (B = 32)
  constexpr int TR = 16 * LR, TC = 8 * LC;  // warp tile: 64 x 64 or 32 x 128
  constexpr int ESZ = IN_BF16 ? 2 : 4;
  const int lane = threadIdx.x & 31;
  const int64_t tiles_c = (a.cols + TC - 1) / TC, tiles_r = (a.rows + TR - 1) / TR;
  const int64_t tile_all = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tile_all >= tiles_c * tiles_r * a.batch) return;  // whole warps leave; nothing below synchronises the block
  // matrix `bi` of the batch: its outputs follow those of matrix bi - 1, so the batch index enters the
  // addresses as extra rows (bi * rows for the K packing, bi * cols for the transposed one)
  // (BATCHED is a template parameter so that the single-matrix kernel carries none of this arithmetic)
  int64_t bi = 0, tile = tile_all;
  if (BATCHED) divmod_fast(tile_all, tiles_c * tiles_r, &bi, &tile);
  const int64_t rows_before = BATCHED ? bi * a.rows : 0, cols_before = BATCHED ? bi * a.cols : 0;
  int64_t tr, tc;
  divmod_fast(tile, tiles_c, &tr, &tc);
  const int lc = lane % LC, lr = lane / LC;
  const int64_t row0 = tr * TR + lr * 16, col0 = tc * TC + lc * 8;
  const bool ok = row0 < a.rows && col0 < a.cols;  // rows % B == 0 and cols % B == 0
  const OuterScale os = make_outer_scale((!F::MX) && a.outer != nullptr, a.outer);
  const uint8_t* src = reinterpret_cast<const uint8_t*>(a.w) + (bi * a.batch_stride + row0 * a.ld + col0) * ESZ;
  const int64_t pitch = a.ld * ESZ;

  // ---- load and block maximum ----
  uint4 raw[IN_BF16 ? 16 : 1];  // bf16: the 16 x 8 elements stay in registers; fp32: rows are read again
  uint32_t amax_bits = 0;
  // the dynamic clip (MX formats) takes the block's sum and sum of squares instead of its maximum
  const bool stats = F::MX && a.mx.clip == 2;
  float sum = 0.0f, sumsq = 0.0f;
  if (IN_BF16) {
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      raw[i] = ok ? __ldg(reinterpret_cast<const uint4*>(src + i * pitch)) : make_uint4(0u, 0u, 0u, 0u);
      acc = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(acc, raw[i].x), raw[i].y), raw[i].z), raw[i].w);
    }
    amax_bits = fold_bf16x2(acc);
    if (stats) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = bf16lo_to_f32(w[j]), hi = bf16hi_to_f32(w[j]);
          sum = __fadd_rn(__fadd_rn(sum, lo), hi);
          sumsq = __fadd_rn(__fadd_rn(sumsq, round_in<true>(__fmul_rn(lo, lo))), round_in<true>(__fmul_rn(hi, hi)));
        }
      }
    }
  } else if (ok) {
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const uint4 p = __ldg(reinterpret_cast<const uint4*>(src + i * pitch));
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(src + i * pitch) + 1);
      const uint32_t ws[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t b = ws[j] & 0x7FFFFFFFu;
        amax_bits = b > amax_bits ? b : amax_bits;
        if (stats) {
          sum = __fadd_rn(sum, u2f(ws[j]));
          sumsq = __fadd_rn(sumsq, __fmul_rn(u2f(ws[j]), u2f(ws[j])));
        }
      }
    }
  }
  // lanes of one block: B / 8 neighbours along the columns, B / 16 row groups
#pragma unroll
  for (int o = 1; o < B / 8; o <<= 1) {
    const uint32_t t = __shfl_xor_sync(0xFFFFFFFFu, amax_bits, o);
    amax_bits = t > amax_bits ? t : amax_bits;
    if (stats) {   // uniform: a launch argument
      sum = __fadd_rn(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, o));
      sumsq = __fadd_rn(sumsq, __shfl_xor_sync(0xFFFFFFFFu, sumsq, o));
    }
  }
  if (B == 32) {
    const uint32_t t = __shfl_xor_sync(0xFFFFFFFFu, amax_bits, LC);
    amax_bits = t > amax_bits ? t : amax_bits;
    if (stats) {
      sum = __fadd_rn(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, LC));
      sumsq = __fadd_rn(sumsq, __shfl_xor_sync(0xFFFFFFFFu, sumsq, LC));
    }
  }
  const BlockScale s = (F::MX && (a.mx.clip | a.mx.uos))
                           ? make_block_scale_opts<FMT, IN_BF16>(amax_bits, sum, sumsq, B * B, a.mx)
                           : make_block_scale<FMT, IN_BF16>(amax_bits, os);
  const bool clip = F::MX && a.mx.clip == 1;

  // ---- encode row by row, K packing ----
  uint32_t kw[F::FP4 ? 16 : 32];  // FP4: one word per row (8 codes); FP8: two words per row (8 bytes)
  with_uniform_fast(s.fast, [&](auto fast_tag) {
    constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float v[8];
      if (IN_BF16) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[2 * j] = bf16lo_to_f32(w[j]);
          v[2 * j + 1] = bf16hi_to_f32(w[j]);
        }
      } else {
        float4 p = make_float4(0.f, 0.f, 0.f, 0.f), q = p;
        if (ok) {
          p = __ldg(reinterpret_cast<const float4*>(src + i * pitch));
          q = __ldg(reinterpret_cast<const float4*>(src + i * pitch) + 1);
        }
        v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w;
        v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
      }
      if (clip) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = round_in<IN_BF16>(__fmul_rn(v[j], 0.75f));
      }
      if (F::FP4 && ROUND == ALTOB200_ROUND_SR_BITS) {
        // the lane's 4 column pairs are 4 consecutive, 16-byte aligned words of each plane
        const bool tiled = a.tile_rows != 0;
        const int64_t row = rows_before + row0 + i;  // row of the flattened view over the batch
        // (a 64-bit modulo only where the flattened row index needs it: it costs ~70 instructions)
        const int64_t rr = !tiled ? row
                           : ((uint64_t)row >> 32) == 0 ? (int64_t)((uint32_t)row % (uint32_t)a.tile_rows)
                                                        : (int64_t)((uint64_t)row % (uint64_t)a.tile_rows);
        const int64_t pp = tiled ? (int64_t)((uint32_t)(col0 >> 1) % (uint32_t)a.tile_pairs) : (col0 >> 1);
        const int64_t pitch = tiled ? a.tile_pairs : (a.cols >> 1);
        const int64_t plane = tiled ? a.tile_rows * a.tile_pairs : a.batch * a.rows * (a.cols >> 1);
        uint4 re = make_uint4(0u, 0u, 0u, 0u), ro = re;
        if (ok) {
          re = __ldg(reinterpret_cast<const uint4*>(a.rand_bits + rr * pitch + pp));
          ro = __ldg(reinterpret_cast<const uint4*>(a.rand_bits + plane + rr * pitch + pp));
        }
        const uint32_t e4[4] = {re.x, re.y, re.z, re.w}, o4[4] = {ro.x, ro.y, ro.z, ro.w};
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          word = merge_shifted(fp4_pair<FMT, IN_BF16, ROUND, FAST>(v[2 * j], v[2 * j + 1], s, e4[j], o4[j]), 8 * j, word);
        kw[i] = word;
        if (ok) *reinterpret_cast<uint32_t*>(a.codes_k + (rows_before + row0 + i) * (a.cols >> 1) + (col0 >> 1)) = kw[i];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = scale_elem<FMT, IN_BF16, FAST>(v[j], s);
        if (F::FP4) {
          kw[i] = e2m1x2_rtn_hw(v[0], v[1]) | (e2m1x2_rtn_hw(v[2], v[3]) << 8) | (e2m1x2_rtn_hw(v[4], v[5]) << 16) |
                  (e2m1x2_rtn_hw(v[6], v[7]) << 24);
          if (ok) *reinterpret_cast<uint32_t*>(a.codes_k + (rows_before + row0 + i) * (a.cols >> 1) + (col0 >> 1)) = kw[i];
        } else {
          kw[2 * i] = fp8x2_rtn_hw<F::E5M2>(v[0], v[1]) | (fp8x2_rtn_hw<F::E5M2>(v[2], v[3]) << 16);
          kw[2 * i + 1] = fp8x2_rtn_hw<F::E5M2>(v[4], v[5]) | (fp8x2_rtn_hw<F::E5M2>(v[6], v[7]) << 16);
          if (ok)
            *reinterpret_cast<uint2*>(a.codes_k + (rows_before + row0 + i) * a.cols + col0) = make_uint2(kw[2 * i], kw[2 * i + 1]);
        }
      }
    }
  });

  // ---- transposed packing: column col0 + c, rows row0 .. row0 + 15 along the packed axis ----
  if (a.codes_t != nullptr) {
    if (F::FP4) {
      // byte j of ev[..] / od[..]: rows 2j (low nibble) and 2j + 1 of an even / odd column
      uint32_t ev[8], od[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t lo = kw[2 * j], hi = kw[2 * j + 1];
        ev[j] = (lo & 0x0F0F0F0Fu) | ((hi << 4) & 0xF0F0F0F0u);  // byte b: column 2b
        od[j] = ((lo >> 4) & 0x0F0F0F0Fu) | (hi & 0xF0F0F0F0u);  // byte b: column 2b + 1
      }
      uint32_t e0[4], e1[4], o0[4], o1[4];
      transpose4x4_bytes(ev, e0);      // e0[b]: bytes 0..3 of column 2b
      transpose4x4_bytes(ev + 4, e1);  // e1[b]: bytes 4..7
      transpose4x4_bytes(od, o0);
      transpose4x4_bytes(od + 4, o1);
      if (ok) {
        uint8_t* dst = a.codes_t + (cols_before + col0) * (a.rows >> 1) + (row0 >> 1);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          *reinterpret_cast<uint2*>(dst + (2 * b) * (a.rows >> 1)) = make_uint2(e0[b], e1[b]);
          *reinterpret_cast<uint2*>(dst + (2 * b + 1) * (a.rows >> 1)) = make_uint2(o0[b], o1[b]);
        }
      }
    } else {
      // kw[2 i + h]: row i, bytes = columns 4h .. 4h + 3
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t t[4][4];  // t[g][b]: rows 4g .. 4g + 3 of column 4h + b
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t in[4] = {kw[2 * (4 * g) + h], kw[2 * (4 * g + 1) + h], kw[2 * (4 * g + 2) + h],
                                  kw[2 * (4 * g + 3) + h]};
          transpose4x4_bytes(in, t[g]);
        }
        if (ok) {
#pragma unroll
          for (int b = 0; b < 4; ++b)
            *reinterpret_cast<uint4*>(a.codes_t + (cols_before + col0 + 4 * h + b) * a.rows + row0) =
                make_uint4(t[0][b], t[1][b], t[2][b], t[3][b]);
        }
      }
    }
  }

  // ---- scales ----
  const bool col_ok = col0 < a.cols, row_ok = row0 < a.rows;
  if (a.scale_plain != nullptr && ok && (lc % (B / 8)) == 0 && (lr % (B / 16)) == 0) {
    const int64_t idx = ((rows_before + row0) / B) * (a.cols / B) + col0 / B;
    if (F::MX) reinterpret_cast<uint8_t*>(a.scale_plain)[idx] = (uint8_t)s.byte;
    else reinterpret_cast<float*>(a.scale_plain)[idx] = s.plain;
  }
  const uint32_t my_byte = ok ? s.byte : 0u;  // blocks outside the matrix contribute zero bytes
  if (a.packed_k != nullptr) {
    // one word per row: the scale bytes of the warp's 4 block columns; the rows of a group are
    // shared out over its LC lanes
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) word |= __shfl_sync(0xFFFFFFFFu, my_byte, lr * LC + j * (B / 8)) << (8 * j);
    const int64_t kb = tc * 4;
    if (row_ok) {
#pragma unroll
      for (int i = 0; i < 16 / LC; ++i) {
        const int64_t row = row0 + lc * (16 / LC) + i;
        *reinterpret_cast<uint32_t*>(a.packed_k + bi * a.packed_k_bytes + packed_scale_offset(row, kb, a.nct_k)) = word;
      }
    }
  }
  if (a.packed_t != nullptr) {
    // rows of this layout are the matrix columns, scale columns the row blocks
    if (LR == 4) {
      // B = 16: the warp's 4 row groups are the 4 bytes of one word; the 8 columns of a lane are
      // shared out over the 4 row groups
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) word |= __shfl_sync(0xFFFFFFFFu, my_byte, j * LC + lc) << (8 * j);
      if (col_ok) {
#pragma unroll
        for (int e = 0; e < 2; ++e)
          *reinterpret_cast<uint32_t*>(a.packed_t + bi * a.packed_t_bytes +
                                       packed_scale_offset(col0 + 2 * lr + e, tr * 4, a.nct_t)) = word;
      }
    } else {
      // B = 32: the warp holds one row block, one byte per column
      if (ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          a.packed_t[bi * a.packed_t_bytes + packed_scale_offset(col0 + 4 * lr + e, tr, a.nct_t)] = (uint8_t)s.byte;
      }
    }
  }
}

// =======================================================================================
// Tensor amax (plain and Hadamard-transformed) with the outer-scale finalisation
// =======================================================================================
struct AmaxArgs {
  const void* x;
  int64_t rows, cols, ld;
  uint32_t* amax_bits;   // [2], written by the last block
  float* outer_scale;    // [2] or NULL
  uint32_t* counter;     // scratch [4]: ticket counter, running maxima; zero on entry, zero on exit
  RhtParams rht;
};

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const uint32_t t = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = t > v ? t : v;
  }
  return v;
}

// outer = max(nan_to_num(amax) / (448 * 6), 1e-30)
//   alto/kernels/fp4/nvfp4/nvfp_quantization.py:484-487
__device__ __forceinline__ float outer_from_amax_bits(uint32_t bits) {
  float amax = u2f(bits);
  if (bits > 0x7F800000u) amax = 0.0f;               // NaN -> 0
  if (bits == 0x7F800000u) amax = 3.4028234663852886e38f;  // nan_to_num(+inf) -> float max
  return fmaxf(__fdiv_rn(amax, 2688.0f), 1.0e-30f);
}

template <bool IN_BF16, bool RHT>
__global__ void __launch_bounds__(256) amax_kernel(AmaxArgs a) {
  grid_dependency_wait();
  __shared__ uint32_t s_red[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t am_plain = 0, am_rht = 0;
  if (!RHT) {
    // flat pass, 16 bytes per thread per step; rows are contiguous when ld == cols
    const int64_t vec = IN_BF16 ? 8 : 4;
    const int64_t vec_per_row = a.cols / vec;
    const int64_t total = a.rows * vec_per_row;
    const bool dense = a.ld == a.cols;  // contiguous rows: no index arithmetic per load
    auto load = [&](int64_t i) -> uint4 {
      int64_t off = i * vec;
      if (!dense) {
        int64_t row, cv;
        divmod_fast(i, vec_per_row, &row, &cv);
        off = row * a.ld + cv * vec;
      }
      return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.x) + off * (IN_BF16 ? 2 : 4)));
    };
    // four independent 16-byte loads are issued before any of them is consumed: the pass is a pure
    // stream and needs bytes in flight, not arithmetic
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i0 < total; i0 += 4 * stride) {
      uint4 wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = i0 + u * stride;
        wv[u] = i < total ? load(i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
      const uint4 w = wv[u];
      if (IN_BF16) {
        uint32_t acc = absmax_bf16x2(0, w.x);
        acc = absmax_bf16x2(acc, w.y);
        acc = absmax_bf16x2(acc, w.z);
        acc = absmax_bf16x2(acc, w.w);
        const uint32_t m = fold_bf16x2(acc) << 16;
        am_plain = m > am_plain ? m : am_plain;
      } else {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t b = ws[j] & 0x7FFFFFFFu;
          am_plain = b > am_plain ? b : am_plain;
        }
      }
      }
    }
  } else {
    // column pass: 16-row groups x 2 columns per lane, as in the column-wise quantizer.  Rounding to
    // the input dtype and the factor 1/4 are monotone in the magnitude, so the maximum is taken over
    // the raw butterfly outputs and scaled and rounded once per thread.
    const int64_t groups = a.rows >> 4;
    const int64_t col_tiles = (a.cols + 63) >> 6;
    const int64_t n_tasks = groups * col_tiles;
    const int64_t warp0 = (int64_t)blockIdx.x * 8 + warp, n_warps = (int64_t)gridDim.x * 8;
    uint32_t raw_rht = 0, plain16 = 0;
    for (int64_t task = warp0; task < n_tasks; task += n_warps) {
      int64_t g, ct;
      divmod_fast(task, col_tiles, &g, &ct);
      const int64_t c = (ct << 6) + 2 * lane;
      if (c >= a.cols) continue;
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.x) + ((g << 4) * a.ld + c) * (IN_BF16 ? 2 : 4);
      float v0[16], v1[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        if (IN_BF16) {
          const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(base + a.rht.row_off[k]));
          plain16 = absmax_bf16x2(plain16, w);
          v0[k] = bf16lo_to_f32(w);
          v1[k] = bf16hi_to_f32(w);
        } else {
          const float2 f = __ldg(reinterpret_cast<const float2*>(base + a.rht.row_off[k]));
          const uint32_t b0 = f2u(f.x) & 0x7FFFFFFFu, b1 = f2u(f.y) & 0x7FFFFFFFu;
          am_plain = b0 > am_plain ? b0 : am_plain;
          am_plain = b1 > am_plain ? b1 : am_plain;
          v0[k] = f.x;
          v1[k] = f.y;
        }
      }
      hadamard16_pair(v0, v1);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        // integer maximum of the magnitudes' bits: a NaN is larger than every number, as in torch.amax
        const uint32_t b0 = f2u(v0[k]) & 0x7FFFFFFFu, b1 = f2u(v1[k]) & 0x7FFFFFFFu;
        raw_rht = b0 > raw_rht ? b0 : raw_rht;
        raw_rht = b1 > raw_rht ? b1 : raw_rht;
      }
    }
    if (IN_BF16) am_plain = fold_bf16x2(plain16) << 16;
    // the row signs of the transform do not change magnitudes
    const float y = __fmul_rn(u2f(raw_rht), 0.25f);
    am_rht = IN_BF16 ? ((f32_to_bf16_bits(y) & 0x7FFFu) << 16) : (f2u(y) & 0x7FFFFFFFu);
  }
  am_plain = warp_max_u32(am_plain);
  am_rht = warp_max_u32(am_rht);
  if (lane == 0) {
    s_red[0][warp] = am_plain;
    s_red[1][warp] = am_rht;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t p = 0, h = 0;
    for (int i = 0; i < 8; ++i) {
      p = s_red[0][i] > p ? s_red[0][i] : p;
      h = s_red[1][i] > h ? s_red[1][i] : h;
    }
    // the running maxima live in the scratch words behind the counter, so that the result buffer needs
    // no clearing launch in front of the kernel; the last block moves them out and leaves the scratch zero
    atomicMax(a.counter + 1, p);
    if (RHT) atomicMax(a.counter + 2, h);
    __threadfence();
    const uint32_t ticket = atomicAdd(a.counter, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      const uint32_t fp = atomicExch(a.counter + 1, 0u), fh = RHT ? atomicExch(a.counter + 2, 0u) : 0u;
      a.amax_bits[0] = fp;
      a.amax_bits[1] = fh;
      if (a.outer_scale != nullptr) {
        a.outer_scale[0] = outer_from_amax_bits(fp);
        if (RHT) a.outer_scale[1] = outer_from_amax_bits(fh);
      }
      *a.counter = 0u;
    }
  }
}

// =======================================================================================
// Tensor amax without any caller- or library-allocated scratch
// =======================================================================================
// Partial maxima (one word per block) and the completion counter live in this file-scope array.
// Every GPU that loads the library holds these bytes until the process exits.
constexpr int NOALLOC_MAX_BLOCKS = 8192;
constexpr int NOALLOC_VEC_PER_THREAD = 16;  // 16-byte vectors per thread -> 64 KiB of input per block
struct NoallocScratch {
  uint32_t counter;
  uint32_t pad[63];
  uint32_t partial[NOALLOC_MAX_BLOCKS];
};
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoallocScratch)];

struct AmaxNoallocArgs {
  const void* x;
  int64_t rows, cols, ld;
  uint32_t* amax_bits;   // [1]
  float* outer_scale;    // [1] or NULL
  NoallocScratch* scratch;
};

template <bool IN_BF16>
__global__ void __launch_bounds__(256) amax_noalloc_kernel(AmaxNoallocArgs a) {
  __shared__ uint32_t s_red[8];
  __shared__ bool s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t vec = IN_BF16 ? 8 : 4;
  const int64_t vec_per_row = a.cols / vec;
  const int64_t total = a.rows * vec_per_row;
  const bool dense = a.ld == a.cols;
  uint32_t am = 0;
  const int64_t base = (int64_t)blockIdx.x * (256 * NOALLOC_VEC_PER_THREAD) + threadIdx.x;
#pragma unroll 4
  for (int j = 0; j < NOALLOC_VEC_PER_THREAD; ++j) {
    const int64_t i = base + (int64_t)j * 256;
    if (i >= total) break;
    int64_t off = i * vec;
    if (!dense) {
      int64_t row, cv;
      divmod_fast(i, vec_per_row, &row, &cv);
      off = row * a.ld + cv * vec;
    }
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(
        reinterpret_cast<const uint8_t*>(a.x) + off * (IN_BF16 ? 2 : 4)));
    if (IN_BF16) {
      uint32_t acc = absmax_bf16x2(0, w.x);
      acc = absmax_bf16x2(acc, w.y);
      acc = absmax_bf16x2(acc, w.z);
      acc = absmax_bf16x2(acc, w.w);
      const uint32_t m = fold_bf16x2(acc) << 16;
      am = m > am ? m : am;
    } else {
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t b = ws[q] & 0x7FFFFFFFu;
        am = b > am ? b : am;
      }
    }
  }
  am = warp_max_u32(am);
  if (lane == 0) s_red[warp] = am;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t m = 0;
    for (int i = 0; i < 8; ++i) m = s_red[i] > m ? s_red[i] : m;
    a.scratch->partial[blockIdx.x] = m;
    __threadfence();
    s_last = atomicAdd(&a.scratch->counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {  // the last block to finish folds every block's partial maximum
    __threadfence();
    uint32_t m = 0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += 256) {
      const uint32_t p = *reinterpret_cast<volatile uint32_t*>(&a.scratch->partial[i]);
      m = p > m ? p : m;
    }
    m = warp_max_u32(m);
    __syncthreads();
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t f = 0;
      for (int i = 0; i < 8; ++i) f = s_red[i] > f ? s_red[i] : f;
      a.amax_bits[0] = f;
      if (a.outer_scale != nullptr) a.outer_scale[0] = outer_from_amax_bits(f);
      a.scratch->counter = 0u;  // ready for the next call
    }
  }
}

// =======================================================================================
// Dequantizer (row-major codes, plain scales)
// =======================================================================================
struct DequantArgs {
  const uint8_t* codes;
  const void* scales;
  const float* outer;
  int64_t rows, cols, ld_out;
  void* out;
  int is_2d;
  int static_clip;  // MXFP4: decoded values are multiplied by 4/3 in the output dtype before scaling
};

template <int FMT, bool OUT_BF16>
__global__ void __launch_bounds__(256) dequantize_kernel(DequantArgs a) {
  grid_dependency_wait();
  using F = Fmt<FMT>;
  const int64_t segs_per_row = a.cols >> 4;
  const int64_t total = a.rows * segs_per_row;
  const float outer = (!F::MX && a.outer != nullptr) ? __ldg(a.outer) : 1.0f;
  const bool use_outer = (!F::MX && a.outer != nullptr);
  const int64_t nsc = a.cols / F::B;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t row, sg;
    divmod_fast(i, segs_per_row, &row, &sg);
    const int64_t col = sg << 4;
    const int64_t srow = a.is_2d ? row / F::B : row;
    float s;
    if (F::MX) {
      s = u2f((uint32_t)reinterpret_cast<const uint8_t*>(a.scales)[srow * nsc + col / F::B] << 23);
    } else {
      s = reinterpret_cast<const float*>(a.scales)[srow * nsc + col / F::B];
      if (use_outer) s = __fmul_rn(s, outer);
    }
    float v[16];
    if (F::FP4) {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(a.codes + row * (a.cols >> 1) + (col >> 1)));
      const uint32_t ws[2] = {w.x, w.y};
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float d = e2m1_decode((ws[j >> 3] >> (4 * (j & 7))) & 0xFu);
        // tests/unittest/mxfp4/utils.py:381-384: cast, times 4/3 in the output dtype, then the scale
        if (a.static_clip) d = round_in<OUT_BF16>(__fmul_rn(d, (float)(4.0 / 3.0)));
        v[j] = __fmul_rn(d, s);
      }
    } else {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(a.codes + row * a.cols + col));
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = fp8x2_decode<F::E5M2>((ws[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
        v[2 * j] = __fmul_rn(f.x, s);
        v[2 * j + 1] = __fmul_rn(f.y, s);
      }
    }
    if (OUT_BF16) {
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o[j] = f32_to_bf16_bits(v[2 * j]) | (f32_to_bf16_bits(v[2 * j + 1]) << 16);
      uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + row * a.ld_out + col);
      d[0] = make_uint4(o[0], o[1], o[2], o[3]);
      d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
      float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + row * a.ld_out + col);
#pragma unroll
      for (int j = 0; j < 4; ++j) d[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  }
}

// =======================================================================================
// Standalone randomised Hadamard transform (n = 16)
// =======================================================================================
struct RhtArgs {
  const void* x;
  void* y;
  int64_t rows, cols, ld, ld_y;
  RhtParams rht;
};

template <bool IN_BF16>
__global__ void __launch_bounds__(256) rht_kernel(RhtArgs a) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t groups = a.rows >> 4;
  const int64_t col_tiles = (a.cols + 63) >> 6;
  const int64_t n_tasks = groups * col_tiles;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + warp, n_warps = (int64_t)gridDim.x * 8;
  for (int64_t task = warp0; task < n_tasks; task += n_warps) {
    int64_t g, ct;
    divmod_fast(task, col_tiles, &g, &ct);
    const int64_t c = (ct << 6) + 2 * lane;
    if (c >= a.cols) continue;
    float v0[16], v1[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int src = a.rht.pinv[k];
      float f0, f1;
      if (IN_BF16) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(
            reinterpret_cast<const __nv_bfloat16*>(a.x) + ((g << 4) + src) * a.ld + c));
        f0 = bf16lo_to_f32(w);
        f1 = bf16hi_to_f32(w);
      } else {
        const float2 f = __ldg(reinterpret_cast<const float2*>(
            reinterpret_cast<const float*>(a.x) + ((g << 4) + src) * a.ld + c));
        f0 = f.x;
        f1 = f.y;
      }
      v0[k] = f0;
      v1[k] = f1;
    }
    hadamard16(v0);
    hadamard16(v1);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      // slot k is output row pinv[k] of the group (y[i] = sign[perm[i]] * u[perm[i]])
      const int64_t orow = (g << 4) + a.rht.pinv[k];
      const float sg = 0.25f * a.rht.sign[k];
      const float y0 = __fadd_rn(__fmul_rn(v0[k], sg), 0.0f), y1 = __fadd_rn(__fmul_rn(v1[k], sg), 0.0f);
      if (IN_BF16) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(a.y) + orow * a.ld_y + c) =
            f32_to_bf16_bits(y0) | (f32_to_bf16_bits(y1) << 16);
      } else {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.y) + orow * a.ld_y + c) = make_float2(y0, y1);
      }
    }
  }
}

// =======================================================================================
// host side
// =======================================================================================
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148;
  }
  return n;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int fill_rht(RhtParams* r, int n, const int32_t* perm, const int32_t* sign) {
  r->n = n;
  if (n == 0) {
    for (int i = 0; i < 16; ++i) {
      r->pinv[i] = (int8_t)i; r->perm[i] = (int8_t)i; r->sign[i] = 1.0f;
      r->qsign[i] = 0.25f; r->perm_off[i] = i * 8;
    }
    return ALTOB200_OK;
  }
  if (n != 16) return ALTOB200_EUNSUPPORTED;
  if (perm == nullptr || sign == nullptr) return ALTOB200_EINVAL_SHAPE;
  bool seen[16] = {false};
  for (int i = 0; i < 16; ++i) {
    if (perm[i] < 0 || perm[i] > 15 || seen[perm[i]]) return ALTOB200_EINVAL_SHAPE;
    if (sign[i] != 1 && sign[i] != -1) return ALTOB200_EINVAL_SHAPE;
    seen[perm[i]] = true;
  }
  // W[i][j] = sign[perm[i]] * H[perm[i]][perm[j]]:  z[k] = x[pinv[k]],  y[i] = sign[perm[i]] * (H z)[perm[i]]
  for (int i = 0; i < 16; ++i) {
    r->perm[i] = (int8_t)perm[i];
    r->pinv[perm[i]] = (int8_t)i;
    r->sign[i] = (float)sign[i];
  }
  for (int k = 0; k < 16; ++k) {
    r->qsign[k] = 0.25f * r->sign[k];
    r->perm_off[k] = (int)r->pinv[k] * 8;
  }
  return ALTOB200_OK;
}

// Byte offsets of the rows that feed butterfly slots 0..15, for a matrix with leading dimension `ld`.
static void fill_rht_row_offsets(RhtParams* r, int64_t ld, int esz) {
  for (int k = 0; k < 16; ++k) r->row_off[k] = (int64_t)r->pinv[k] * ld * esz;
}

template <int FMT, bool IN_BF16>
static int launch_rowwise(const RowwiseArgs& a, int rounding, cudaStream_t st) {
  const int64_t tasks = ceil_div(a.rows, ROW_R) * ((a.cols + 511) >> 9);
  int64_t blocks = ceil_div(tasks, 8);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (rounding == ALTOB200_ROUND_RTN)
    (void)launch_after(quantize_rowwise_kernel<FMT, IN_BF16, ALTOB200_ROUND_RTN>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  else if (rounding == ALTOB200_ROUND_SR_BITS && Fmt<FMT>::FP4)
    (void)launch_after(quantize_rowwise_kernel<FMT, IN_BF16, Fmt<FMT>::FP4 ? ALTOB200_ROUND_SR_BITS : ALTOB200_ROUND_RTN>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  else if (rounding == ALTOB200_ROUND_SR_PHILOX && Fmt<FMT>::FP4)
    (void)launch_after(quantize_rowwise_kernel<FMT, IN_BF16, Fmt<FMT>::FP4 ? ALTOB200_ROUND_SR_PHILOX : ALTOB200_ROUND_RTN>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  else
    return ALTOB200_EUNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

template <int FMT, bool IN_BF16>
static int launch_colwise(const ColwiseArgs& a, int rounding, cudaStream_t st) {
  const bool rht = a.rht.n != 0;
  if (!Fmt<FMT>::FP4 && (rht || rounding != ALTOB200_ROUND_RTN)) return ALTOB200_EUNSUPPORTED;
  const unsigned gx = (unsigned)ceil_div(a.cols, COL_TN);
  if (rounding == ALTOB200_ROUND_RTN) {
    constexpr int NT = COL_NT;
    const dim3 grid(gx, (unsigned)ceil_div(a.rows, NT));
    if (rht) (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, ALTOB200_ROUND_RTN, Fmt<FMT>::FP4>, dim3(grid), dim3(NT), 0, st, a);
    else (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, ALTOB200_ROUND_RTN, false>, dim3(grid), dim3(NT), 0, st, a);
  } else if (rounding == ALTOB200_ROUND_SR_BITS) {
    constexpr int R = Fmt<FMT>::FP4 ? ALTOB200_ROUND_SR_BITS : ALTOB200_ROUND_RTN;
    constexpr int NT = COL_NT;
    const dim3 grid(gx, (unsigned)ceil_div(a.rows, NT));
    if (rht) (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, R, Fmt<FMT>::FP4>, dim3(grid), dim3(NT), 0, st, a);
    else (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, R, false>, dim3(grid), dim3(NT), 0, st, a);
  } else if (rounding == ALTOB200_ROUND_SR_PHILOX) {
    constexpr int R = Fmt<FMT>::FP4 ? ALTOB200_ROUND_SR_PHILOX : ALTOB200_ROUND_RTN;
    constexpr int NT = COL_NT;
    const dim3 grid(gx, (unsigned)ceil_div(a.rows, NT));
    if (rht) (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, R, Fmt<FMT>::FP4>, dim3(grid), dim3(NT), 0, st, a);
    else (void)launch_after(quantize_colwise_kernel<FMT, IN_BF16, R, false>, dim3(grid), dim3(NT), 0, st, a);
  } else {
    return ALTOB200_EUNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

template <int FMT, bool IN_BF16>
static int launch_2d(const Quant2dArgs& a, int rounding, cudaStream_t st) {
  // one warp per tile of 4 block columns x (64 rows for 16-blocks, 32 rows for 32-blocks)
  constexpr int TC = 4 * Fmt<FMT>::B, TR = 1024 / Fmt<FMT>::B;
  const int64_t tiles = ceil_div(a.cols, TC) * ceil_div(a.rows, TR) * a.batch;
  const unsigned blocks = (unsigned)ceil_div(tiles, 8);
  constexpr int SR = Fmt<FMT>::FP4 ? ALTOB200_ROUND_SR_BITS : ALTOB200_ROUND_RTN;
  const bool batched = a.batch > 1;
  if (rounding == ALTOB200_ROUND_RTN) {
    if (batched) (void)launch_after(quantize_2d_kernel<FMT, IN_BF16, ALTOB200_ROUND_RTN, true>, dim3(blocks), dim3(256), 0, st, a);
    else (void)launch_after(quantize_2d_kernel<FMT, IN_BF16, ALTOB200_ROUND_RTN, false>, dim3(blocks), dim3(256), 0, st, a);
  } else if (rounding == ALTOB200_ROUND_SR_BITS && Fmt<FMT>::FP4) {
    if (batched) (void)launch_after(quantize_2d_kernel<FMT, IN_BF16, SR, true>, dim3(blocks), dim3(256), 0, st, a);
    else (void)launch_after(quantize_2d_kernel<FMT, IN_BF16, SR, false>, dim3(blocks), dim3(256), 0, st, a);
  } else {
    return ALTOB200_EUNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

#define DISPATCH_FMT_DT(fmt, dt, CALL)                                                      \
  do {                                                                                      \
    const bool _bf = (dt) == ALTOB200_DT_BF16;                                              \
    switch (fmt) {                                                                          \
      case ALTOB200_FMT_NVFP4:                                                              \
        return _bf ? CALL(ALTOB200_FMT_NVFP4, true) : CALL(ALTOB200_FMT_NVFP4, false);      \
      case ALTOB200_FMT_MXFP4:                                                              \
        return _bf ? CALL(ALTOB200_FMT_MXFP4, true) : CALL(ALTOB200_FMT_MXFP4, false);      \
      case ALTOB200_FMT_MXFP8_E4M3:                                                         \
        return _bf ? CALL(ALTOB200_FMT_MXFP8_E4M3, true) : CALL(ALTOB200_FMT_MXFP8_E4M3, false); \
      case ALTOB200_FMT_MXFP8_E5M2:                                                         \
        return _bf ? CALL(ALTOB200_FMT_MXFP8_E5M2, true) : CALL(ALTOB200_FMT_MXFP8_E5M2, false); \
      default:                                                                              \
        return ALTOB200_EUNSUPPORTED;                                                       \
    }                                                                                       \
  } while (0)

static int block_of(int fmt) { return fmt == ALTOB200_FMT_NVFP4 ? 16 : 32; }
static bool is_fp4(int fmt) { return fmt == ALTOB200_FMT_NVFP4 || fmt == ALTOB200_FMT_MXFP4; }

// Zero a packed-scale buffer when the tile grid has padding the kernels do not visit.
static int clear_packed_if_padded(void* buf, int64_t rows, int64_t ncols, cudaStream_t st) {
  if (buf == nullptr) return ALTOB200_OK;
  if ((rows & 127) == 0 && (ncols & 3) == 0) return ALTOB200_OK;
  ALTOB200_CUDA_CHECK(cudaMemsetAsync(buf, 0, altob200_packed_scale_bytes(rows, ncols), st));
  return ALTOB200_OK;
}

// The reference's stochastic-rounding words (alto/kernels/fp4/fp4_common/triton_fp4_ops.py:13-19):
// every BLOCK_M x BLOCK_N tile of the quantisation-axis-last view draws
//   r1, r2, _, _ = randint4x(seed, offset + m * (BLOCK_N / 2) + n),  m < BLOCK_M, n < BLOCK_N / 2
// with tile-local m, n and the SAME offset in every tile, r1 for the even and r2 for the odd
// element of pair n.  The words therefore form one [2][BLOCK_M][BLOCK_N/2] table that repeats over
// the matrix; this kernel writes the table (one Philox call per entry pair) and the quantizers index
// it periodically.
__global__ void __launch_bounds__(256) philox_tile_kernel(uint32_t* out, int64_t tile_rows, int64_t tile_pairs,
                                                          uint32_t offset, PhiloxKeys pk) {
  grid_dependency_wait();
  const int64_t n = tile_rows * tile_pairs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t o[4];
    // Triton's randint4x on an int32 offset tensor: counter = (uint32(offset + i), 0, 0, 0)
    philox4x32_10_keys(offset + (uint32_t)i, 0u, pk, o);
    out[i] = o[0];
    out[n + i] = o[1];
  }
}

// clip_mode / use_uos exist for MXFP4 only, as in the reference
static int fill_mx_opts(MxOpts* o, const altob200_quant_params* p, bool allow_dynamic) {
  o->clip = p->clip_mode;
  o->uos = p->use_uos != 0 ? 1 : 0;
  if (o->clip < ALTOB200_CLIP_NONE || o->clip > ALTOB200_CLIP_DYNAMIC) return ALTOB200_EINVAL_SHAPE;
  if ((o->clip | o->uos) != 0 && p->format != ALTOB200_FMT_MXFP4) return ALTOB200_EUNSUPPORTED;
  if (o->clip == ALTOB200_CLIP_DYNAMIC && !allow_dynamic) return ALTOB200_EUNSUPPORTED;
  return ALTOB200_OK;
}

}  // namespace altob200

using namespace altob200;

extern "C" {

int altob200_version(void) { return 1; }

const char* altob200_status_string(int status) {
  switch (status) {
    case ALTOB200_OK: return "ok";
    case ALTOB200_EINVAL_SHAPE: return "invalid shape or size contract";
    case ALTOB200_EINVAL_ALIGN: return "misaligned pointer or leading dimension";
    case ALTOB200_ETIMEOUT_DEVICE: return "bounded device-side wait timed out";
    case ALTOB200_ECUDA: return "CUDA call failed";
    case ALTOB200_EUNSUPPORTED: return "unsupported configuration";
    case ALTOB200_ELIMIT: return "size exceeds a fixed maximum";
    default: return "unknown status";
  }
}

size_t altob200_packed_scale_bytes(int64_t rows, int64_t ncols) {
  return (size_t)(ceil_div(rows, 128) * ceil_div(ncols, 4) * 512);
}

int altob200_philox_tile(uint64_t seed, uint64_t offset, int64_t tile_rows, int64_t tile_pairs, uint32_t* out,
                         void* stream) {
  if (out == nullptr || tile_rows <= 0 || tile_pairs <= 0 || tile_rows * tile_pairs > (1ll << 24))
    return ALTOB200_EINVAL_SHAPE;
  if (!aligned16(out)) return ALTOB200_EINVAL_ALIGN;
  PhiloxKeys pk;
  philox_make_keys(seed, &pk);
  const int64_t n = tile_rows * tile_pairs;
  int64_t blocks = ceil_div(n, 256);
  if (blocks > 148) blocks = 148;
  (void)launch_after(philox_tile_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, out, tile_rows, tile_pairs, (uint32_t)offset,
                                                                        pk);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

int altob200_quantize_rowwise(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              const altob200_quant_params* p, void* codes, void* scale_plain,
                              void* scale_packed, void* stream) {
  if (x == nullptr || p == nullptr || codes == nullptr) return ALTOB200_EINVAL_SHAPE;
  const int B = block_of(p->format);
  if (rows <= 0 || cols <= 0 || cols % B != 0 || ld < cols) return ALTOB200_EINVAL_SHAPE;
  const int esz = p->in_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(x) || (ld * esz) % 16 != 0 || !aligned16(codes)) return ALTOB200_EINVAL_ALIGN;
  if (p->rounding == ALTOB200_ROUND_SR_BITS && (p->rand_bits == nullptr || !aligned16(p->rand_bits)))
    return ALTOB200_EINVAL_ALIGN;
  if (p->rht_n != 0) return ALTOB200_EUNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  RowwiseArgs a;
  a.x = x; a.rows = rows; a.cols = cols; a.ld = ld;
  a.codes = (uint8_t*)codes; a.scale_plain = scale_plain; a.scale_packed = (uint8_t*)scale_packed;
  a.ncol_tiles = ceil_div(cols / B, 4);
  a.outer = p->outer_scale; a.rand_bits = p->rand_bits;
  a.tile_rows = p->rand_tile_rows; a.tile_pairs = p->rand_tile_pairs;
  if ((a.tile_rows != 0) != (a.tile_pairs != 0) || a.tile_rows < 0 || a.tile_pairs % 8 != 0)
    return ALTOB200_EINVAL_SHAPE;
  if (a.tile_rows != 0 && (rows >= (1ll << 32) || cols >= (1ll << 32))) return ALTOB200_ELIMIT;
  a.philox_seed = p->philox_seed; a.philox_offset = p->philox_offset;
  philox_make_keys(p->philox_seed, &a.pk);
  int rc = fill_mx_opts(&a.mx, p, true);
  if (rc != ALTOB200_OK) return rc;
  rc = clear_packed_if_padded(scale_packed, rows, cols / B, st);
  if (rc != ALTOB200_OK) return rc;
  const int rounding = p->rounding;
#define CALL_ROW(F, BF) launch_rowwise<F, BF>(a, rounding, st)
  DISPATCH_FMT_DT(p->format, p->in_dtype, CALL_ROW);
#undef CALL_ROW
}

int altob200_quantize_colwise(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              const altob200_quant_params* p, void* codes, void* scale_plain,
                              void* scale_packed, void* stream) {
  if (x == nullptr || p == nullptr || codes == nullptr) return ALTOB200_EINVAL_SHAPE;
  const int B = block_of(p->format);
  if (rows <= 0 || cols <= 0 || rows % B != 0 || cols % 8 != 0 || ld < cols) return ALTOB200_EINVAL_SHAPE;
  if (p->rht_n != 0 && rows % p->rht_n != 0) return ALTOB200_EINVAL_SHAPE;
  // every output row must start on a 16-byte boundary
  const int64_t out_row_bytes = is_fp4(p->format) ? rows / 2 : rows;
  if (out_row_bytes % 8 != 0) return ALTOB200_EINVAL_SHAPE;
  const int esz = p->in_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(x) || (ld * esz) % 16 != 0 || !aligned16(codes) || out_row_bytes % 16 != 0)
    return ALTOB200_EINVAL_ALIGN;
  if (p->rounding == ALTOB200_ROUND_SR_BITS && p->rand_bits == nullptr) return ALTOB200_EINVAL_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  ColwiseArgs a;
  a.x = x; a.rows = rows; a.cols = cols; a.ld = ld;
  a.codes = (uint8_t*)codes; a.scale_plain = scale_plain; a.scale_packed = (uint8_t*)scale_packed;
  a.ncol_tiles = ceil_div(rows / B, 4);
  a.outer = p->outer_scale; a.rand_bits = p->rand_bits;
  a.tile_rows = p->rand_tile_rows; a.tile_pairs = p->rand_tile_pairs;
  if ((a.tile_rows != 0) != (a.tile_pairs != 0) || a.tile_rows < 0 || a.tile_pairs < 0) return ALTOB200_EINVAL_SHAPE;
  if (a.tile_rows != 0 && (rows >= (1ll << 32) || cols >= (1ll << 32) || a.tile_rows >= (1ll << 32) ||
                           a.tile_pairs >= (1ll << 32)))
    return ALTOB200_ELIMIT;
  a.philox_seed = p->philox_seed; a.philox_offset = p->philox_offset;
  philox_make_keys(p->philox_seed, &a.pk);
  int rc = fill_rht(&a.rht, p->rht_n, p->rht_perm, p->rht_sign);
  if (rc != ALTOB200_OK) return rc;
  fill_rht_row_offsets(&a.rht, ld, p->in_dtype == ALTOB200_DT_BF16 ? 2 : 4);
  rc = fill_mx_opts(&a.mx, p, true);
  if (rc != ALTOB200_OK) return rc;
  rc = clear_packed_if_padded(scale_packed, cols, rows / B, st);
  if (rc != ALTOB200_OK) return rc;
  const int rounding = p->rounding;
#define CALL_COL(F, BF) launch_colwise<F, BF>(a, rounding, st)
  DISPATCH_FMT_DT(p->format, p->in_dtype, CALL_COL);
#undef CALL_COL
}

int altob200_quantize_2d(const void* w, int64_t rows, int64_t cols, int64_t ld,
                         const altob200_quant_params* p, void* codes_k, void* codes_t,
                         void* scale_plain, void* scale_packed_k, void* scale_packed_t,
                         void* stream) {
  return altob200_quantize_2d_batched(w, 1, rows * ld, rows, cols, ld, p, codes_k, codes_t, scale_plain,
                                      scale_packed_k, scale_packed_t, stream);
}

int altob200_quantize_2d_batched(const void* w, int64_t batch, int64_t batch_stride, int64_t rows, int64_t cols,
                                 int64_t ld, const altob200_quant_params* p, void* codes_k, void* codes_t,
                                 void* scale_plain, void* scale_packed_k, void* scale_packed_t, void* stream) {
  if (w == nullptr || p == nullptr || codes_k == nullptr || batch <= 0) return ALTOB200_EINVAL_SHAPE;
  const int B = block_of(p->format);
  if (rows <= 0 || cols <= 0 || rows % B != 0 || cols % B != 0 || ld < cols) return ALTOB200_EINVAL_SHAPE;
  if (p->rht_n != 0) return ALTOB200_EUNSUPPORTED;
  if (p->rounding != ALTOB200_ROUND_RTN && p->rounding != ALTOB200_ROUND_SR_BITS) return ALTOB200_EUNSUPPORTED;
  if (p->rounding == ALTOB200_ROUND_SR_BITS && (p->rand_bits == nullptr || !aligned16(p->rand_bits)))
    return ALTOB200_EINVAL_SHAPE;
  const int esz = p->in_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(w) || (ld * esz) % 16 != 0 || !aligned16(codes_k)) return ALTOB200_EINVAL_ALIGN;
  if (codes_t != nullptr && !aligned16(codes_t)) return ALTOB200_EINVAL_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  Quant2dArgs a;
  a.w = w; a.rows = rows; a.cols = cols; a.ld = ld;
  a.codes_k = (uint8_t*)codes_k; a.codes_t = (uint8_t*)codes_t; a.scale_plain = scale_plain;
  a.packed_k = (uint8_t*)scale_packed_k; a.packed_t = (uint8_t*)scale_packed_t;
  a.nct_k = ceil_div(cols / B, 4); a.nct_t = ceil_div(rows / B, 4);
  a.batch = batch; a.batch_stride = batch_stride;
  a.packed_k_bytes = altob200_packed_scale_bytes(rows, cols / B);
  a.packed_t_bytes = altob200_packed_scale_bytes(cols, rows / B);
  if (batch > 1 && ((batch_stride * (p->in_dtype == ALTOB200_DT_BF16 ? 2 : 4)) % 16 != 0 ||
                    (rows * (is_fp4(p->format) ? cols / 2 : cols)) % 16 != 0))
    return ALTOB200_EINVAL_ALIGN;
  a.outer = p->outer_scale;
  a.rand_bits = p->rand_bits; a.tile_rows = p->rand_tile_rows; a.tile_pairs = p->rand_tile_pairs;
  if ((a.tile_rows != 0) != (a.tile_pairs != 0) || a.tile_rows < 0 || a.tile_pairs < 0 || (a.tile_pairs & 3) != 0)
    return ALTOB200_EINVAL_SHAPE;
  if (a.tile_rows >= (1ll << 32) || a.tile_pairs >= (1ll << 32)) return ALTOB200_ELIMIT;
  int rc = fill_mx_opts(&a.mx, p, true);
  if (rc != ALTOB200_OK) return rc;
  // padding entries of the packed layouts are zero (the kernel does not visit them)
  if (scale_packed_k != nullptr && ((rows & 127) != 0 || ((cols / B) & 3) != 0))
    ALTOB200_CUDA_CHECK(cudaMemsetAsync(scale_packed_k, 0, (size_t)(batch * a.packed_k_bytes), st));
  if (scale_packed_t != nullptr && ((cols & 127) != 0 || ((rows / B) & 3) != 0))
    ALTOB200_CUDA_CHECK(cudaMemsetAsync(scale_packed_t, 0, (size_t)(batch * a.packed_t_bytes), st));
  const int rounding = p->rounding;
#define CALL_2D(F, BF) launch_2d<F, BF>(a, rounding, st)
  DISPATCH_FMT_DT(p->format, p->in_dtype, CALL_2D);
#undef CALL_2D
}

int altob200_amax(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, int64_t ld,
                  int32_t rht_n, const int32_t* rht_perm, const int32_t* rht_sign,
                  uint32_t* amax_bits, float* outer_scale, void* scratch, void* stream) {
  if (x == nullptr || amax_bits == nullptr || scratch == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || ld < cols) return ALTOB200_EINVAL_SHAPE;
  if (rht_n != 0 && rows % rht_n != 0) return ALTOB200_EINVAL_SHAPE;
  const int esz = in_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(x) || (ld * esz) % 16 != 0) return ALTOB200_EINVAL_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  AmaxArgs a;
  a.x = x; a.rows = rows; a.cols = cols; a.ld = ld;
  a.amax_bits = amax_bits; a.outer_scale = outer_scale; a.counter = (uint32_t*)scratch;
  int rc = fill_rht(&a.rht, rht_n, rht_perm, rht_sign);
  if (rc != ALTOB200_OK) return rc;
  fill_rht_row_offsets(&a.rht, ld, esz);
  const int64_t work = rht_n ? (rows / 16) * ceil_div(cols, 64) / 8 + 1
                             : rows * cols / (16 / esz) / 256 + 1;
  int64_t blocks = work;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const bool bf = in_dtype == ALTOB200_DT_BF16;
  if (rht_n) {
    if (bf) (void)launch_after(amax_kernel<true, true>, dim3((unsigned)blocks), dim3(256), 0, st, a);
    else (void)launch_after(amax_kernel<false, true>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  } else {
    if (bf) (void)launch_after(amax_kernel<true, false>, dim3((unsigned)blocks), dim3(256), 0, st, a);
    else (void)launch_after(amax_kernel<false, false>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  }
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

int altob200_dequantize(const void* codes, const void* scale_plain, const float* outer_scale,
                        int32_t format, int32_t is_2d, int64_t rows, int64_t cols,
                        int32_t out_dtype, void* out, int64_t ld_out, void* stream) {
  if (codes == nullptr || scale_plain == nullptr || out == nullptr) return ALTOB200_EINVAL_SHAPE;
  const int B = block_of(format);
  if (rows <= 0 || cols <= 0 || cols % B != 0 || ld_out < cols) return ALTOB200_EINVAL_SHAPE;
  if ((is_2d & 1) && rows % B != 0) return ALTOB200_EINVAL_SHAPE;
  const int esz = out_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(codes) || !aligned16(out) || (ld_out * esz) % 16 != 0) return ALTOB200_EINVAL_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  DequantArgs a;
  a.codes = (const uint8_t*)codes; a.scales = scale_plain; a.outer = outer_scale;
  a.rows = rows; a.cols = cols; a.ld_out = ld_out; a.out = out; a.is_2d = is_2d & 1;
  a.static_clip = (is_2d >> 1) & 1;
  if (a.static_clip && format != ALTOB200_FMT_MXFP4) return ALTOB200_EUNSUPPORTED;
  int64_t blocks = ceil_div(rows * (cols / 16), 256);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const bool bf = out_dtype == ALTOB200_DT_BF16;
#define LAUNCH_DQ(F)                                                              \
  if (bf) (void)launch_after(dequantize_kernel<F, true>, dim3((unsigned)blocks), dim3(256), 0, st, a);        \
  else (void)launch_after(dequantize_kernel<F, false>, dim3((unsigned)blocks), dim3(256), 0, st, a);          \
  break;
  switch (format) {
    case ALTOB200_FMT_NVFP4: LAUNCH_DQ(ALTOB200_FMT_NVFP4)
    case ALTOB200_FMT_MXFP4: LAUNCH_DQ(ALTOB200_FMT_MXFP4)
    case ALTOB200_FMT_MXFP8_E4M3: LAUNCH_DQ(ALTOB200_FMT_MXFP8_E4M3)
    case ALTOB200_FMT_MXFP8_E5M2: LAUNCH_DQ(ALTOB200_FMT_MXFP8_E5M2)
    default: return ALTOB200_EUNSUPPORTED;
  }
#undef LAUNCH_DQ
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

int altob200_rht(const void* x, int32_t dtype, int64_t rows, int64_t cols, int64_t ld,
                 int32_t rht_n, const int32_t* rht_perm, const int32_t* rht_sign, void* y,
                 int64_t ld_y, void* stream) {
  if (x == nullptr || y == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (rht_n != 16) return ALTOB200_EUNSUPPORTED;
  if (rows <= 0 || cols <= 0 || rows % 16 != 0 || cols % 8 != 0 || ld < cols || ld_y < cols)
    return ALTOB200_EINVAL_SHAPE;
  const int esz = dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(x) || !aligned16(y) || (ld * esz) % 16 != 0 || (ld_y * esz) % 16 != 0)
    return ALTOB200_EINVAL_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  RhtArgs a;
  a.x = x; a.y = y; a.rows = rows; a.cols = cols; a.ld = ld; a.ld_y = ld_y;
  int rc = fill_rht(&a.rht, rht_n, rht_perm, rht_sign);
  if (rc != ALTOB200_OK) return rc;
  int64_t blocks = (rows / 16) * ceil_div(cols, 64) / 8 + 1;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (dtype == ALTOB200_DT_BF16) (void)launch_after(rht_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  else (void)launch_after(rht_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

int altob200_amax_noalloc(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, int64_t ld,
                          uint32_t* amax_bits, float* outer_scale, void* stream) {
  if (x == nullptr || amax_bits == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || ld < cols) return ALTOB200_EINVAL_SHAPE;
  if (in_dtype != ALTOB200_DT_BF16 && in_dtype != ALTOB200_DT_F32) return ALTOB200_EUNSUPPORTED;
  const int esz = in_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if (!aligned16(x) || (ld * esz) % 16 != 0) return ALTOB200_EINVAL_ALIGN;
  // the fixed array has one slot per block of 64 KiB of input
  if (rows > ALTOB200_NOALLOC_MAX_BYTES / esz / cols) return ALTOB200_ELIMIT;
  // Set-up, once per device, with that device current: the array's name is only a host-side
  // handle, the kernel needs the device address behind it.
  // The cache is atomic because the first calls on a device may come from two host threads at
  // once (they would store the same address).  The address stays valid for the life of the
  // device's context; after cudaDeviceReset it must not be used, so a process that resets a
  // device must not call this entry point on it again.
  static std::atomic<void*> scratch_of_device[64];
  int dev = 0;
  ALTOB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ALTOB200_ELIMIT;
  void* cached = scratch_of_device[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* ptr = nullptr;
    ALTOB200_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return ALTOB200_ECUDA;
    scratch_of_device[dev].store(ptr, std::memory_order_release);
    cached = ptr;
  }
  NoallocScratch* scratch = reinterpret_cast<NoallocScratch*>(cached);
  cudaStream_t st = (cudaStream_t)stream;
  // the counter must start at zero even if an earlier launch never finished
  ALTOB200_CUDA_CHECK(cudaMemsetAsync(&scratch->counter, 0, sizeof(uint32_t), st));
  AmaxNoallocArgs a;
  a.x = x; a.rows = rows; a.cols = cols; a.ld = ld;
  a.amax_bits = amax_bits; a.outer_scale = outer_scale; a.scratch = scratch;
  const int64_t total_vec = rows * (cols / (16 / esz));
  const int64_t blocks = ceil_div(total_vec, 256 * NOALLOC_VEC_PER_THREAD);
  if (blocks > NOALLOC_MAX_BLOCKS) return ALTOB200_ELIMIT;
  if (in_dtype == ALTOB200_DT_BF16) amax_noalloc_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(a);
  else amax_noalloc_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

}  // extern "C"
