// Macro-block (128) two-level scaling and descaling.
//
// Per block of 128 elements along the last axis of each row (1D) or per 128 x 128 tile (2D):
//   amax  = max(|x| as fp32, 1e-12)
//   bits  = fp32 bits of (6.0 / amax) & 0x007F8000      (the top 8 mantissa bits)
//   code  = bits >> 15                                   (uint8, stored)
//   s     = float(bits | 127 << 23)                      (a factor in [1, 2))
//   y     = cast(x * s)     descaling:  x = cast(y / float(code << 15 | 127 << 23))
// which restates the reference's Triton kernels (fp32 multiply, then the cast)
//   alto/kernels/fp4/mxfp4/macro_block_scaling.py:35-96 and :100-146.
// Elements past the end of a ragged last block do not take part in the amax.
//
// Work layout: 1D - a warp task is 4 rows x 256 columns: a lane holds 8 contiguous elements of
// each row (all loads issued before the first is used), a block is 16 lanes wide and its maximum
// a half-warp shuffle reduction (rows that do not allow 8-wide accesses take a one-block-per-warp
// variant with 4 elements per lane).  2D - a CTA of 256 threads owns one tile, a warp 16 rows; the
// tile maximum goes through shared memory.  Both are one read and one write per element.
#include "common.cuh"

namespace altob200 {

struct MacroArgs {
  const void* x;       // [batch, rows, cols] contiguous
  void* y;             // same shape
  uint8_t* scale;      // 1D: [batch, rows, nblk]   2D: [batch, ceil(rows/128), nblk]
  int64_t batch, rows, cols, nblk;
  int vec;             // rows start on a 4-element boundary: 4-wide loads and stores are legal
  int wide;            // rows are a multiple of 8 elements and 32-byte (fp32) / 16-byte (bf16) aligned
};

__device__ __forceinline__ float macro_factor_from_amax(float amax, uint32_t* code) {
  amax = fmaxf(amax, 1e-12f);
  const uint32_t bits = f2u(__fdiv_rn(6.0f, amax)) & 0x007F8000u;
  *code = bits >> 15;
  return u2f(bits + (127u << 23));
}
__device__ __forceinline__ float macro_factor_from_code(uint32_t code) { return u2f((code << 15) + (127u << 23)); }

template <bool IN_BF16>
__device__ __forceinline__ void load4(const void* base, int64_t off, int valid, bool vec, float v[4]) {
  // `valid` elements (0..4) starting at element offset `off` exist; the rest read as zero
  if (valid == 4 && vec) {
    if (IN_BF16) {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + off));
      v[0] = bf16lo_to_f32(w.x); v[1] = bf16hi_to_f32(w.x); v[2] = bf16lo_to_f32(w.y); v[3] = bf16hi_to_f32(w.y);
    } else {
      const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = 0.0f;
      if (j < valid) {
        if (IN_BF16) v[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off + j]);
        else v[j] = reinterpret_cast<const float*>(base)[off + j];
      }
    }
  }
}

template <bool IN_BF16>
__device__ __forceinline__ void store4(void* base, int64_t off, int valid, bool vec, const float v[4]) {
  if (valid == 4 && vec) {
    if (IN_BF16) {
      const uint32_t a = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
      const uint32_t b = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = make_uint2(a, b);
    } else {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else {
    for (int j = 0; j < valid; ++j) {
      if (IN_BF16) reinterpret_cast<__nv_bfloat16*>(base)[off + j] = __float2bfloat16_rn(v[j]);
      else reinterpret_cast<float*>(base)[off + j] = v[j];
    }
  }
}

__device__ __forceinline__ float warp_max_f32(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// ---- 1D: one warp per (row, 128-column block) ----
template <bool IN_BF16, bool DESCALE>
__global__ void __launch_bounds__(256) macro_scale_1d_kernel(MacroArgs a) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t n_tasks = a.batch * a.rows * a.nblk;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
  for (int64_t task = warp0; task < n_tasks; task += n_warps) {
    const int64_t row = task / a.nblk, blk = task - row * a.nblk;  // row counts over batch * rows
    const int64_t col = blk * 128 + lane * 4;
    int valid = (int)(a.cols - col);
    valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
    float v[4];
    load4<IN_BF16>(a.x, row * a.cols + col, valid, a.vec, v);
    float f;
    if (DESCALE) {
      f = macro_factor_from_code(a.scale[row * a.nblk + blk]);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __fdiv_rn(v[j], f);
    } else {
      float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
      m = warp_max_f32(m);
      uint32_t code;
      f = macro_factor_from_amax(m, &code);
      if (lane == 0) a.scale[row * a.nblk + blk] = (uint8_t)code;
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(v[j], f);
    }
    store4<IN_BF16>(a.y, row * a.cols + col, valid, a.vec, v);
  }
}

// ---- 1D, rows of a multiple of 8 elements: a warp task is 4 rows x 256 columns ----
template <bool IN_BF16, bool DESCALE>
__global__ void __launch_bounds__(256) macro_scale_1d_wide_kernel(MacroArgs a) {
  grid_dependency_wait();
  constexpr int R = 4;
  const int lane = threadIdx.x & 31;
  const int64_t n_rows = a.batch * a.rows;
  const int64_t chunks = (a.cols + 255) >> 8;
  const int64_t n_tasks = ((n_rows + R - 1) / R) * chunks;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
  for (int64_t task = warp0; task < n_tasks; task += n_warps) {
    const int64_t rg = task / chunks, chunk = task - rg * chunks;
    const int64_t row0 = rg * R;
    const int64_t col = (chunk << 8) + lane * 8;
    const int64_t blk = (chunk << 1) + (lane >> 4);
    const bool col_ok = col < a.cols;   // cols is a multiple of 8: a lane's 8 elements exist together
    float v[R][8];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const bool ok = col_ok && row0 + i < n_rows;
      const int64_t off = (row0 + i) * a.cols + col;
      if (IN_BF16) {
        const uint4 w = ok ? __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.x) + off))
                           : make_uint4(0u, 0u, 0u, 0u);
        v[i][0] = bf16lo_to_f32(w.x); v[i][1] = bf16hi_to_f32(w.x); v[i][2] = bf16lo_to_f32(w.y); v[i][3] = bf16hi_to_f32(w.y);
        v[i][4] = bf16lo_to_f32(w.z); v[i][5] = bf16hi_to_f32(w.z); v[i][6] = bf16lo_to_f32(w.w); v[i][7] = bf16hi_to_f32(w.w);
      } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + off);
        const float4 f0 = ok ? __ldg(p) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 f1 = ok ? __ldg(p + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[i][0] = f0.x; v[i][1] = f0.y; v[i][2] = f0.z; v[i][3] = f0.w;
        v[i][4] = f1.x; v[i][5] = f1.y; v[i][6] = f1.z; v[i][7] = f1.w;
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int64_t row = row0 + i;
      const bool ok = col_ok && row < n_rows;
      float f;
      if (DESCALE) {
        f = macro_factor_from_code(ok ? a.scale[row * a.nblk + blk] : 0u);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __fdiv_rn(v[i][j], f);
      } else {
        float m = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[i][j]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        uint32_t code;
        f = macro_factor_from_amax(m, &code);
        if (ok && (lane & 15) == 0) a.scale[row * a.nblk + blk] = (uint8_t)code;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __fmul_rn(v[i][j], f);
      }
      if (ok) {
        const int64_t off = row * a.cols + col;
        if (IN_BF16) {
          uint4 o;
          o.x = f32_to_bf16_bits(v[i][0]) | (f32_to_bf16_bits(v[i][1]) << 16);
          o.y = f32_to_bf16_bits(v[i][2]) | (f32_to_bf16_bits(v[i][3]) << 16);
          o.z = f32_to_bf16_bits(v[i][4]) | (f32_to_bf16_bits(v[i][5]) << 16);
          o.w = f32_to_bf16_bits(v[i][6]) | (f32_to_bf16_bits(v[i][7]) << 16);
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + off) = o;
        } else {
          float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + off);
          p[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          p[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
      }
    }
  }
}

// ---- 2D and column blocks: one CTA per 128 x 128 tile ----
// COLS = false: one factor per tile.  COLS = true: one factor per column of the tile (blocks of
// 128 run down the rows, the reference's axis=0 on a matrix); scale is [batch, cols, ceil(rows/128)].
template <bool IN_BF16, bool DESCALE, bool COLS>
__global__ void __launch_bounds__(256) macro_scale_tile_kernel(MacroArgs a) {
  grid_dependency_wait();
  __shared__ float s_max[COLS ? 8 * 128 : 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.z, tm = blockIdx.y, tn = blockIdx.x;
  const int64_t mtiles = (a.rows + 127) / 128;
  const int64_t col = tn * 128 + lane * 4;
  int valid = (int)(a.cols - col);
  valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
  float v[16][4];
  float cm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = tm * 128 + warp * 16 + i;
    const int vr = r < a.rows ? valid : 0;
    load4<IN_BF16>(a.x, (b * a.rows + (r < a.rows ? r : 0)) * a.cols + col, vr, a.vec, v[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) cm[j] = fmaxf(cm[j], fabsf(v[i][j]));
  }
  float f[4];
  if (COLS) {
    // factor index: [batch, cols, mtiles]
    if (DESCALE) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        f[j] = j < valid ? macro_factor_from_code(a.scale[(b * a.cols + col + j) * mtiles + tm]) : 1.0f;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) s_max[warp * 128 + lane * 4 + j] = cm[j];
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float t = s_max[lane * 4 + j];
#pragma unroll
        for (int w = 1; w < 8; ++w) t = fmaxf(t, s_max[w * 128 + lane * 4 + j]);
        uint32_t code;
        f[j] = macro_factor_from_amax(t, &code);
        if (warp == 0 && j < valid) a.scale[(b * a.cols + col + j) * mtiles + tm] = (uint8_t)code;
      }
    }
  } else {
    const int64_t sidx = (b * mtiles + tm) * a.nblk + tn;
    float ft;
    if (DESCALE) {
      ft = macro_factor_from_code(a.scale[sidx]);
    } else {
      float m = warp_max_f32(fmaxf(fmaxf(cm[0], cm[1]), fmaxf(cm[2], cm[3])));
      if (lane == 0) s_max[warp] = m;
      __syncthreads();
      float t = s_max[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) t = fmaxf(t, s_max[i]);
      uint32_t code;
      ft = macro_factor_from_amax(t, &code);
      if (threadIdx.x == 0) a.scale[sidx] = (uint8_t)code;
    }
    f[0] = f[1] = f[2] = f[3] = ft;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = tm * 128 + warp * 16 + i;
    if (r >= a.rows) break;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[i][j] = DESCALE ? __fdiv_rn(v[i][j], f[j]) : __fmul_rn(v[i][j], f[j]);
    store4<IN_BF16>(a.y, (b * a.rows + r) * a.cols + col, valid, a.vec, v[i]);
  }
}

// ---- 2D and column blocks, bf16 with 4-wide accesses: the tile stays packed in registers ----
// Same work split as above (a warp 16 rows, a lane 4 columns), but the 16 x 4 elements are kept as
// the 32 words they were loaded as and the maxima are taken on the packed bit patterns (|bf16| orders
// like its integer bits), which leaves room for four CTAs per SM instead of two: the kernel is a plain
// stream, and what limits it is the number of bytes in flight.
template <bool DESCALE, bool COLS>
__global__ void __launch_bounds__(256, 4) macro_scale_tile_bf16_kernel(MacroArgs a) {
  grid_dependency_wait();
  __shared__ __align__(16) uint2 s_max[COLS ? 8 * 32 : 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.z, tm = blockIdx.y, tn = blockIdx.x;
  const int64_t mtiles = (a.rows + 127) / 128;
  const int64_t col = tn * 128 + lane * 4;
  const bool col_ok = col < a.cols;   // cols is a multiple of 4: a lane's 4 elements exist together
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.x);
  uint2 raw[16];
  uint2 acc = make_uint2(0u, 0u);     // packed per-column maxima of |x| bit patterns
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = tm * 128 + warp * 16 + i;
    raw[i] = (col_ok && r < a.rows) ? __ldg(reinterpret_cast<const uint2*>(src + (b * a.rows + r) * a.cols + col))
                                    : make_uint2(0u, 0u);
    acc.x = __vmaxu2(acc.x, raw[i].x & 0x7FFF7FFFu);
    acc.y = __vmaxu2(acc.y, raw[i].y & 0x7FFF7FFFu);
  }
  float f[4];
  if (COLS) {
    if (DESCALE) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        f[j] = col_ok ? macro_factor_from_code(a.scale[(b * a.cols + col + j) * mtiles + tm]) : 1.0f;
    } else {
      s_max[warp * 32 + lane] = acc;
      __syncthreads();
      uint2 t = s_max[lane];
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        const uint2 o = s_max[w * 32 + lane];
        t.x = __vmaxu2(t.x, o.x);
        t.y = __vmaxu2(t.y, o.y);
      }
      const float m[4] = {u2f(t.x << 16), u2f(t.x & 0xFFFF0000u), u2f(t.y << 16), u2f(t.y & 0xFFFF0000u)};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t code;
        f[j] = macro_factor_from_amax(m[j], &code);
        if (warp == 0 && col_ok) a.scale[(b * a.cols + col + j) * mtiles + tm] = (uint8_t)code;
      }
    }
  } else {
    const int64_t sidx = (b * mtiles + tm) * a.nblk + tn;
    float ft;
    if (DESCALE) {
      ft = macro_factor_from_code(a.scale[sidx]);
    } else {
      uint32_t m2 = __vmaxu2(acc.x, acc.y);
      m2 = __vmaxu2(m2, m2 >> 16) & 0xFFFFu;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const uint32_t t = __shfl_xor_sync(0xFFFFFFFFu, m2, o);
        m2 = t > m2 ? t : m2;
      }
      if (lane == 0) s_max[warp].x = m2;
      __syncthreads();
      uint32_t t = s_max[0].x;
#pragma unroll
      for (int i = 1; i < 8; ++i) t = s_max[i].x > t ? s_max[i].x : t;
      uint32_t code;
      ft = macro_factor_from_amax(u2f(t << 16), &code);
      if (threadIdx.x == 0) a.scale[sidx] = (uint8_t)code;
    }
    f[0] = f[1] = f[2] = f[3] = ft;
  }
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y);
  if (!col_ok) return;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = tm * 128 + warp * 16 + i;
    if (r >= a.rows) break;
    float v[4] = {bf16lo_to_f32(raw[i].x), bf16hi_to_f32(raw[i].x), bf16lo_to_f32(raw[i].y), bf16hi_to_f32(raw[i].y)};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = DESCALE ? __fdiv_rn(v[j], f[j]) : __fmul_rn(v[j], f[j]);
    const uint32_t lo = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
    const uint32_t hi = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
    *reinterpret_cast<uint2*>(dst + (b * a.rows + r) * a.cols + col) = make_uint2(lo, hi);
  }
}

template <bool BF, bool DESCALE>
static void launch_mode(const MacroArgs& a, int32_t mode, cudaStream_t st) {
  if (mode == 0) {
    if (a.wide) {
      int64_t blocks = ceil_div(ceil_div(a.batch * a.rows, 4) * ceil_div(a.cols, 256), 8);
      if (blocks > 148 * 8) blocks = 148 * 8;
      (void)launch_after(macro_scale_1d_wide_kernel<BF, DESCALE>, dim3((unsigned)blocks), dim3(256), 0, st, a);
      return;
    }
    int64_t blocks = ceil_div(a.batch * a.rows * a.nblk, 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    (void)launch_after(macro_scale_1d_kernel<BF, DESCALE>, dim3((unsigned)blocks), dim3(256), 0, st, a);
  } else {
    dim3 grid((unsigned)a.nblk, (unsigned)ceil_div(a.rows, 128), (unsigned)a.batch);
    if (BF && a.vec) {
      if (mode == 1) (void)launch_after(macro_scale_tile_bf16_kernel<DESCALE, false>, dim3(grid), dim3(256), 0, st, a);
      else (void)launch_after(macro_scale_tile_bf16_kernel<DESCALE, true>, dim3(grid), dim3(256), 0, st, a);
      return;
    }
    if (mode == 1) (void)launch_after(macro_scale_tile_kernel<BF, DESCALE, false>, dim3(grid), dim3(256), 0, st, a);
    else (void)launch_after(macro_scale_tile_kernel<BF, DESCALE, true>, dim3(grid), dim3(256), 0, st, a);
  }
}

static int macro_launch(const void* x, int32_t dtype, int64_t batch, int64_t rows, int64_t cols, int32_t mode,
                        void* y, uint8_t* scale, bool descale, cudaStream_t st) {
  if (x == nullptr || y == nullptr || scale == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (batch <= 0 || rows <= 0 || cols <= 0) return ALTOB200_EINVAL_SHAPE;
  if (dtype != ALTOB200_DT_BF16 && dtype != ALTOB200_DT_F32) return ALTOB200_EUNSUPPORTED;
  MacroArgs a;
  // 4-wide accesses need every row to start on a 4-element boundary; otherwise element accesses
  a.vec = (cols % 4 == 0) && !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15);
  a.wide = (cols % 8 == 0) && !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15);
  a.x = x; a.y = y; a.scale = scale; a.batch = batch; a.rows = rows; a.cols = cols; a.nblk = ceil_div(cols, 128);
  if (mode < 0 || mode > 2) return ALTOB200_EUNSUPPORTED;
  if (mode != 0 && (ceil_div(rows, 128) > 65535 || batch > 65535)) return ALTOB200_ELIMIT;
  if (dtype == ALTOB200_DT_BF16) {
    if (descale) launch_mode<true, true>(a, mode, st); else launch_mode<true, false>(a, mode, st);
  } else {
    if (descale) launch_mode<false, true>(a, mode, st); else launch_mode<false, false>(a, mode, st);
  }
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

}  // namespace altob200

extern "C" {

int altob200_macro_block_scaling(const void* x, int32_t dtype, int64_t batch, int64_t rows, int64_t cols,
                                 int32_t mode, void* y, uint8_t* scale, void* stream) {
  return altob200::macro_launch(x, dtype, batch, rows, cols, mode, y, scale, false, (cudaStream_t)stream);
}

int altob200_macro_block_descaling(const void* y, const uint8_t* scale, int32_t dtype, int64_t batch, int64_t rows,
                                   int64_t cols, int32_t mode, void* x, void* stream) {
  return altob200::macro_launch(y, dtype, batch, rows, cols, mode, x, const_cast<uint8_t*>(scale), true,
                                (cudaStream_t)stream);
}

}  // extern "C"
