// Block Hadamard-type transform with an arbitrary n x n matrix:
//   y[g*n + i, c] = cast( (sum_j W[i, j] * x[g*n + j, c]) * (1 / sqrt(n)) )      n in {16, 32, 64}
//
// The reference's transform (alto/kernels/hadamard_transform/transform.py:115-142, left_mul=True)
// is a batched fp32 matmul with W = weight[perm][:, perm] followed by a division by sqrt(n) held in
// a 0-dim tensor, then the cast back to the input dtype.  On CUDA, PyTorch evaluates a division by
// such a scalar as a multiplication by its fp32 reciprocal; the kernel does the same.  The fused
// quantizer kernels cover the Sylvester-16 case with an in-register butterfly; this kernel serves
// every other matrix (the reference's default block size 32 uses a table matrix that is not of
// Sylvester type), at n multiply-adds per element.
//
// A thread owns two adjacent columns of one n-row block: the 2n inputs sit in registers as pairs, so
// that one packed fp32 multiply-add (fma.rn.f32x2) serves both columns; W is read from shared memory
// four entries at a time (all threads of a warp read the same address), every output row is
// produced, scaled, converted and stored at once.  Exact while the partial sums are
// exact (entries of W are +-1); the accumulation order is j = 0 .. n-1.
#include <math.h>

#include "common.cuh"

namespace altob200 {

struct RhtDenseArgs {
  const void* x;
  void* y;
  const float* w;        // device, n x n row-major
  int64_t rows, cols, ld, ld_y;
  float inv_scale;       // fp32(1 / fp32(sqrt(n)))
};

template <int N, bool IN_BF16>
__global__ void __launch_bounds__(128) rht_dense_kernel(RhtDenseArgs a) {
  __shared__ __align__(16) float s_w[N * N];
  for (int i = threadIdx.x; i < N * N; i += 128) s_w[i] = a.w[i];
  __syncthreads();
  const int64_t groups = a.rows / N;
  const int64_t col_tiles = (a.cols + 255) >> 8;
  const int64_t n_tasks = groups * col_tiles;
  for (int64_t task = blockIdx.x; task < n_tasks; task += gridDim.x) {
    const int64_t g = task / col_tiles, ct = task - g * col_tiles;
    const int64_t c = (ct << 8) + 2 * threadIdx.x;
    if (c >= a.cols) continue;
    const bool two = c + 1 < a.cols;
    float2 xs[N];   // the two columns of a row side by side: one packed multiply-add serves both
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int64_t off = (g * N + j) * a.ld + c;
      if (IN_BF16) {
        const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(a.x) + off;
        if (two) {
          const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(p));
          xs[j] = make_float2(bf16lo_to_f32(w), bf16hi_to_f32(w));
        } else {
          xs[j] = make_float2(__bfloat162float(*p), 0.0f);
        }
      } else {
        const float* p = reinterpret_cast<const float*>(a.x) + off;
        xs[j] = make_float2(__ldg(p), two ? __ldg(p + 1) : 0.0f);
      }
    }
#pragma unroll 2
    for (int i = 0; i < N; ++i) {
      float2 acc = make_float2(0.0f, 0.0f);
      const float4* wr = reinterpret_cast<const float4*>(s_w + i * N);
#pragma unroll
      for (int q = 0; q < N / 4; ++q) {
        const float4 w = wr[q];
        acc = __ffma2_rn(make_float2(w.x, w.x), xs[4 * q], acc);
        acc = __ffma2_rn(make_float2(w.y, w.y), xs[4 * q + 1], acc);
        acc = __ffma2_rn(make_float2(w.z, w.z), xs[4 * q + 2], acc);
        acc = __ffma2_rn(make_float2(w.w, w.w), xs[4 * q + 3], acc);
      }
      // adding +0.0 turns a -0.0 sum into +0.0, as the matmul's accumulation from zero does
      const float y0 = __fmul_rn(__fadd_rn(acc.x, 0.0f), a.inv_scale);
      const float y1 = __fmul_rn(__fadd_rn(acc.y, 0.0f), a.inv_scale);
      const int64_t off = (g * N + i) * a.ld_y + c;
      if (IN_BF16) {
        __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(a.y) + off;
        if (two) *reinterpret_cast<uint32_t*>(p) = f32_to_bf16_bits(y0) | (f32_to_bf16_bits(y1) << 16);
        else *p = __float2bfloat16_rn(y0);
      } else {
        float* p = reinterpret_cast<float*>(a.y) + off;
        p[0] = y0;
        if (two) p[1] = y1;
      }
    }
  }
}

template <int N>
static void launch_rht_dense(const RhtDenseArgs& a, bool bf16, cudaStream_t st) {
  const int64_t n_tasks = (a.rows / N) * ((a.cols + 255) >> 8);
  int64_t blocks = n_tasks < 148 * 8 ? n_tasks : 148 * 8;
  if (blocks < 1) blocks = 1;
  if (bf16) rht_dense_kernel<N, true><<<(unsigned)blocks, 128, 0, st>>>(a);
  else rht_dense_kernel<N, false><<<(unsigned)blocks, 128, 0, st>>>(a);
}

}  // namespace altob200

extern "C" int altob200_rht_dense(const void* x, int32_t dtype, int64_t rows, int64_t cols, int64_t ld, int32_t n,
                                  const float* w, void* y, int64_t ld_y, void* stream) {
  using namespace altob200;
  if (x == nullptr || y == nullptr || w == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (n != 16 && n != 32 && n != 64) return ALTOB200_EUNSUPPORTED;
  if (rows <= 0 || cols <= 0 || rows % n != 0 || ld < cols || ld_y < cols) return ALTOB200_EINVAL_SHAPE;
  if (dtype != ALTOB200_DT_BF16 && dtype != ALTOB200_DT_F32) return ALTOB200_EUNSUPPORTED;
  // bf16: two adjacent columns are accessed as one 4-byte word
  if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(y) & 3)) return ALTOB200_EINVAL_ALIGN;
  if (dtype == ALTOB200_DT_BF16 && (ld % 2 || ld_y % 2)) return ALTOB200_EINVAL_ALIGN;
  RhtDenseArgs a;
  a.x = x; a.y = y; a.w = w; a.rows = rows; a.cols = cols; a.ld = ld; a.ld_y = ld_y;
  a.inv_scale = 1.0f / (float)sqrt((double)n);
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf16 = dtype == ALTOB200_DT_BF16;
  if (n == 16) launch_rht_dense<16>(a, bf16, st);
  else if (n == 32) launch_rht_dense<32>(a, bf16, st);
  else launch_rht_dense<64>(a, bf16, st);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
