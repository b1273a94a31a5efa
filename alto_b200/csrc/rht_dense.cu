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
  grid_dependency_wait();
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

// ---------------------------------------------------------------------------------------
// n = 32, bf16: the same transform on the tensor cores.  The matrix has entries +-1 (exact in bf16),
// the inputs are bf16, so every product is exact and the fp32 accumulation is exact under the same
// condition as the multiply-add chain above (partial sums representable in fp32).  At 32 multiply-adds
// per element the kernel above is bound by the FP32 pipes (0.43 ms for the 67712 x 2880 activations
// of the MoE configuration, 40 % of the FP32 rate); as `mma.sync.m16n8k16` the arithmetic is free and
// the kernel becomes a stream.
//
// A warp owns 32 rows x 64 columns: it copies them into its private part of a shared-memory tile,
// takes the B fragments with `ldmatrix.trans` (the tile is row-major [k][n]), multiplies by the
// 32 x 32 matrix held as A fragments in registers, writes the bf16 results over the tile and
// copies it out with 16-byte stores.  Nothing is shared between warps, so no block barrier.
// ---------------------------------------------------------------------------------------
constexpr int MMA_PITCH = (256 + 8) * 2;   // bytes per tile row: 16-byte aligned, 16 bytes off a multiple of 128

__device__ __forceinline__ uint32_t pack_bf16_exact(float lo, float hi) {
  return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}

__global__ void __launch_bounds__(128) rht32_mma_kernel(RhtDenseArgs a) {
  grid_dependency_wait();
  __shared__ __align__(16) uint8_t s_tile[32 * MMA_PITCH];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // A fragments of W (two 16-row tiles x two 16-column tiles), mma.m16n8k16 row-major layout
  uint32_t fa[2][2][4];
  {
    const int r = lane >> 2, c2 = 2 * (lane & 3);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        const float* w = a.w + (mt * 16 + r) * 32 + kt * 16 + c2;
        fa[mt][kt][0] = pack_bf16_exact(w[0], w[1]);
        fa[mt][kt][1] = pack_bf16_exact(w[8 * 32], w[8 * 32 + 1]);
        fa[mt][kt][2] = pack_bf16_exact(w[8], w[9]);
        fa[mt][kt][3] = pack_bf16_exact(w[8 * 32 + 8], w[8 * 32 + 9]);
      }
  }
  const int64_t groups = a.rows / 32;
  const int64_t col_tiles = (a.cols + 255) >> 8;
  const int64_t n_tasks = groups * col_tiles;
  uint8_t* my = s_tile + warp * 128;                     // this warp's 64 columns of every tile row
  const uint32_t my_s = (uint32_t)__cvta_generic_to_shared(my);
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(a.y);
  for (int64_t task = blockIdx.x; task < n_tasks; task += gridDim.x) {
    const int64_t g = task / col_tiles, ct = task - g * col_tiles;
    const int64_t c0 = (ct << 8) + warp * 64;            // first column of this warp
    // ---- global -> shared: 32 rows x 8 chunks of 16 bytes, a row's 128 bytes by 8 consecutive lanes ----
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = i * 4 + (lane >> 3), ch = lane & 7;
      const int64_t c = c0 + ch * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (c < a.cols) v = __ldg(reinterpret_cast<const uint4*>(x + (g * 32 + row) * a.ld + c));
      *reinterpret_cast<uint4*>(my + row * MMA_PITCH + ch * 16) = v;
    }
    __syncwarp();
    // ---- 8 column tiles of 8: B fragments, 4 MMAs, results back into the tile ----
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      uint32_t b[4];   // b[0], b[1]: k 0-15; b[2], b[3]: k 16-31
      const uint32_t addr = my_s + (uint32_t)lane * MMA_PITCH + t * 16;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
      float acc[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                       : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                       : "r"(fa[mt][kt][0]), "r"(fa[mt][kt][1]), "r"(fa[mt][kt][2]), "r"(fa[mt][kt][3]),
                         "r"(b[2 * kt]), "r"(b[2 * kt + 1]));
      }
      __syncwarp();   // every lane's fragment of this column tile has been read
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int r = mt * 16 + (lane >> 2);
        uint8_t* d = my + r * MMA_PITCH + t * 16 + (lane & 3) * 4;
        // adding +0.0 turns a -0.0 sum into +0.0, as the matmul's accumulation from zero does
        *reinterpret_cast<uint32_t*>(d) =
            pack_bf16_exact(__fmul_rn(__fadd_rn(acc[mt][0], 0.0f), a.inv_scale), __fmul_rn(__fadd_rn(acc[mt][1], 0.0f), a.inv_scale));
        *reinterpret_cast<uint32_t*>(d + 8 * MMA_PITCH) =
            pack_bf16_exact(__fmul_rn(__fadd_rn(acc[mt][2], 0.0f), a.inv_scale), __fmul_rn(__fadd_rn(acc[mt][3], 0.0f), a.inv_scale));
      }
    }
    __syncwarp();
    // ---- shared -> global ----
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = i * 4 + (lane >> 3), ch = lane & 7;
      const int64_t c = c0 + ch * 8;
      if (c < a.cols)
        *reinterpret_cast<uint4*>(y + (g * 32 + row) * a.ld_y + c) = *reinterpret_cast<const uint4*>(my + row * MMA_PITCH + ch * 16);
    }
    __syncwarp();   // the tile is free for the next task
  }
}

template <int N>
static void launch_rht_dense(const RhtDenseArgs& a, bool bf16, cudaStream_t st) {
  const int64_t n_tasks = (a.rows / N) * ((a.cols + 255) >> 8);
  int64_t blocks = n_tasks < 148 * 8 ? n_tasks : 148 * 8;
  if (blocks < 1) blocks = 1;
  if (bf16) (void)launch_after(rht_dense_kernel<N, true>, dim3((unsigned)blocks), dim3(128), 0, st, a);
  else (void)launch_after(rht_dense_kernel<N, false>, dim3((unsigned)blocks), dim3(128), 0, st, a);
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
  const bool vec = cols % 8 == 0 && ld % 8 == 0 && ld_y % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                   !(reinterpret_cast<uintptr_t>(y) & 15);
  if (n == 32 && bf16 && vec) {
    const int64_t n_tasks = (rows / 32) * ((cols + 255) >> 8);
    int64_t blocks = n_tasks < 148 * 12 ? n_tasks : 148 * 12;
    (void)launch_after(rht32_mma_kernel, dim3((unsigned)blocks), dim3(128), 0, st, a);
  } else if (n == 16) launch_rht_dense<16>(a, bf16, st);
  else if (n == 32) launch_rht_dense<32>(a, bf16, st);
  else launch_rht_dense<64>(a, bf16, st);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
