// Row gather with zero fill: dst[i] = index[i] >= 0 ? src[index[i]] : 0.
//
// This is the data movement of the MoE token path around the grouped GEMMs: sorting routed token
// rows by expert and padding every expert's run to a multiple of 128 rows (index -1 = padding row),
// and the inverse on the way back.  The reference delegates it to its TorchTitan fork's token
// dispatcher (call sites alto/modifiers/lpt/base.py:194-201, alto/kernels/dispatch/tensor.py:224-263);
// the grouped kernels only require the result: runs of 128 rows per expert, zero rows as padding
// (alto/kernels/fp4/fp4_common/grouped_utils.py:81-94).
//
// One warp per output row, 16 bytes per lane per step; rows are independent, the kernel is a
// plain HBM copy (row_bytes read + row_bytes written per row).
#include "common.cuh"

namespace altob200 {

__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, int64_t src_rows,
                                                          int64_t row_vec, const int32_t* __restrict__ index,
                                                          int64_t out_rows, uint4* __restrict__ dst) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
  for (int64_t r = warp0; r < out_rows; r += n_warps) {
    const int64_t s = __ldg(index + r);
    uint4* d = dst + r * row_vec;
    if (s >= 0 && s < src_rows) {
      const uint4* p = src + s * row_vec;
      for (int64_t c = lane; c < row_vec; c += 32) d[c] = __ldg(p + c);
    } else {
      for (int64_t c = lane; c < row_vec; c += 32) d[c] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// Weighted combine of a token's k routed rows:  out[t] = bf16( sum_j f32( bf16( rows[index[t k + j]] * score[t k + j] ) ) ),
// the roundings of the tensor-op form (gather, multiply in bf16, sum over k with fp32 accumulation).
// index -1 contributes nothing; scores == NULL means weights of one.  One warp per token, 8 columns
// (16 bytes) per lane and step.
__global__ void __launch_bounds__(256) combine_rows_kernel(const uint4* __restrict__ rows, int64_t n_rows, int64_t row_vec,
                                                           const int32_t* __restrict__ index,
                                                           const __nv_bfloat16* __restrict__ scores, int64_t T, int k,
                                                           uint4* __restrict__ out) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
  for (int64_t t = warp0; t < T; t += n_warps) {
    for (int64_t c = lane; c < row_vec; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int64_t r = __ldg(index + t * k + j);
        if (r < 0 || r >= n_rows) continue;
        const float s = scores != nullptr ? __bfloat162float(scores[t * k + j]) : 1.0f;
        const uint4 w = __ldg(rows + r * row_vec + c);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float lo = u2f(f32_to_bf16_bits(__fmul_rn(bf16lo_to_f32(ws[q]), s)) << 16);
          const float hi = u2f(f32_to_bf16_bits(__fmul_rn(bf16hi_to_f32(ws[q]), s)) << 16);
          acc[2 * q] = __fadd_rn(acc[2 * q], lo);
          acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], hi);
        }
      }
      uint4 o;
      o.x = f32_to_bf16_bits(acc[0]) | (f32_to_bf16_bits(acc[1]) << 16);
      o.y = f32_to_bf16_bits(acc[2]) | (f32_to_bf16_bits(acc[3]) << 16);
      o.z = f32_to_bf16_bits(acc[4]) | (f32_to_bf16_bits(acc[5]) << 16);
      o.w = f32_to_bf16_bits(acc[6]) | (f32_to_bf16_bits(acc[7]) << 16);
      out[t * row_vec + c] = o;
    }
  }
}

// Its gradient with respect to the rows:  grad_rows[r] = bf16( grad_out[p / k] * score[p] ) with p = position[r]
// (the routed slot that row r feeds), zero rows where position[r] < 0.
__global__ void __launch_bounds__(256) spread_rows_kernel(const uint4* __restrict__ grad_out, int64_t T, int k,
                                                          int64_t row_vec, const int32_t* __restrict__ position,
                                                          const __nv_bfloat16* __restrict__ scores, int64_t n_rows,
                                                          uint4* __restrict__ grad_rows) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
  for (int64_t r = warp0; r < n_rows; r += n_warps) {
    const int64_t p = __ldg(position + r);
    uint4* d = grad_rows + r * row_vec;
    if (p < 0 || p >= T * k) {
      for (int64_t c = lane; c < row_vec; c += 32) d[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float s = scores != nullptr ? __bfloat162float(scores[p]) : 1.0f;
    const uint4* g = grad_out + (p / k) * row_vec;
    for (int64_t c = lane; c < row_vec; c += 32) {
      const uint4 w = __ldg(g + c);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o[q] = f32_to_bf16_bits(__fmul_rn(bf16lo_to_f32(ws[q]), s)) | (f32_to_bf16_bits(__fmul_rn(bf16hi_to_f32(ws[q]), s)) << 16);
      d[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace altob200

extern "C" int altob200_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes, const int32_t* index,
                                    int64_t out_rows, void* dst, void* stream) {
  using namespace altob200;
  if (out_rows == 0) return ALTOB200_OK;
  if (src == nullptr || dst == nullptr || index == nullptr || src_rows < 0 || out_rows < 0 || row_bytes <= 0)
    return ALTOB200_EINVAL_SHAPE;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return ALTOB200_EINVAL_ALIGN;
  int64_t blocks = ceil_div(out_rows, 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  (void)launch_after(gather_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 
      reinterpret_cast<const uint4*>(src), src_rows, row_bytes / 16, index, out_rows, reinterpret_cast<uint4*>(dst));
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

extern "C" int altob200_combine_rows(const void* rows, int64_t n_rows, int64_t row_bytes, const int32_t* index,
                                     const void* scores, int64_t tokens, int32_t k, void* out, void* stream) {
  using namespace altob200;
  if (tokens == 0) return ALTOB200_OK;
  if (rows == nullptr || out == nullptr || index == nullptr || n_rows < 0 || tokens < 0 || k <= 0 || row_bytes <= 0)
    return ALTOB200_EINVAL_SHAPE;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(rows) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return ALTOB200_EINVAL_ALIGN;
  int64_t blocks = ceil_div(tokens, 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  (void)launch_after(combine_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 
      reinterpret_cast<const uint4*>(rows), n_rows, row_bytes / 16, index, reinterpret_cast<const __nv_bfloat16*>(scores),
      tokens, k, reinterpret_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

extern "C" int altob200_spread_rows(const void* grad_out, int64_t tokens, int32_t k, int64_t row_bytes,
                                    const int32_t* position, const void* scores, int64_t n_rows, void* grad_rows,
                                    void* stream) {
  using namespace altob200;
  if (n_rows == 0) return ALTOB200_OK;
  if (grad_out == nullptr || grad_rows == nullptr || position == nullptr || n_rows < 0 || tokens < 0 || k <= 0 ||
      row_bytes <= 0)
    return ALTOB200_EINVAL_SHAPE;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(grad_out) & 15) || (reinterpret_cast<uintptr_t>(grad_rows) & 15))
    return ALTOB200_EINVAL_ALIGN;
  int64_t blocks = ceil_div(n_rows, 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  (void)launch_after(spread_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 
      reinterpret_cast<const uint4*>(grad_out), tokens, k, row_bytes / 16, position,
      reinterpret_cast<const __nv_bfloat16*>(scores), n_rows, reinterpret_cast<uint4*>(grad_rows));
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
