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
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), src_rows, row_bytes / 16, index, out_rows, reinterpret_cast<uint4*>(dst));
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
