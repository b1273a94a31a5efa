// DGE factor applied to a weight gradient:  dW[n, k] = cast(float(dW[n, k]) * lut[code(W[n, k])]).
//
// The reference multiplies the weight gradient by dge_bwd(FP4 bin value of the weight)
// (alto/kernels/dge/dge.py:81-93; alto/kernels/fp4/nvfp4/nvfp_linear.py:250-268,
// alto/kernels/fp4/mxfp4/mxfp_linear.py:546-566).  The bin value of an element is one of sixteen
// numbers, so the factor is a sixteen-entry table indexed by the element's E2M1 code; the host
// evaluates the reference's expression on the sixteen values and passes the table.
//
// The codes come from the weight operand saved for dgrad, which is stored transposed:
// codes_t[k, n / 2], element n in nibble n & 1.  A CTA handles 64 rows x 64 columns of dW: the
// 64 x 32 bytes of codes are staged through shared memory so that both the code reads and the
// gradient reads and writes are coalesced.
#include "common.cuh"

namespace altob200 {

struct DgeArgs {
  void* dw;
  const uint8_t* codes_t;
  int64_t N, K, ld;
  float lut[16];
};

template <bool IS_BF16>
__global__ void __launch_bounds__(256) dge_scale_kernel(DgeArgs a) {
  __shared__ uint8_t s_codes[64][32 + 4];  // [k in tile][n / 2 in tile], padded against bank conflicts
  __shared__ float s_lut[16];
  const int64_t n0 = (int64_t)blockIdx.y * 64, k0 = (int64_t)blockIdx.x * 64;
  if (threadIdx.x < 16) s_lut[threadIdx.x] = a.lut[threadIdx.x];
  const int64_t half_n = a.N >> 1;
  for (int t = threadIdx.x; t < 64 * 32; t += 256) {
    const int kk = t >> 5, b = t & 31;
    const int64_t k = k0 + kk, nb = (n0 >> 1) + b;
    s_codes[kk][b] = (k < a.K && nb < half_n) ? a.codes_t[k * half_n + nb] : 0;
  }
  __syncthreads();
  // thread -> (row n, 16 consecutive k): 64 rows x 4 segments
  const int nn = threadIdx.x >> 2, seg = threadIdx.x & 3;
  const int64_t n = n0 + nn;
  if (n >= a.N) return;
#pragma unroll 4
  for (int j = 0; j < 16; ++j) {
    const int kk = seg * 16 + j;
    const int64_t k = k0 + kk;
    if (k >= a.K) break;
    const uint32_t byte = s_codes[kk][nn >> 1];
    const float f = s_lut[(byte >> (4 * (nn & 1))) & 0xFu];
    if (IS_BF16) {
      __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(a.dw) + n * a.ld + k;
      *p = __float2bfloat16_rn(__fmul_rn(__bfloat162float(*p), f));
    } else {
      float* p = reinterpret_cast<float*>(a.dw) + n * a.ld + k;
      *p = __fmul_rn(*p, f);
    }
  }
}

}  // namespace altob200

extern "C" int altob200_dge_scale(void* dw, int32_t dtype, int64_t N, int64_t K, int64_t ld, const void* codes_t,
                                  const float* lut16_host, void* stream) {
  using namespace altob200;
  if (dw == nullptr || codes_t == nullptr || lut16_host == nullptr) return ALTOB200_EINVAL_SHAPE;
  if (N <= 0 || K <= 0 || N % 2 != 0 || ld < K) return ALTOB200_EINVAL_SHAPE;
  if (dtype != ALTOB200_DT_BF16 && dtype != ALTOB200_DT_F32) return ALTOB200_EUNSUPPORTED;
  if (ceil_div(N, 64) > 65535) return ALTOB200_ELIMIT;
  DgeArgs a;
  a.dw = dw; a.codes_t = (const uint8_t*)codes_t; a.N = N; a.K = K; a.ld = ld;
  for (int i = 0; i < 16; ++i) a.lut[i] = lut16_host[i];
  dim3 grid((unsigned)ceil_div(K, 64), (unsigned)ceil_div(N, 64));
  if (dtype == ALTOB200_DT_BF16) dge_scale_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  else dge_scale_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
