// Per-step bookkeeping of weight de-oscillation, one pass over five arrays:
//   dist_w   += |w - prev|
//   dist_qdq += |qdq(w) - qdq(prev)|
//   prev      = w
// which the reference does with five separate tensor ops per parameter per optimizer step
// (alto/components/optimizer.py:381-386).  Arithmetic is done in the arrays' dtype, as the tensor ops
// do: with bf16 arrays the difference and the sum are each rounded to bf16.
#include "common.cuh"

namespace altob200 {

template <bool IS_BF16>
__device__ __forceinline__ float rnd(float v) {
  return IS_BF16 ? u2f(f32_to_bf16_bits(v) << 16) : v;
}

template <bool IS_BF16>
__global__ void __launch_bounds__(256) deosc_accumulate_kernel(const void* __restrict__ w, void* __restrict__ prev,
                                                               const void* __restrict__ w_qdq,
                                                               const void* __restrict__ prev_qdq,
                                                               void* __restrict__ dist_w, void* __restrict__ dist_q,
                                                               int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float a, p, qa, qp, dw, dq;
    if (IS_BF16) {
      a = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
      p = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(prev)[i]);
      qa = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w_qdq)[i]);
      qp = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(prev_qdq)[i]);
      dw = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(dist_w)[i]);
      dq = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(dist_q)[i]);
    } else {
      a = reinterpret_cast<const float*>(w)[i];
      p = reinterpret_cast<const float*>(prev)[i];
      qa = reinterpret_cast<const float*>(w_qdq)[i];
      qp = reinterpret_cast<const float*>(prev_qdq)[i];
      dw = reinterpret_cast<const float*>(dist_w)[i];
      dq = reinterpret_cast<const float*>(dist_q)[i];
    }
    dw = rnd<IS_BF16>(__fadd_rn(dw, fabsf(rnd<IS_BF16>(__fsub_rn(a, p)))));
    dq = rnd<IS_BF16>(__fadd_rn(dq, fabsf(rnd<IS_BF16>(__fsub_rn(qa, qp)))));
    if (IS_BF16) {
      reinterpret_cast<__nv_bfloat16*>(dist_w)[i] = __float2bfloat16_rn(dw);
      reinterpret_cast<__nv_bfloat16*>(dist_q)[i] = __float2bfloat16_rn(dq);
      reinterpret_cast<__nv_bfloat16*>(prev)[i] = reinterpret_cast<const __nv_bfloat16*>(w)[i];
    } else {
      reinterpret_cast<float*>(dist_w)[i] = dw;
      reinterpret_cast<float*>(dist_q)[i] = dq;
      reinterpret_cast<float*>(prev)[i] = a;
    }
  }
}

}  // namespace altob200

extern "C" int altob200_deosc_accumulate(const void* w, void* prev, const void* w_qdq, const void* prev_qdq,
                                         void* dist_w, void* dist_qdq, int64_t n, int32_t dtype, void* stream) {
  using namespace altob200;
  if (n == 0) return ALTOB200_OK;
  if (w == nullptr || prev == nullptr || w_qdq == nullptr || prev_qdq == nullptr || dist_w == nullptr ||
      dist_qdq == nullptr || n < 0)
    return ALTOB200_EINVAL_SHAPE;
  if (dtype != ALTOB200_DT_BF16 && dtype != ALTOB200_DT_F32) return ALTOB200_EUNSUPPORTED;
  int64_t blocks = ceil_div(n, 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ALTOB200_DT_BF16)
    deosc_accumulate_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(w, prev, w_qdq, prev_qdq, dist_w, dist_qdq, n);
  else
    deosc_accumulate_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(w, prev, w_qdq, prev_qdq, dist_w, dist_qdq, n);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}
