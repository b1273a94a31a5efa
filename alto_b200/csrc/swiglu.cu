// SwiGLU between the two grouped GEMMs of an expert MLP, forward and backward, one kernel each.
//
//   forward   out[r, c]      = bf16( bf16(silu(g)) * u ),   g = h[r, c], u = h[r, H + c]
//   backward  grad_h[r, c]   = bf16( bf16(go * u) * s * (1 + g * (1 - s)) ),   s = 1 / (1 + exp(-g))
//             grad_h[r, H+c] = bf16( go * bf16(silu(g)) )
//
// The expert MLP that the reference converts (the GroupedExperts module of its TorchTitan fork,
// alto/modifiers/lpt/base.py:186-187; the module itself is not among the reference's sources) puts a
// SiLU-gated product between its grouped GEMMs.  With the gate and up projections fused into one
// GEMM that writes [rows, 2H], tensor ops on the two halves cost eight passes over the routed rows
// forward and backward.  Intermediate roundings to bf16 are kept where the tensor-op form
// silu(h[:, :H]) * h[:, H:] and its autograd have them, so that the values equal that form's.
//
// One thread handles 8 columns of one row (16-byte loads and stores); both kernels are plain HBM
// streams: forward reads 4H and writes 2H bytes per row, backward reads 6H and writes 4H.
#include "common.cuh"

namespace altob200 {

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

__device__ __forceinline__ void unpack8(const uint4& w, float v[8]) {
  v[0] = bf16lo_to_f32(w.x); v[1] = bf16hi_to_f32(w.x); v[2] = bf16lo_to_f32(w.y); v[3] = bf16hi_to_f32(w.y);
  v[4] = bf16lo_to_f32(w.z); v[5] = bf16hi_to_f32(w.z); v[6] = bf16lo_to_f32(w.w); v[7] = bf16hi_to_f32(w.w);
}
__device__ __forceinline__ uint4 pack8(const float v[8]) {
  uint4 o;
  o.x = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
  o.y = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
  o.z = f32_to_bf16_bits(v[4]) | (f32_to_bf16_bits(v[5]) << 16);
  o.w = f32_to_bf16_bits(v[6]) | (f32_to_bf16_bits(v[7]) << 16);
  return o;
}
__device__ __forceinline__ float round_bf16(float x) { return u2f(f32_to_bf16_bits(x) << 16); }

template <bool BACKWARD>
__global__ void __launch_bounds__(256) swiglu_kernel(const uint4* __restrict__ h, const uint4* __restrict__ go,
                                                     int64_t rows, int64_t hv /* H / 8 */, int64_t ldv /* ld_h / 8 */,
                                                     uint4* __restrict__ out) {
  grid_dependency_wait();
  const int64_t n = rows * hv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / hv, c = i - r * hv;
    float g[8], u[8];
    unpack8(__ldg(h + r * ldv + c), g);
    unpack8(__ldg(h + r * ldv + hv + c), u);
    if (!BACKWARD) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(round_bf16(silu_f32(g[j])), u[j]);
      out[r * hv + c] = pack8(o);
    } else {
      float d[8], dg[8], du[8];
      unpack8(__ldg(go + r * hv + c), d);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float s = 1.0f / (1.0f + expf(-g[j]));
        const float ds = round_bf16(__fmul_rn(d[j], u[j]));
        dg[j] = ds * s * (1.0f + g[j] * (1.0f - s));
        du[j] = __fmul_rn(d[j], round_bf16(silu_f32(g[j])));
      }
      out[r * ldv + c] = pack8(dg);
      out[r * ldv + hv + c] = pack8(du);
    }
  }
}

static int swiglu_launch(const void* h, const void* go, int64_t rows, int64_t H, int64_t ld_h, void* out, bool backward,
                         cudaStream_t st) {
  if (rows == 0) return ALTOB200_OK;
  if (h == nullptr || out == nullptr || (backward && go == nullptr) || rows < 0 || H <= 0 || ld_h < 2 * H)
    return ALTOB200_EINVAL_SHAPE;
  if (H % 8 != 0 || ld_h % 8 != 0 || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (backward && (reinterpret_cast<uintptr_t>(go) & 15)))
    return ALTOB200_EINVAL_ALIGN;
  int64_t blocks = ceil_div(rows * (H / 8), 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (backward)
    (void)launch_after(swiglu_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, st, reinterpret_cast<const uint4*>(h), reinterpret_cast<const uint4*>(go),
                                                          rows, H / 8, ld_h / 8, reinterpret_cast<uint4*>(out));
  else
    (void)launch_after(swiglu_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, st, reinterpret_cast<const uint4*>(h), nullptr, rows, H / 8, ld_h / 8,
                                                           reinterpret_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

}  // namespace altob200

extern "C" {

int altob200_swiglu_forward(const void* h, int64_t rows, int64_t H, int64_t ld_h, void* out, void* stream) {
  return altob200::swiglu_launch(h, nullptr, rows, H, ld_h, out, false, (cudaStream_t)stream);
}

int altob200_swiglu_backward(const void* h, const void* grad_out, int64_t rows, int64_t H, int64_t ld_h, void* grad_h,
                             void* stream) {
  return altob200::swiglu_launch(h, grad_out, rows, H, ld_h, grad_h, true, (cudaStream_t)stream);
}

}  // extern "C"
