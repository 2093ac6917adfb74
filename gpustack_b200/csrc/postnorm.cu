// Norm-after-sum residual stream kept in fp32, and the small element-wise steps around it.
//
//   sum_layer_norm:  z = alpha * x + y  (or z = x when there is no branch output), then the bias-free
//                    layer norm  (z - mean) / sqrt(var + eps) * w * out_scale,  var = mean((z - mean)^2).
//                    The sum, both statistics and the product are fp32; the normalised row is written as
//                    the new fp32 residual stream and, rounded once, as the next projection's bf16 input.
//                    With a row list it gathers (final norm of the rows whose logits are wanted).
//   embed_rows:      token embedding -> fp32 residual stream + bf16 copy.
//   relu2:           max(u, 0)^2, the feed-forward activation between the up and down projections.
// One CTA per row, the row is staged in shared memory once (two-pass variance, no E[z^2] - E[z]^2).
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float pn_f32(float v) { return v; }
__device__ __forceinline__ float pn_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void pn_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void pn_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float pn_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();                       // red may still be read by the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
sum_layer_norm_kernel(const TY* __restrict__ y, int64_t ldy, const float* x_in, const int32_t* __restrict__ rows,
                      const bf16* __restrict__ w, float* x_out, TO* xb_out, int D, float alpha, float eps,
                      float out_scale) {
  extern __shared__ float zrow[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x_in + (size_t)src * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float z = xr[i];
    if (y != nullptr) z = fmaf(alpha, z, pn_f32(y[(size_t)r * ldy + i]));
    zrow[i] = z;
    s += z;
  }
  const float mean = pn_block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float d = zrow[i] - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = 1.0f / sqrtf(pn_block_sum(q, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float o = (zrow[i] - mean) * rstd * __bfloat162float(w[i]) * out_scale;
    if (x_out != nullptr) x_out[(size_t)r * D + i] = o;
    if (xb_out != nullptr) pn_store(xb_out + (size_t)r * D + i, o);
  }
}

template <typename TO>
__global__ void embed_rows_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ table, float* x_out,
                                  TO* xb_out, int T, int D, int V) {
  const size_t n = (size_t)T * D;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / D), d = (int)(i % D);
    const int id = ids[t];
    const bf16 v = (id >= 0 && id < V) ? table[(size_t)id * D + d] : __float2bfloat16_rn(0.f);
    x_out[i] = __bfloat162float(v);
    if (xb_out != nullptr) pn_store(xb_out + i, __bfloat162float(v));
  }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ u, T* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(pn_f32(u[i]), 0.f);
    pn_store(out + i, v * v);
  }
}

static int ew_blocks(size_t n) {
  size_t b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 4096 ? 4096 : b));
}

}  // namespace b200

using namespace b200;

extern "C" int b200_sum_layer_norm(const void* y, int y_f32, int64_t ldy, const float* x_in, const int32_t* rows,
                                   const void* w, float* x_out, void* xb_out, int xb_f32, int T, int D, float alpha,
                                   float eps, float out_scale, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0, "sum_layer_norm: bad shape T=%d D=%d", T, D);
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)D * sizeof(float);
  B200_REQUIRE(smem <= 48 * 1024, "sum_layer_norm: D=%d exceeds the staged row (12288)", D);
  const bf16* wp = (const bf16*)w;
#define B200_SLN(TY, TO)                                                                                      \
  sum_layer_norm_kernel<TY, TO><<<T, 256, smem, s>>>((const TY*)y, ldy, x_in, rows, wp, x_out, (TO*)xb_out, D, \
                                                     alpha, eps, out_scale)
  if (y_f32 && xb_f32) B200_SLN(float, float);
  else if (y_f32) B200_SLN(float, bf16);
  else if (xb_f32) B200_SLN(bf16, float);
  else B200_SLN(bf16, bf16);
#undef B200_SLN
  return b200_check_launch("b200_sum_layer_norm");
}

extern "C" int b200_embed_rows_f32(const int32_t* ids, const void* table, float* x_out, void* xb_out, int xb_f32,
                                   int T, int D, int V, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && V > 0, "embed_rows: bad shape");
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = ew_blocks((size_t)T * D);
  if (xb_f32)
    embed_rows_kernel<float><<<blocks, 256, 0, s>>>(ids, (const bf16*)table, x_out, (float*)xb_out, T, D, V);
  else
    embed_rows_kernel<bf16><<<blocks, 256, 0, s>>>(ids, (const bf16*)table, x_out, (bf16*)xb_out, T, D, V);
  return b200_check_launch("b200_embed_rows_f32");
}

extern "C" int b200_relu2(const void* u, void* out, int f32, int64_t n, void* stream) {
  B200_REQUIRE(n >= 0, "relu2: bad size");
  if (n == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (f32) relu2_kernel<float><<<ew_blocks((size_t)n), 256, 0, s>>>((const float*)u, (float*)out, (size_t)n);
  else relu2_kernel<bf16><<<ew_blocks((size_t)n), 256, 0, s>>>((const bf16*)u, (bf16*)out, (size_t)n);
  return b200_check_launch("b200_relu2");
}
