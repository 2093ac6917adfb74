// Pre-norm residual kept as S parallel fp32 streams joined by learned scalars (static hyper-connections),
// with the statistics-free tanh norm  tanh(alpha u) w + b  fused into the same pass.
//
//   streams_step:  for every row, with X the S streams of the row ([T][S][D] fp32):
//                    (1) when a branch output y is given:  X_t <- sum_s mix[s][t] X_s + m out[t] y   (all t from the old X)
//                    (2) u = sum_t in[t] X_t  (in == NULL: the plain sum of the streams)
//                    (3) xb = tanh(alpha u) w + b, rounded once to the element type the next projection reads.
//                  One launch does the write-back of sublayer q and the read + norm of sublayer q + 1; with a row
//                  list it is the final norm of the rows whose logits are wanted.  S == 1 with in = out = mix = 1
//                  is the ordinary pre-norm residual  x <- x + m y.
//   embed_streams: token embedding times a scale into every stream.
// Everything is element-wise over D: no reduction, one read and one write of the streams.  fp32 throughout.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

constexpr int kMaxStreams = 8;

__device__ __forceinline__ float st_f32(float v) { return v; }
__device__ __forceinline__ float st_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void st_out(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_out(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// hc = [in: S | out: S | mix: S*S (from, to)] of the sublayer that produced y (hc_w) and of the one that reads
// next (hc_r; NULL = sum of the streams).  VEC elements of D per thread (4: 16-byte accesses of the streams).
template <typename TY, typename TO, int VEC>
__global__ void __launch_bounds__(256)
streams_step_kernel(const TY* __restrict__ y, int64_t ldy, float* X, const int32_t* __restrict__ rows,
                    const float* __restrict__ hc_w, float m, const float* __restrict__ hc_r,
                    const float* __restrict__ alpha_p, const bf16* __restrict__ w, const bf16* __restrict__ b,
                    TO* xb_out, int T, int S, int D) {
  __shared__ float c_mix[kMaxStreams * kMaxStreams], c_out[kMaxStreams], c_in[kMaxStreams];
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = hc_w != nullptr ? hc_w[2 * S + threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = hc_w != nullptr ? m * hc_w[S + threadIdx.x] : 0.f;
    c_in[threadIdx.x] = hc_r != nullptr ? hc_r[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const float alpha = xb_out != nullptr ? alpha_p[0] : 0.f;
  const int dv = D / VEC;
  const size_t total = (size_t)T * dv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / dv), d = (int)(i % dv) * VEC;
    const int src = rows != nullptr ? rows[r] : r;
    float* xr = X + (size_t)src * S * D + d;
    float x[kMaxStreams][VEC];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) {
      if (s < S) {
        if (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * D);
          x[s][0] = v.x; x[s][VEC > 1 ? 1 : 0] = v.y; x[s][VEC > 2 ? 2 : 0] = v.z; x[s][VEC > 3 ? 3 : 0] = v.w;
        } else {
          x[s][0] = xr[(size_t)s * D];
        }
      }
    }
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = 0.f;
    if (y != nullptr) {
      float yv[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) yv[e] = st_f32(y[(size_t)r * ldy + d + e]);
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float n[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) n[e] = c_out[t] * yv[e];
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s) {
            if (s < S) {
#pragma unroll
              for (int e = 0; e < VEC; ++e) n[e] = fmaf(c_mix[s * S + t], x[s][e], n[e]);
            }
          }
          if (VEC == 4) *reinterpret_cast<float4*>(xr + (size_t)t * D) = make_float4(n[0], n[VEC > 1 ? 1 : 0], n[VEC > 2 ? 2 : 0], n[VEC > 3 ? 3 : 0]);
          else xr[(size_t)t * D] = n[0];
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = fmaf(c_in[t], n[e], u[e]);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = fmaf(c_in[t], x[t][e], u[e]);
        }
      }
    }
    if (xb_out != nullptr) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float o = fmaf(tanhf(alpha * u[e]), __bfloat162float(w[d + e]), __bfloat162float(b[d + e]));
        st_out(xb_out + (size_t)r * D + d + e, o);
      }
    }
  }
}

__global__ void embed_streams_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ table, float* X,
                                     int T, int S, int D, int V, float scale) {
  const size_t n = (size_t)T * D;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / D), d = (int)(i % D);
    const int id = ids[t];
    const float v = (id >= 0 && id < V) ? __bfloat162float(table[(size_t)id * D + d]) * scale : 0.f;
    for (int s = 0; s < S; ++s) X[((size_t)t * S + s) * D + d] = v;
  }
}

static int st_blocks(size_t n) {
  size_t b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 8192 ? 8192 : b));
}

}  // namespace b200

using namespace b200;

extern "C" int b200_streams_step(const void* y, int y_f32, int64_t ldy, float* X, const int32_t* rows,
                                 const float* hc_write, float mult, const float* hc_read, const float* alpha,
                                 const void* w, const void* b, void* xb_out, int xb_f32, int T, int S, int D,
                                 void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && S >= 1 && S <= kMaxStreams, "streams_step: bad shape T=%d S=%d D=%d (S <= %d)", T, S, D,
               kMaxStreams);
  B200_REQUIRE(y == nullptr || (hc_write != nullptr && rows == nullptr), "streams_step: a branch output needs its weights and no row list");
  B200_REQUIRE(xb_out == nullptr || (alpha != nullptr && w != nullptr && b != nullptr), "streams_step: the norm needs alpha, w and b");
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = D % 4 == 0 && (y == nullptr || (ldy % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0)) &&
                   reinterpret_cast<uintptr_t>(X) % 16 == 0;
  const int blocks = st_blocks((size_t)T * (vec ? D / 4 : D));
#define B200_ST(TY, TO, V)                                                                                          \
  streams_step_kernel<TY, TO, V><<<blocks, 256, 0, s>>>((const TY*)y, ldy, X, rows, hc_write, mult, hc_read, alpha, \
                                                        (const bf16*)w, (const bf16*)b, (TO*)xb_out, T, S, D)
#define B200_ST2(TY, TO) do { if (vec) B200_ST(TY, TO, 4); else B200_ST(TY, TO, 1); } while (0)
  if (y_f32 && xb_f32) B200_ST2(float, float);
  else if (y_f32) B200_ST2(float, bf16);
  else if (xb_f32) B200_ST2(bf16, float);
  else B200_ST2(bf16, bf16);
#undef B200_ST2
#undef B200_ST
  return b200_check_launch("b200_streams_step");
}

extern "C" int b200_embed_streams(const int32_t* ids, const void* table, float* X, int T, int S, int D, int V,
                                  float scale, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && V > 0 && S >= 1 && S <= kMaxStreams, "embed_streams: bad shape");
  if (T == 0) return B200_OK;
  embed_streams_kernel<<<st_blocks((size_t)T * D), 256, 0, (cudaStream_t)stream>>>(ids, (const bf16*)table, X, T, S, D, V,
                                                                                 scale);
  return b200_check_launch("b200_embed_streams");
}
