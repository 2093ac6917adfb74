// Preparation steps of latent attention (keys and values expanded from one small latent per token).
//
//   rms_rows:     out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w over a column slice of a wider row
//                 (the query latent between its two projections).  fp32 statistics.
//   latent_prep:  one pass over a token's fused projection row  [ ... | latent: R | key part: dr ]  and its
//                 query rows  [H][dn unrotated | dr rotated]:
//                   * the latent is RMS-normed (weight, eps) and written to the token's cache row [0, R),
//                   * the key part is rotated at the token's position and written to cache row [R, R + dr),
//                   * every head's rotated query part is rotated and written to qa[t][h][R, R + dr) -- the tail
//                     of the absorbed query, whose first R entries  W_uk[h]^T q_unrotated  a batched linear fills.
//                 Rotation: the first `dims` entries of a part, pairs (2i, 2i+1) ("interleaved") or
//                 (i, i + dims/2) ("half"), angle = position * freq[i] formed and reduced to [-pi, pi] in fp64 (once
//                 per token and pair, shared by the key part and all heads), cos and sin multiplied by one factor
//                 (frequency-scaled variants); the rest of the part passes unchanged.
// Cache layout: [blocks][page][R + dr]: one row per token shared by all heads.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float lt_f32(float v) { return v; }
__device__ __forceinline__ float lt_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void lt_out(float* p, float v) { *p = v; }
__device__ __forceinline__ void lt_out(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kLtWarps = 4;
constexpr int kLtPrepMaxWarps = 16;

template <typename TA>
__global__ void __launch_bounds__(kLtWarps * 32)
rms_rows_kernel(const TA* __restrict__ x, int64_t ldx, const bf16* __restrict__ w, TA* out, int64_t ldo, int T, int n,
                float eps) {
  const int t = blockIdx.x * kLtWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const TA* xr = x + (size_t)t * ldx;
  float ss = 0.f;
  for (int d = lane; d < n; d += 32) {
    const float v = lt_f32(xr[d]);
    ss = fmaf(v, v, ss);
  }
  const float mul = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  for (int d = lane; d < n; d += 32) lt_out(out + (size_t)t * ldo + d, lt_f32(xr[d]) * mul * __bfloat162float(w[d]));
}

constexpr int kLtMaxPairs = 256;   // rotated pairs per part (dims <= 512)

// src / dst: a part of `width` entries; entries [0, dims) are rotated by the token's angles (cs / sn, one per pair).
template <typename TA>
__device__ __forceinline__ void rotate_part(const TA* src, TA* dst, int width, int dims, int half_layout,
                                            const float* cs, const float* sn, int lane) {
  const int half = dims >> 1;
  for (int i = lane; i < half; i += 32) {
    const int a = half_layout ? i : 2 * i, b = half_layout ? i + half : 2 * i + 1;
    const float c = cs[i], s = sn[i];
    const float u = lt_f32(src[a]), v = lt_f32(src[b]);
    lt_out(dst + a, u * c - v * s);
    lt_out(dst + b, v * c + u * s);
  }
  for (int d = dims + lane; d < width; d += 32) lt_out(dst + d, lt_f32(src[d]));
}

// One CTA per token.  The token's cos / sin (angle formed and reduced in fp64, one evaluation per pair for all heads)
// go to shared memory first; then the warps take the tasks in turn: task 0 = the latent and the key part, task 1 + h =
// head h's rotated query part.
template <typename TA>
__global__ void __launch_bounds__(kLtPrepMaxWarps * 32)
latent_prep_kernel(const TA* __restrict__ proj, int64_t ld, int kv_col, const TA* __restrict__ q, int64_t ldq,
                   const bf16* __restrict__ kv_norm_w, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ slots, TA* cache, TA* qa, int64_t ldqa, int H, int dn, int dr, int R,
                   int dims, int half_layout, const double* __restrict__ freq, float mag, float eps) {
  __shared__ float cs[kLtMaxPairs], sn[kLtMaxPairs];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < (dims >> 1); i += blockDim.x) {
    // the angle and its reduction to [-pi, pi] in fp64 (a handful of operations), cos / sin of the remainder in fp32
    const double ang = (double)pos * freq[i];
    const double turns = rint(ang * 0.15915494309189535);
    const float rem = (float)fma(-turns, 6.283185307179586, ang);
    float s_, c_;
    sincosf(rem, &s_, &c_);
    cs[i] = c_ * mag;
    sn[i] = s_ * mag;
  }
  __syncthreads();
  for (int task = warp; task <= H; task += (int)(blockDim.x >> 5)) {
    if (task == 0) {
      const int slot = slots[t];
      if (slot < 0) continue;                     // a padding row: nothing to cache
      const TA* kv = proj + (size_t)t * ld + kv_col;
      TA* row = cache + (size_t)slot * (R + dr);
      float ss = 0.f;
      for (int d = lane; d < R; d += 32) {
        const float v = lt_f32(kv[d]);
        ss = fmaf(v, v, ss);
      }
      const float mul = 1.0f / sqrtf(warp_sum(ss) / (float)R + eps);
      for (int d = lane; d < R; d += 32) lt_out(row + d, lt_f32(kv[d]) * mul * __bfloat162float(kv_norm_w[d]));
      rotate_part(kv + R, row + R, dr, dims, half_layout, cs, sn, lane);
      continue;
    }
    const int h = task - 1;
    rotate_part(q + (size_t)t * ldq + (size_t)h * (dn + dr) + dn, qa + (size_t)t * ldqa + (size_t)h * (R + dr) + R, dr, dims,
                half_layout, cs, sn, lane);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rms_rows(const void* x, int f32, int64_t ldx, const void* w, void* out, int64_t ldo, int T, int n,
                             float eps, void* stream) {
  B200_REQUIRE(T >= 0 && n > 0 && ldx >= n && ldo >= n, "rms_rows: bad shape T=%d n=%d", T, n);
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = (T + kLtWarps - 1) / kLtWarps;
  if (f32) rms_rows_kernel<float><<<grid, kLtWarps * 32, 0, s>>>((const float*)x, ldx, (const bf16*)w, (float*)out, ldo, T, n, eps);
  else rms_rows_kernel<bf16><<<grid, kLtWarps * 32, 0, s>>>((const bf16*)x, ldx, (const bf16*)w, (bf16*)out, ldo, T, n, eps);
  return b200_check_launch("b200_rms_rows");
}

extern "C" int b200_latent_prep(const void* proj, int f32, int64_t ld, int kv_col, const void* q, int64_t ldq,
                                const void* kv_norm_w, const int32_t* positions, const int32_t* slots, void* cache,
                                void* qa, int64_t ldqa, int T, int H, int dn, int dr, int R, int dims, int half_layout,
                                const double* freq, float mag, float eps, void* stream) {
  B200_REQUIRE(T >= 0 && H > 0 && dn >= 0 && dr > 0 && R > 0 && dims > 0 && dims % 2 == 0 && dims <= dr &&
                   dims <= 2 * kLtMaxPairs,
               "latent_prep: bad shape H=%d dn=%d dr=%d R=%d dims=%d", H, dn, dr, R, dims);
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(T);
  const int threads = 32 * (H + 1 < kLtWarps ? H + 1 : kLtWarps);
  if (f32)
    latent_prep_kernel<float><<<grid, threads, 0, s>>>((const float*)proj, ld, kv_col, (const float*)q, ldq,
                                                            (const bf16*)kv_norm_w, positions, slots, (float*)cache,
                                                            (float*)qa, ldqa, H, dn, dr, R, dims, half_layout, freq, mag, eps);
  else
    latent_prep_kernel<bf16><<<grid, threads, 0, s>>>((const bf16*)proj, ld, kv_col, (const bf16*)q, ldq,
                                                           (const bf16*)kv_norm_w, positions, slots, (bf16*)cache,
                                                           (bf16*)qa, ldqa, H, dn, dr, R, dims, half_layout, freq, mag, eps);
  return b200_check_launch("b200_latent_prep");
}
