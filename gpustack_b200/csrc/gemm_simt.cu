// General linear layer on the CUDA cores: y = x W^T (+ bias), x [M,K] bf16 or fp32, W [N,K] bf16,
// fp32 FMA accumulation in a fixed order over K, y bf16 or fp32.  No shape or alignment rule.
// It serves (1) every projection of a model that runs in true 32-bit (fp32 activations, no
// reduced-precision tensor mode), and (2) bf16 projections whose shape the tcgen05 kernel cannot take
// (K not a multiple of 64, rows that are not 16-byte aligned: per-head gate projections with a
// handful of outputs).  A result element never depends on M or on the row's place in the batch.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

constexpr int kSimtBM = 64, kSimtBN = 64, kSimtBK = 16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f32(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ X, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                 TY* __restrict__ Y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy) {
  __shared__ float Xs[kSimtBK][kSimtBM + 4];
  __shared__ float Ws[kSimtBK][kSimtBN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * kSimtBM, n0 = blockIdx.x * kSimtBN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  // loader mapping: 64 rows x 16 k = 1024 elements, 4 per thread (k fastest: contiguous in memory)
  const int lk = tid & 15, lr = tid >> 4;          // row lr + 16 i
  for (int k0 = 0; k0 < K; k0 += kSimtBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = lr + 16 * i;
      const int k = k0 + lk;
      float xv = 0.f, wv = 0.f;
      if (k < K) {
        if (m0 + r < M) xv = to_f32(X[(int64_t)(m0 + r) * ldx + k]);
        if (n0 + r < N) wv = to_f32(W[(int64_t)(n0 + r) * ldw + k]);
      }
      Xs[lk][r] = xv;
      Ws[lk][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += __bfloat162float(bias[n]);
      from_f32(Y + (int64_t)m * ldy + n, v);
    }
  }
}

template <typename TX, typename TY>
static int launch_simt(const void* X, const void* W, const void* bias, void* Y, int M, int N, int K, int64_t ldx,
                       int64_t ldw, int64_t ldy, cudaStream_t s) {
  dim3 grid((N + kSimtBN - 1) / kSimtBN, (M + kSimtBM - 1) / kSimtBM);
  gemm_simt_kernel<TX, TY><<<grid, 256, 0, s>>>((const TX*)X, (const bf16*)W, (const bf16*)bias, (TY*)Y, M, N, K,
                                                ldx, ldw, ldy);
  return b200_check_launch("b200_linear_simt");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_linear_simt(const void* X, int x_f32, const void* W, const void* bias, void* Y, int y_f32, int M,
                                int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, void* stream) {
  B200_REQUIRE(M >= 0 && N > 0 && K > 0, "linear_simt: bad shape M=%d N=%d K=%d", M, N, K);
  B200_REQUIRE(ldx >= K && ldw >= K && ldy >= N, "linear_simt: leading dimensions too small");
  if (M == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (x_f32 && y_f32) return launch_simt<float, float>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, s);
  if (x_f32) return launch_simt<float, bf16>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, s);
  if (y_f32) return launch_simt<bf16, float>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, s);
  return launch_simt<bf16, bf16>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, s);
}
