// Matrix-memory recurrence (mLSTM) with a running-maximum stabiliser, state in fp32.
//
// Per head, with log input gate i_t and log forget gate f_t:
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        (S: dk x dv)
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// with S, n, m = 0 before a sequence's first token.  The gates come from raw per-head projections
// a: i = cap * tanh((a_i + b_i) / cap), f = logsigmoid(cap * tanh((a_f + b_f) / cap)).
//
// `mlstm_scan` runs a sequence's new tokens in order (a prompt portion, or the single token of a
// decode step: the same launch serves mixed batches).  grid (sequences, heads, ceil(dv / 32)): a CTA
// owns 32 value columns of one head's state, each of its 8 warps 4 of them; lane r of a warp holds the
// key rows r, r + 32, ... of those columns in registers.  Tokens are staged 16 at a time in shared
// memory; within a chunk the warps run on their own (S^T q and n.q are warp-shuffle reductions: no
// block barrier per token).  The normaliser n and the stabiliser m are kept once per column slice, so
// CTAs of one head never read what another one writes.  State of slot s, laid out so that a warp's
// loads and stores are contiguous: S [slots][H][dv][dk] (key index fastest), n [slots][H][Z][dk],
// m [slots][H][Z], Z = ceil(dv / 32).  A sequence whose context is empty starts from zero, whatever
// the slot held before.
//
// `mlstm_out` then divides every head's o_t by its root mean square, multiplies by the norm
// weight and the sigmoid output gate, and rounds to the activation type.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float ml_f32(float v) { return v; }
__device__ __forceinline__ float ml_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void ml_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void ml_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kScanWarps = 8, kScanColsPerWarp = 4, kScanCols = kScanWarps * kScanColsPerWarp, kScanTok = 16;

__device__ __forceinline__ float log_sigmoid(float x) {
  // -softplus(-x), stable on both sides
  return x < 0.f ? x - log1pf(expf(x)) : -log1pf(expf(-x));
}

// EPT = key rows per lane = ceil(dk / 32)
template <typename TA, int EPT>
__global__ void __launch_bounds__(kScanWarps * 32)
mlstm_scan_kernel(const TA* __restrict__ proj, int64_t ld, int q_col, int k_col, int v_col,
                  const float* __restrict__ gates, const bf16* __restrict__ gate_bias,
                  const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                  const int32_t* __restrict__ state_slots, float* S_state, float* n_state, float* m_state,
                  float* __restrict__ o_raw, int H, int dk, int dv, float cap, float qscale) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // [16][dk]
  float* ks = qs + kScanTok * dk;                     // [16][dk]
  float* vs = ks + kScanTok * dk;                     // [16][32]
  float* gs = vs + kScanTok * kScanCols;              // [16][2]  (i, f) log gates
  const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, Z = gridDim.z;
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = z * kScanCols + warp * kScanColsPerWarp;          // this warp's first column
  float* Sp = S_state + ((size_t)slot * H + h) * dv * dk;
  float* np = n_state + (((size_t)slot * H + h) * Z + z) * dk;
  float* mp = m_state + ((size_t)slot * H + h) * Z + z;
  float S[EPT][kScanColsPerWarp], nn[EPT], m = 0.f;
  const bool fresh = ctx_lens[s] == 0;
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int row = lane + 32 * j;
#pragma unroll
    for (int c = 0; c < kScanColsPerWarp; ++c)
      S[j][c] = (!fresh && row < dk && c0 + c < dv) ? Sp[(size_t)(c0 + c) * dk + row] : 0.f;
    nn[j] = (!fresh && row < dk) ? np[row] : 0.f;
  }
  if (!fresh) m = *mp;
  const float bi = __bfloat162float(gate_bias[h]), bfg = __bfloat162float(gate_bias[H + h]);
  if (t1 - t0 == 1) {
    // a decode row: no staging and no barrier -- every lane fetches its own key / query elements, so the state
    // and the inputs are in flight together and the CTA's life is one memory round trip
    const TA* row = proj + (size_t)t0 * ld;
    float kk[EPT], qq[EPT], v[kScanColsPerWarp];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
      const int r = lane + 32 * j;
      kk[j] = r < dk ? ml_f32(row[k_col + h * dk + r]) : 0.f;
      qq[j] = r < dk ? ml_f32(row[q_col + h * dk + r]) * qscale : 0.f;
    }
#pragma unroll
    for (int c = 0; c < kScanColsPerWarp; ++c) v[c] = c0 + c < dv ? ml_f32(row[v_col + h * dv + c0 + c]) : 0.f;
    const float* gr = gates + (size_t)t0 * 2 * H;
    const float ig = cap * tanhf((gr[h] + bi) / cap), fg = log_sigmoid(cap * tanhf((gr[H + h] + bfg) / cap));
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), b = expf(ig - m_new);
    m = m_new;
    float num[kScanColsPerWarp], nq = 0.f;
#pragma unroll
    for (int c = 0; c < kScanColsPerWarp; ++c) num[c] = 0.f;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
      const float bk = b * kk[j];
      nn[j] = fmaf(a, nn[j], bk);
      nq = fmaf(nn[j], qq[j], nq);
#pragma unroll
      for (int c = 0; c < kScanColsPerWarp; ++c) {
        S[j][c] = fmaf(a, S[j][c], bk * v[c]);
        num[c] = fmaf(S[j][c], qq[j], num[c]);
      }
    }
    nq = warp_sum(nq);
#pragma unroll
    for (int c = 0; c < kScanColsPerWarp; ++c) num[c] = warp_sum(num[c]);
    const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    if (lane < kScanColsPerWarp && c0 + lane < dv) {
      float mine = num[0];
#pragma unroll
      for (int c = 1; c < kScanColsPerWarp; ++c) mine = lane == c ? num[c] : mine;
      o_raw[(size_t)t0 * H * dv + h * dv + c0 + lane] = mine / den;
    }
  } else
  for (int ch = t0; ch < t1; ch += kScanTok) {
    const int nt = min(kScanTok, t1 - ch);
    __syncthreads();                                  // every warp is done with the previous chunk
    for (int i = threadIdx.x; i < nt * dk; i += blockDim.x) {
      const int tt = i / dk, d = i - tt * dk;
      const TA* row = proj + (size_t)(ch + tt) * ld;
      qs[i] = ml_f32(row[q_col + h * dk + d]) * qscale;
      ks[i] = ml_f32(row[k_col + h * dk + d]);
    }
    for (int i = threadIdx.x; i < nt * kScanCols; i += blockDim.x) {
      const int tt = i / kScanCols, c = z * kScanCols + (i % kScanCols);
      vs[i] = c < dv ? ml_f32(proj[(size_t)(ch + tt) * ld + v_col + h * dv + c]) : 0.f;
    }
    if (threadIdx.x < nt) {
      const float* gr = gates + (size_t)(ch + threadIdx.x) * 2 * H;
      const float ai = gr[h] + bi, af = gr[H + h] + bfg;
      gs[threadIdx.x * 2] = cap * tanhf(ai / cap);
      gs[threadIdx.x * 2 + 1] = log_sigmoid(cap * tanhf(af / cap));
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float ig = gs[tt * 2], fg = gs[tt * 2 + 1];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b = expf(ig - m_new);
      m = m_new;
      float v[kScanColsPerWarp], num[kScanColsPerWarp], nq = 0.f;
#pragma unroll
      for (int c = 0; c < kScanColsPerWarp; ++c) {
        v[c] = vs[tt * kScanCols + warp * kScanColsPerWarp + c];
        num[c] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        const int row = lane + 32 * j;
        if (row < dk) {
          const float kk = ks[tt * dk + row], qq = qs[tt * dk + row];
          const float bk = b * kk;
          nn[j] = fmaf(a, nn[j], bk);
          nq = fmaf(nn[j], qq, nq);
#pragma unroll
          for (int c = 0; c < kScanColsPerWarp; ++c) {
            S[j][c] = fmaf(a, S[j][c], bk * v[c]);
            num[c] = fmaf(S[j][c], qq, num[c]);
          }
        }
      }
      nq = warp_sum(nq);
#pragma unroll
      for (int c = 0; c < kScanColsPerWarp; ++c) num[c] = warp_sum(num[c]);
      const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
      if (lane < kScanColsPerWarp && c0 + lane < dv) {
        float mine = num[0];
#pragma unroll
        for (int c = 1; c < kScanColsPerWarp; ++c) mine = lane == c ? num[c] : mine;
        o_raw[(size_t)(ch + tt) * H * dv + h * dv + c0 + lane] = mine / den;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int row = lane + 32 * j;
    if (row < dk) {
#pragma unroll
      for (int c = 0; c < kScanColsPerWarp; ++c)
        if (c0 + c < dv) Sp[(size_t)(c0 + c) * dk + row] = S[j][c];
      if (warp == 0) np[row] = nn[j];
    }
  }
  if (threadIdx.x == 0) *mp = m;
}

// ------------------------------------------------------------------------------------- chunk form
// The same recurrence for prompt portions, 16 tokens at a time, without a serial dependency between the
// tokens of a chunk.  With the state (S_0, n_0, m_0) at the chunk's start, F_t = f_1 + ... + f_t and the
// stabilisers m_t of the serial form (a 16-step scalar chain):
//     S_t^T q_t = e^{F_t + m_0 - m_t} S_0^T q_t + sum_{s<=t} e^{F_t - F_s + i_s - m_t} (k_s . q_t) v_s
//     n_t . q_t = e^{F_t + m_0 - m_t} n_0 . q_t + sum_{s<=t} e^{F_t - F_s + i_s - m_t} (k_s . q_t)
//     S_L       = e^{F_L + m_0 - m_L} S_0       + sum_s     e^{F_L - F_s + i_s - m_L} k_s v_s^T
// Every exponent is <= 0 by the definition of m.  All products and sums are fp32 FMAs; only the grouping
// of the sums differs from the serial form.  grid (sequences, heads, ceil(dv / 32)), 512 threads; the
// CTA's 32 columns of S live in shared memory for the whole portion.
constexpr int kChunkTok = 16, kChunkThreads = 512, kChunkPre = 8;   // 16 * 256 / 512

template <typename TA>
__global__ void __launch_bounds__(kChunkThreads)
mlstm_chunk_kernel(const TA* __restrict__ proj, int64_t ld, int q_col, int k_col, int v_col,
                   const float* __restrict__ gates, const bf16* __restrict__ gate_bias,
                   const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                   const int32_t* __restrict__ state_slots, float* S_state, float* n_state, float* m_state,
                   float* __restrict__ o_raw, int H, int dk, int dv, float cap, float qscale) {
  extern __shared__ float smem[];
  const int dkp = dk + 1;
  float* Ssm = smem;                                  // [dk][33]
  float* qs = Ssm + dk * 33;                          // [16][dk + 1]
  float* ks = qs + kChunkTok * dkp;                   // [16][dk + 1]
  float* vs = ks + kChunkTok * dkp;                   // [16][32]
  float* A = vs + kChunkTok * 32;                     // [16][17]   k_s . q_t
  float* nsm = A + kChunkTok * 17;                    // [dk]
  float* ig = nsm + dk;                               // [16] log input gates
  float* fg = ig + kChunkTok;                         // [16] log forget gates
  float* Fc = fg + kChunkTok;                         // [16] cumulative log forget gates
  float* mm = Fc + kChunkTok;                         // [16] stabilisers
  float* nq0 = mm + kChunkTok;                        // [16] n_0 . q_t
  float* gl = nq0 + kChunkTok;                        // [16] weights of the state update
  __shared__ float m_start;
  const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, Z = gridDim.z;
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = z * 32;
  float* Sp = S_state + ((size_t)slot * H + h) * dv * dk;
  float* np = n_state + (((size_t)slot * H + h) * Z + z) * dk;
  float* mp = m_state + ((size_t)slot * H + h) * Z + z;
  const bool fresh = ctx_lens[s] == 0;
  for (int i = tid; i < dk * 32; i += kChunkThreads) {
    const int c = i / dk, r = i - c * dk;             // r fastest: contiguous global reads
    Ssm[r * 33 + c] = (!fresh && c0 + c < dv) ? Sp[(size_t)(c0 + c) * dk + r] : 0.f;
  }
  for (int r = tid; r < dk; r += kChunkThreads) nsm[r] = fresh ? 0.f : np[r];
  if (tid == 0) m_start = fresh ? 0.f : *mp;
  const float bi = __bfloat162float(gate_bias[h]), bfg = __bfloat162float(gate_bias[H + h]);
  // The next chunk's inputs travel in registers while the current chunk is computed (kChunkPre elements of q
  // and of k per thread: key width <= 256), so the loop never waits for a global load it has just issued.
  TA rq[kChunkPre], rk[kChunkPre], rv;
  float rgi = 0.f, rgf = 0.f;
  auto fetch = [&](int ch, int nt) {
#pragma unroll
    for (int u = 0; u < kChunkPre; ++u) {
      const int i = tid + u * kChunkThreads;
      if (i < nt * dk) {
        const int tt = i / dk, d = i - tt * dk;
        const TA* row = proj + (size_t)(ch + tt) * ld;
        rq[u] = row[q_col + h * dk + d];
        rk[u] = row[k_col + h * dk + d];
      }
    }
    {
      const int tt = tid >> 5, c = c0 + (tid & 31);
      if (tt < nt && c < dv) rv = proj[(size_t)(ch + tt) * ld + v_col + h * dv + c];
    }
    if (tid < nt) {
      const float* gr = gates + (size_t)(ch + tid) * 2 * H;
      rgi = gr[h];
      rgf = gr[H + h];
    }
  };
  fetch(t0, min(kChunkTok, t1 - t0));
  for (int ch = t0; ch < t1; ch += kChunkTok) {
    const int nt = min(kChunkTok, t1 - ch);
    __syncthreads();                                  // state update of the previous chunk done, inputs free
#pragma unroll
    for (int u = 0; u < kChunkPre; ++u) {
      const int i = tid + u * kChunkThreads;
      if (i < nt * dk) {
        const int tt = i / dk, d = i - tt * dk;
        qs[tt * dkp + d] = ml_f32(rq[u]) * qscale;
        ks[tt * dkp + d] = ml_f32(rk[u]);
      }
    }
    {
      const int tt = tid >> 5, c = c0 + (tid & 31);
      vs[tid] = (tt < nt && c < dv) ? ml_f32(rv) : 0.f;
    }
    if (tid < nt) {
      ig[tid] = cap * tanhf((rgi + bi) / cap);
      fg[tid] = log_sigmoid(cap * tanhf((rgf + bfg) / cap));
    }
    if (ch + kChunkTok < t1) fetch(ch + kChunkTok, min(kChunkTok, t1 - ch - kChunkTok));
    __syncthreads();
    // (a) k_s . q_t for s <= t, n_0 . q_t, and -- one thread -- the serial scalars of the chunk
    if (tid < 256) {
      const int t = tid >> 4, sx = tid & 15;
      if (t < nt && sx <= t) {
        float acc = 0.f;
        const float* kr = ks + sx * dkp;
        const float* qr = qs + t * dkp;
        for (int r = 0; r < dk; ++r) acc = fmaf(kr[r], qr[r], acc);
        A[t * 17 + sx] = acc;
      }
    } else if (tid < 256 + kChunkTok) {
      const int t = tid - 256;
      if (t < nt) {
        float acc = 0.f;
        const float* qr = qs + t * dkp;
        for (int r = 0; r < dk; ++r) acc = fmaf(nsm[r], qr[r], acc);
        nq0[t] = acc;
      }
    } else if (tid == 288) {
      float m = m_start, F = 0.f;
      for (int t = 0; t < nt; ++t) {
        m = fmaxf(fg[t] + m, ig[t]);
        F += fg[t];
        mm[t] = m;
        Fc[t] = F;
      }
      const float mL = m, FL = F;
      for (int t = 0; t < nt; ++t) gl[t] = expf(FL - Fc[t] + ig[t] - mL);
    }
    __syncthreads();
    // (b) outputs: thread = (token = warp, column = lane)
    if (warp < nt) {
      const int t = warp;
      const float mt = mm[t], Ft = Fc[t];
      const float d0 = expf(Ft + m_start - mt);
      float acc = 0.f;
      const float* qr = qs + t * dkp;
      for (int r = 0; r < dk; ++r) acc = fmaf(Ssm[r * 33 + lane], qr[r], acc);
      float num = d0 * acc, nqv = d0 * nq0[t];
      for (int sx = 0; sx <= t; ++sx) {
        const float wa = expf(Ft - Fc[sx] + ig[sx] - mt) * A[t * 17 + sx];
        num = fmaf(wa, vs[sx * 32 + lane], num);
        nqv += wa;
      }
      const float den = fmaxf(fabsf(nqv), expf(-mt)) + 1e-6f;
      if (c0 + lane < dv) o_raw[(size_t)(ch + t) * H * dv + h * dv + c0 + lane] = num / den;
    }
    __syncthreads();
    // (c) state at the chunk's end
    {
      const float dL = expf(Fc[nt - 1] + m_start - mm[nt - 1]);
      for (int r = warp; r < dk; r += kChunkThreads / 32) {
        float acc = dL * Ssm[r * 33 + lane];
        for (int sx = 0; sx < nt; ++sx) acc = fmaf(gl[sx] * ks[sx * dkp + r], vs[sx * 32 + lane], acc);
        Ssm[r * 33 + lane] = acc;
      }
      for (int r = tid; r < dk; r += kChunkThreads) {
        float acc = dL * nsm[r];
        for (int sx = 0; sx < nt; ++sx) acc = fmaf(gl[sx], ks[sx * dkp + r], acc);
        nsm[r] = acc;
      }
    }
    __syncthreads();
    if (tid == 0) m_start = mm[nt - 1];
  }
  __syncthreads();
  for (int i = tid; i < dk * 32; i += kChunkThreads) {
    const int c = i / dk, r = i - c * dk;
    if (c0 + c < dv) Sp[(size_t)(c0 + c) * dk + r] = Ssm[r * 33 + c];
  }
  for (int r = tid; r < dk; r += kChunkThreads) np[r] = nsm[r];
  if (tid == 0) *mp = m_start;
}

// The chunk form again for key widths that are multiples of 4 (every real size), written for the instruction
// count: 16-byte shared-memory loads of the token-major q / k rows (row pitch dk + 4), and register tiles so that
// one loaded state element serves four tokens.  Phases per chunk (4 block barriers):
//   P0  staged inputs -> shared memory; the next chunk's loads are issued
//   P1  warps 0-7: A[t][s] = k_s . q_t (s <= t);  warps 8-11: n_0 . q_t;  warp 12: the serial scalars m_t, F_t
//   P2  W[t][s] = e^{F_t - F_s + i_s - m_t} A[t][s];  partial S_0^T q_t: thread = (column, 4 tokens, a quarter of the rows)
//   P3  o_t = (e^{F_t + m_0 - m_t} S_0^T q_t + sum_s W[t][s] v_s) / den_t            (thread = token, column)
//   P4  S, n <- e^{F_L + m_0 - m_L} (S, n) + sum_s g_s k_s (v_s^T, 1)               (thread = column, 4-row groups)
template <typename TA>
__global__ void __launch_bounds__(kChunkThreads)
mlstm_chunk4_kernel(const TA* __restrict__ proj, int64_t ld, int q_col, int k_col, int v_col,
                    const float* __restrict__ gates, const bf16* __restrict__ gate_bias,
                    const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                    const int32_t* __restrict__ state_slots, float* S_state, float* n_state, float* m_state,
                    float* __restrict__ o_raw, int H, int dk, int dv, float cap, float qscale) {
  extern __shared__ __align__(16) float smem[];
  const int dkp = dk + 4;
  float* qs = smem;                                   // [16][dk + 4]   (16-byte aligned rows)
  float* ks = qs + kChunkTok * dkp;                   // [16][dk + 4]
  float* Ssm = ks + kChunkTok * dkp;                  // [dk][33]
  float* vs = Ssm + dk * 33;                          // [16][32]
  float* A = vs + kChunkTok * 32;                     // [16][16]
  float* Wt = A + kChunkTok * 16;                     // [16][16]
  float* Pp = Wt + kChunkTok * 16;                    // [4][16][32] partial S_0^T q_t
  float* nsm = Pp + 4 * kChunkTok * 32;               // [dk]
  float* ig = nsm + dk;                               // [16] each from here on
  float* fg = ig + kChunkTok;
  float* Fc = fg + kChunkTok;
  float* mm = Fc + kChunkTok;
  float* nq0 = mm + kChunkTok;
  float* gl = nq0 + kChunkTok;
  __shared__ float m_start;
  const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, Z = gridDim.z;
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = z * 32;
  float* Sp = S_state + ((size_t)slot * H + h) * dv * dk;
  float* np = n_state + (((size_t)slot * H + h) * Z + z) * dk;
  float* mp = m_state + ((size_t)slot * H + h) * Z + z;
  const bool fresh = ctx_lens[s] == 0;
  for (int i = tid; i < dk * 32; i += kChunkThreads) {
    const int c = i / dk, r = i - c * dk;
    Ssm[r * 33 + c] = (!fresh && c0 + c < dv) ? Sp[(size_t)(c0 + c) * dk + r] : 0.f;
  }
  for (int r = tid; r < dk; r += kChunkThreads) nsm[r] = fresh ? 0.f : np[r];
  if (tid == 0) m_start = fresh ? 0.f : *mp;
  const float bi = __bfloat162float(gate_bias[h]), bfg = __bfloat162float(gate_bias[H + h]);
  // staging map: warp = token of the chunk, lane + 32 u = element of the head (no division)
  TA rq[kChunkPre], rk[kChunkPre], rv;
  float rgi = 0.f, rgf = 0.f;
  auto fetch = [&](int ch, int nt) {
    if (warp < nt) {
      const TA* row = proj + (size_t)(ch + warp) * ld;
#pragma unroll
      for (int u = 0; u < kChunkPre; ++u) {
        const int d = lane + 32 * u;
        if (d < dk) {
          rq[u] = row[q_col + h * dk + d];
          rk[u] = row[k_col + h * dk + d];
        }
      }
      if (c0 + lane < dv) rv = row[v_col + h * dv + c0 + lane];
    }
    if (tid < nt) {
      const float* gr = gates + (size_t)(ch + tid) * 2 * H;
      rgi = gr[h];
      rgf = gr[H + h];
    }
  };
  fetch(t0, min(kChunkTok, t1 - t0));
  for (int ch = t0; ch < t1; ch += kChunkTok) {
    const int nt = min(kChunkTok, t1 - ch);
    __syncthreads();                                  // P4 of the previous chunk is done, inputs are free
    // ---- P0
    if (warp < nt) {
#pragma unroll
      for (int u = 0; u < kChunkPre; ++u) {
        const int d = lane + 32 * u;
        if (d < dk) {
          qs[warp * dkp + d] = ml_f32(rq[u]) * qscale;
          ks[warp * dkp + d] = ml_f32(rk[u]);
        }
      }
    } else {
      // rows of a short last chunk: zeros, so that the unconditional 16-token loops below add nothing
#pragma unroll
      for (int u = 0; u < kChunkPre; ++u) {
        const int d = lane + 32 * u;
        if (d < dk) qs[warp * dkp + d] = ks[warp * dkp + d] = 0.f;
      }
    }
    vs[tid] = (warp < nt && c0 + lane < dv) ? ml_f32(rv) : 0.f;
    if (tid < nt) {
      ig[tid] = cap * tanhf((rgi + bi) / cap);
      fg[tid] = log_sigmoid(cap * tanhf((rgf + bfg) / cap));
    }
    if (ch + kChunkTok < t1) fetch(ch + kChunkTok, min(kChunkTok, t1 - ch - kChunkTok));
    __syncthreads();
    // ---- P1
    if (warp < 8) {
      const int t = tid >> 4, sx = tid & 15;
      float acc = 0.f;
      if (t < nt && sx <= t) {
        const float4* kr = reinterpret_cast<const float4*>(ks + sx * dkp);
        const float4* qr = reinterpret_cast<const float4*>(qs + t * dkp);
        for (int r4 = 0; r4 < dk / 4; ++r4) {
          const float4 a = kr[r4], b = qr[r4];
          acc = fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc))));
        }
      }
      A[t * 16 + sx] = acc;
    } else if (warp < 12) {
      const int tb = (warp - 8) * 4;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r4 = lane; r4 < dk / 4; r4 += 32) {
        const float4 nv = reinterpret_cast<const float4*>(nsm)[r4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 b = reinterpret_cast<const float4*>(qs + (tb + k) * dkp)[r4];
          acc[k] = fmaf(nv.x, b.x, fmaf(nv.y, b.y, fmaf(nv.z, b.z, fmaf(nv.w, b.w, acc[k]))));
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v = warp_sum(acc[k]);
        if (lane == 0 && tb + k < nt) nq0[tb + k] = v;
      }
    } else if (tid == 12 * 32) {
      float m = m_start, F = 0.f;
      for (int t = 0; t < nt; ++t) {
        m = fmaxf(fg[t] + m, ig[t]);
        F += fg[t];
        mm[t] = m;
        Fc[t] = F;
      }
      const float mL = m, FL = F;
      for (int t = 0; t < nt; ++t) gl[t] = expf(FL - Fc[t] + ig[t] - mL);
    }
    __syncthreads();
    // ---- P2
    if (tid < 256) {
      const int t = tid >> 4, sx = tid & 15;
      Wt[tid] = (t < nt && sx <= t) ? expf(Fc[t] - Fc[sx] + ig[sx] - mm[t]) * A[tid] : 0.f;
    }
    {
      const int tg = warp & 3, rp = warp >> 2;          // tokens 4 tg .. 4 tg + 3, row groups rp, rp + 4, ...
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r4 = rp; r4 < dk / 4; r4 += 4) {
        const int r0 = r4 * 4;
        const float s0 = Ssm[r0 * 33 + lane], s1 = Ssm[(r0 + 1) * 33 + lane], s2 = Ssm[(r0 + 2) * 33 + lane],
                    s3 = Ssm[(r0 + 3) * 33 + lane];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 b = reinterpret_cast<const float4*>(qs + (tg * 4 + k) * dkp)[r4];
          acc[k] = fmaf(s0, b.x, fmaf(s1, b.y, fmaf(s2, b.z, fmaf(s3, b.w, acc[k]))));
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) Pp[(rp * kChunkTok + tg * 4 + k) * 32 + lane] = acc[k];
    }
    __syncthreads();
    // ---- P3
    if (warp < nt) {
      const int t = warp;
      const float mt = mm[t];
      const float d0 = expf(Fc[t] + m_start - mt);
      float num = d0 * (Pp[t * 32 + lane] + Pp[(kChunkTok + t) * 32 + lane] + Pp[(2 * kChunkTok + t) * 32 + lane] +
                        Pp[(3 * kChunkTok + t) * 32 + lane]);
      float nqv = d0 * nq0[t];
      for (int sx = 0; sx <= t; ++sx) {
        const float wa = Wt[t * 16 + sx];
        num = fmaf(wa, vs[sx * 32 + lane], num);
        nqv += wa;
      }
      const float den = fmaxf(fabsf(nqv), expf(-mt)) + 1e-6f;
      if (c0 + lane < dv) o_raw[(size_t)(ch + t) * H * dv + h * dv + c0 + lane] = num / den;
    }
    // ---- P4 (reads nothing that P3 writes; Ssm and nsm were last read before the barrier above)
    {
      const float dL = expf(Fc[nt - 1] + m_start - mm[nt - 1]);
      float gv[kChunkTok];
#pragma unroll
      for (int sx = 0; sx < kChunkTok; ++sx) gv[sx] = sx < nt ? gl[sx] * vs[sx * 32 + lane] : 0.f;
      for (int r4 = warp; r4 < dk / 4; r4 += kChunkThreads / 32) {
        const int r0 = r4 * 4;
        float a0 = dL * Ssm[r0 * 33 + lane], a1 = dL * Ssm[(r0 + 1) * 33 + lane], a2 = dL * Ssm[(r0 + 2) * 33 + lane],
              a3 = dL * Ssm[(r0 + 3) * 33 + lane];
#pragma unroll
        for (int sx = 0; sx < kChunkTok; ++sx) {
          const float4 kq = reinterpret_cast<const float4*>(ks + sx * dkp)[r4];   // rows beyond nt carry gv = 0
          a0 = fmaf(kq.x, gv[sx], a0);
          a1 = fmaf(kq.y, gv[sx], a1);
          a2 = fmaf(kq.z, gv[sx], a2);
          a3 = fmaf(kq.w, gv[sx], a3);
        }
        Ssm[r0 * 33 + lane] = a0;
        Ssm[(r0 + 1) * 33 + lane] = a1;
        Ssm[(r0 + 2) * 33 + lane] = a2;
        Ssm[(r0 + 3) * 33 + lane] = a3;
      }
      for (int r = tid; r < dk; r += kChunkThreads) {
        float acc = dL * nsm[r];
        for (int sx = 0; sx < nt; ++sx) acc = fmaf(gl[sx], ks[sx * dkp + r], acc);
        nsm[r] = acc;
      }
    }
    __syncthreads();
    if (tid == 0) m_start = mm[nt - 1];
  }
  __syncthreads();
  for (int i = tid; i < dk * 32; i += kChunkThreads) {
    const int c = i / dk, r = i - c * dk;
    if (c0 + c < dv) Sp[(size_t)(c0 + c) * dk + r] = Ssm[r * 33 + c];
  }
  for (int r = tid; r < dk; r += kChunkThreads) np[r] = nsm[r];
  if (tid == 0) *mp = m_start;
}

template <typename TA>
static int launch_chunk(const void* proj, int64_t ld, int q_col, int k_col, int v_col, const float* gates,
                        const void* gate_bias, const int32_t* cu_seq, const int32_t* ctx_lens,
                        const int32_t* state_slots, float* S_state, float* n_state, float* m_state, float* o_raw,
                        int n_seq, int H, int dk, int dv, float cap, float qscale, cudaStream_t s) {
  dim3 grid(n_seq, H, (dv + 31) / 32);
  const size_t smem = sizeof(float) * ((size_t)dk * 33 + 2 * kChunkTok * (dk + 1) + kChunkTok * 32 + kChunkTok * 17 + dk +
                                       6 * kChunkTok);
  if (smem > 200 * 1024 || dk > kChunkPre * kChunkThreads / kChunkTok) {
    b200_set_error("mlstm_scan: key width %d exceeds %d", dk, kChunkPre * kChunkThreads / kChunkTok);
    return B200_ERR_UNSUPPORTED;
  }
  if (dk % 4 == 0) {
    const size_t smem4 = sizeof(float) * ((size_t)2 * kChunkTok * (dk + 4) + (size_t)dk * 33 + kChunkTok * 32 +
                                          2 * kChunkTok * 16 + 4 * kChunkTok * 32 + dk + 6 * kChunkTok);
    if (smem4 > 48 * 1024)
      cudaFuncSetAttribute(mlstm_chunk4_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
    mlstm_chunk4_kernel<TA><<<grid, kChunkThreads, smem4, s>>>((const TA*)proj, ld, q_col, k_col, v_col, gates,
                                                              (const bf16*)gate_bias, cu_seq, ctx_lens, state_slots,
                                                              S_state, n_state, m_state, o_raw, H, dk, dv, cap, qscale);
    return b200_check_launch("b200_mlstm_scan(chunk4)");
  }
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(mlstm_chunk_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  mlstm_chunk_kernel<TA><<<grid, kChunkThreads, smem, s>>>((const TA*)proj, ld, q_col, k_col, v_col, gates,
                                                          (const bf16*)gate_bias, cu_seq, ctx_lens, state_slots, S_state,
                                                          n_state, m_state, o_raw, H, dk, dv, cap, qscale);
  return b200_check_launch("b200_mlstm_scan(chunk)");
}

// one warp per (token, head), 8 warps per CTA: o / rms(o) * w * sigmoid(gate); the head is read once
constexpr int kOutWarps = 8, kOutPer = 8;   // value width <= 256
template <typename TA>
__global__ void __launch_bounds__(kOutWarps * 32)
mlstm_out_kernel(const float* __restrict__ o_raw, const TA* __restrict__ proj, int64_t ld, int gate_col,
                 const bf16* __restrict__ norm_w, TA* out, int64_t ldo, int T, int H, int dv, float eps) {
  const int idx = blockIdx.x * kOutWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= T * H) return;
  const int t = idx / H, h = idx - t * H;
  const float* o = o_raw + (size_t)t * H * dv + h * dv;
  float x[kOutPer];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kOutPer; ++i) {
    const int d = lane + 32 * i;
    x[i] = d < dv ? o[d] : 0.f;
    ss = fmaf(x[i], x[i], ss);
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)dv + eps);
#pragma unroll
  for (int i = 0; i < kOutPer; ++i) {
    const int d = lane + 32 * i;
    if (d < dv) {
      float v = x[i] * r * __bfloat162float(norm_w[h * dv + d]);
      if (gate_col >= 0) {
        const float gv = ml_f32(proj[(size_t)t * ld + gate_col + h * dv + d]);
        v *= 1.0f / (1.0f + expf(-gv));
      }
      ml_store(out + (size_t)t * ldo + h * dv + d, v);
    }
  }
}

template <typename TA>
static int launch_scan(const void* proj, int64_t ld, int q_col, int k_col, int v_col, const float* gates,
                       const void* gate_bias, const int32_t* cu_seq, const int32_t* ctx_lens,
                       const int32_t* state_slots, float* S_state, float* n_state, float* m_state, float* o_raw,
                       int n_seq, int H, int dk, int dv, float cap, float qscale, cudaStream_t s) {
  const int Z = (dv + kScanCols - 1) / kScanCols;
  dim3 grid(n_seq, H, Z);
  const size_t smem = sizeof(float) * ((size_t)2 * kScanTok * dk + kScanTok * kScanCols + kScanTok * 2);
  const int ept = (dk + 31) / 32;
#define B200_SCAN(E)                                                                                              \
  do {                                                                                                            \
    if (smem > 48 * 1024)                                                                                         \
      cudaFuncSetAttribute(mlstm_scan_kernel<TA, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    mlstm_scan_kernel<TA, E><<<grid, kScanWarps * 32, smem, s>>>(                                                 \
        (const TA*)proj, ld, q_col, k_col, v_col, gates, (const bf16*)gate_bias, cu_seq, ctx_lens, state_slots,  \
        S_state, n_state, m_state, o_raw, H, dk, dv, cap, qscale);                                                \
  } while (0)
  if (ept <= 1) B200_SCAN(1);
  else if (ept <= 2) B200_SCAN(2);
  else if (ept <= 4) B200_SCAN(4);
  else if (ept <= 8) B200_SCAN(8);
  else {
    b200_set_error("mlstm_scan: key width %d exceeds 256", dk);
    return B200_ERR_UNSUPPORTED;
  }
#undef B200_SCAN
  return b200_check_launch("b200_mlstm_scan");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_mlstm_state_slices(int dv) { return (dv + kScanCols - 1) / kScanCols; }

extern "C" int b200_mlstm_scan(const void* proj, int f32, int64_t ld, int q_col, int k_col, int v_col,
                               const float* gates, const void* gate_bias, const int32_t* cu_seq,
                               const int32_t* ctx_lens, const int32_t* state_slots, float* S_state, float* n_state,
                               float* m_state, float* o_raw, int n_seq, int H, int dk, int dv, float cap, float qscale,
                               int max_len, void* stream) {
  B200_REQUIRE(n_seq >= 0 && H > 0 && dk > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad shape H=%d dk=%d dv=%d", H, dk,
               dv);
  if (n_seq == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (max_len >= 4) {   // prompt portions: the chunk form; single rows and tiny portions: the serial form
    if (f32)
      return launch_chunk<float>(proj, ld, q_col, k_col, v_col, gates, gate_bias, cu_seq, ctx_lens, state_slots, S_state,
                                 n_state, m_state, o_raw, n_seq, H, dk, dv, cap, qscale, s);
    return launch_chunk<bf16>(proj, ld, q_col, k_col, v_col, gates, gate_bias, cu_seq, ctx_lens, state_slots, S_state,
                              n_state, m_state, o_raw, n_seq, H, dk, dv, cap, qscale, s);
  }
  if (f32)
    return launch_scan<float>(proj, ld, q_col, k_col, v_col, gates, gate_bias, cu_seq, ctx_lens, state_slots, S_state,
                              n_state, m_state, o_raw, n_seq, H, dk, dv, cap, qscale, s);
  return launch_scan<bf16>(proj, ld, q_col, k_col, v_col, gates, gate_bias, cu_seq, ctx_lens, state_slots, S_state,
                           n_state, m_state, o_raw, n_seq, H, dk, dv, cap, qscale, s);
}

extern "C" int b200_mlstm_out(const float* o_raw, const void* proj, int f32, int64_t ld, int gate_col,
                              const void* norm_w, void* out, int64_t ldo, int T, int H, int dv, float eps,
                              void* stream) {
  B200_REQUIRE(T >= 0 && H > 0 && dv > 0 && dv <= 32 * kOutPer, "mlstm_out: bad shape (value width <= %d)", 32 * kOutPer);
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = (int)(((size_t)T * H + kOutWarps - 1) / kOutWarps);
  if (f32)
    mlstm_out_kernel<float><<<grid, kOutWarps * 32, 0, s>>>(o_raw, (const float*)proj, ld, gate_col, (const bf16*)norm_w,
                                                            (float*)out, ldo, T, H, dv, eps);
  else
    mlstm_out_kernel<bf16><<<grid, kOutWarps * 32, 0, s>>>(o_raw, (const bf16*)proj, ld, gate_col, (const bf16*)norm_w,
                                                           (bf16*)out, ldo, T, H, dv, eps);
  return b200_check_launch("b200_mlstm_out");
}
