// Latent attention in the absorbed form on the tensor cores (bf16): every head of a query row scores against
// the SAME cached row per token,  [latent: R | rotated key part: dr]  (W = R + dr wide), and takes the first R
// entries of those rows as its values.  So the heads are the M rows of the matrix products: a CTA owns 32
// (query row, head) pairs -- two m-tiles of 16; 32 heads of one row, or 32 / HB rows of HB heads when the model has
// fewer heads -- and streams the sequence's cache rows ONCE for all of them, 32 keys at a time with cp.async
// (double-buffered while two CTAs still fit an SM; with wide rows one buffer per CTA, and the two resident CTAs
// overlap each other's fetches).  Key rows land in shared memory with a 16-byte pad per row, conflict-free for ldmatrix.
//
// Per 32-key block, with 4 warps per m-tile:
//   S:   warp w scores its tile's 16 pairs against keys [8 w, 8 w + 8)       (mma.sync m16n8k16, k over W)
//   max: the block's row maxima are exchanged through shared memory; every warp keeps the same running
//        maximum m and rescales its accumulators by 2^(m_old - m_new)       (fp32, base-2 domain)
//   P:   exp2(S - m) is written to shared memory as bf16 [16][32]; each warp keeps the fp32 sum of its own
//        8 columns (the four partial sums meet at the end)
//   O:   warp w accumulates O[16][R/4 columns from w R/4] += P V, V = the block's rows read transposed.
// The end: l = sum of the partial sums (+ exp(sink_h - m): a learned per-head term of the denominator with no key
// and no value), O / l, one rounding to bf16.  Causal: pair (row i, head) sees keys 0 .. p0 + i.
// One kernel serves prompt portions (tile list, as the other prefill kernels) and single new rows (decode).
// Shapes: W a multiple of 16, R a multiple of 64 up to 512; anything else runs on the generic kernels.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

#include <math.h>

namespace b200 {

constexpr int kLaTiles = 2, kLaTileWarps = 4, kLaWarps = kLaTiles * kLaTileWarps;   // 2 m-tiles of 16 pairs, 4 warps each
constexpr int kLaKeys = 32, kLaRows = 16 * kLaTiles;
constexpr int kLaPPitch = kLaKeys * 2 + 16;          // bytes per row of a probability tile

struct LaArgs {
  const bf16* qa;
  int64_t ldq;
  const bf16* cache;
  int page;
  const int32_t* block_table;
  int max_blocks;
  const int32_t* cu_q;        // prompt portions: tile list (tile_seq != NULL)
  const int32_t* ctx_lens;
  const int32_t* tile_seq;
  const int32_t* tile_q0;
  const int32_t* seq_lens;    // single rows: row b sees keys [0, seq_lens[b])
  const float* sink;
  bf16* out;
  int64_t ldo;
  int H, W, R, HB;            // HB heads per CTA (a power of two <= 32)
  int QR;                     // query rows per CTA (HB * QR <= 32 pairs)
  float scale_log2;
  int page_shift;             // log2(page)
  int nsplit;                 // single rows only: the keys are cut into nsplit ranges (grid.z), partial results
  float* ws;                  //   [row][head][split][R + 2] = unnormalised O, running maximum, partial sum -> merge kernel
  int nbuf;                   // key buffers: 2 = the next block is fetched while this one is used; 1 (wide rows) = one
                              // buffer, the two CTAs of an SM overlap each other's fetches instead
};

template <int NT>   // n-tiles (8 columns) of the output per warp: R = 32 NT
__global__ void __launch_bounds__(kLaWarps * 32, 2)
latent_attn_mma_kernel(LaArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int W = a.W, R = a.R, HB = a.HB, QR = a.QR;
  const int pitch = W * 2 + 16;                       // bytes; W / 8 chunks + 1: odd, so 8 rows hit 8 bank groups
  uint8_t* q_s = smem;                                // [32][pitch]
  uint8_t* k_s = q_s + kLaRows * pitch;               // [nbuf][32][pitch]
  uint8_t* p_s = k_s + a.nbuf * kLaKeys * pitch;      // [2 tiles][16][kLaPPitch]
  float* red_m = reinterpret_cast<float*>(p_s + kLaRows * kLaPPitch);   // [2 tiles][4 warps][16]
  float* red_l = red_m + kLaWarps * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = warp / kLaTileWarps, wq = warp % kLaTileWarps;          // m-tile, and this warp's place in it
  const int h0 = blockIdx.y * HB;

  int s, nq, p0;
  size_t grow0;
  if (a.tile_seq != nullptr) {
    s = a.tile_seq[blockIdx.x];
    const int q0 = a.tile_q0[blockIdx.x] + QR * blockIdx.z;
    const int row0 = a.cu_q[s], qlen = a.cu_q[s + 1] - row0;
    if (q0 >= qlen) return;
    nq = min(QR, qlen - q0);
    p0 = a.ctx_lens[s] + q0;
    grow0 = (size_t)(row0 + q0);
  } else {
    s = blockIdx.x;
    nq = 1;
    p0 = a.seq_lens[s] - 1;
    grow0 = (size_t)s;
    if (p0 < 0) {                                      // a padding row of a captured batch: defined output, no keys
      for (int i = threadIdx.x; i < HB * R; i += blockDim.x) {
        const int h = h0 + i / R;
        if (h < a.H) a.out[grow0 * a.ldo + (size_t)h * R + i % R] = __float2bfloat16_rn(0.f);
      }
      if (a.nsplit > 1 && threadIdx.x < HB && h0 + threadIdx.x < a.H) {     // an empty range for the merge kernel
        float* w = a.ws + (((size_t)s * a.H + h0 + threadIdx.x) * a.nsplit + blockIdx.z) * (R + 2);
        w[R] = -INFINITY;
        w[R + 1] = 0.f;
      }
      return;
    }
  }
  const int kv_end = p0 + nq;
  int blk_begin = 0, n_blk = (kv_end + kLaKeys - 1) / kLaKeys;
  if (a.tile_seq == nullptr && a.nsplit > 1) {         // this CTA's range of key blocks (it may be empty)
    const int per = (n_blk + a.nsplit - 1) / a.nsplit;
    blk_begin = min(n_blk, (int)blockIdx.z * per);
    n_blk = min(n_blk, blk_begin + per);
  }
  const int32_t* bt = a.block_table + (size_t)s * a.max_blocks;
  const int cpr = W / 8;                               // 16-byte chunks per row

  // a warp copies whole key rows (rows w, w + 8, ...): one page lookup per row, lanes take the row's 16-byte chunks
  auto issue = [&](int blk) {
    uint8_t* dst = k_s + (a.nbuf == 2 ? (blk & 1) : 0) * kLaKeys * pitch;
    const int k0 = blk * kLaKeys;
#pragma unroll
    for (int r = warp; r < kLaKeys; r += kLaWarps) {
      const int key = k0 + r;
      const bool live = key < kv_end;
      const int kk = live ? key : 0;
      const int pg = kk >> a.page_shift;
      const bf16* src = a.cache + ((size_t)__ldg(bt + pg) * a.page + (kk - (pg << a.page_shift))) * W;
      uint8_t* d = dst + r * pitch;
      for (int c = lane; c < cpr; c += 32) cp_async_16_zfill(d + c * 16, src + c * 8, live);
    }
  };
  if (blk_begin < n_blk) issue(blk_begin);
  cp_async_commit();

  // ---- the 32 (row, head) pairs' absorbed queries: pair i = query row i / HB, head h0 + i % HB
  for (int ci = threadIdx.x; ci < kLaRows * cpr; ci += blockDim.x) {
    const int i = ci / cpr, c = ci - i * cpr;
    const int qi = i / HB, h = h0 + i % HB;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qi < nq && h < a.H) v = ld_v4(a.qa + (grow0 + qi) * a.ldq + (size_t)h * W + c * 8);
    *reinterpret_cast<uint4*>(q_s + i * pitch + c * 16) = v;
  }

  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;    // this lane's two pairs
  const int t0 = lane >> 2, t1 = t0 + 8;                // ... and their rows inside the m-tile
  const int lim0 = p0 + r0 / HB, lim1 = p0 + r1 / HB;   // last visible key of each
  const bool tile_live = (mt * 16) / HB < nq;           // an m-tile whose first pair is beyond the rows has none
  const uint32_t q_base = smem_u32(q_s) + mt * 16 * pitch, p_base = smem_u32(p_s) + mt * 16 * kLaPPitch;
  float* rm = red_m + mt * kLaTileWarps * 16;
  float* rl = red_l + mt * kLaTileWarps * 16;
  const int ai = lane >> 3, arr = lane & 7;
  const int a_row = arr + (ai & 1) * 8;                 // A-operand (row-major 16 x 16) ldmatrix addressing
  const int v_tok = arr + (ai & 1) * 8;                 // B-operand of P V: keys as k (transposed load)
  const int ks_n = W / 16;
  const int col_chunk0 = wq * (R / 4) / 8;              // first 16-byte chunk of this warp's output columns

  const bool two = a.nbuf == 2;
  for (int blk = blk_begin; blk < n_blk; ++blk) {
    if (two) {
      if (blk + 1 < n_blk) issue(blk + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                                    // block blk (and, first time, the queries) visible to all
    const uint32_t k_base = smem_u32(k_s + (two ? (blk & 1) : 0) * kLaKeys * pitch);

    // S: this m-tile's 16 pairs x this warp's 8 keys.  One ldmatrix.x4 brings the key operand of TWO k-steps
    // (matrices: step ks low / high half, step ks + 1 low / high half); two accumulators alternate.
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    if (tile_live) {
      const uint32_t qa_addr = q_base + a_row * pitch + (ai >> 1) * 16;
      const uint32_t kb_addr = k_base + (wq * 8 + arr) * pitch + ai * 16;
      int ks = 0;
#pragma unroll 2
      for (; ks + 1 < ks_n; ks += 2) {
        uint32_t qf[4], qg[4], b0, b1, b2, b3;
        ldsm_x4(kb_addr + ks * 32, b0, b1, b2, b3);
        ldsm_x4(qa_addr + ks * 32, qf[0], qf[1], qf[2], qf[3]);
        ldsm_x4(qa_addr + ks * 32 + 32, qg[0], qg[1], qg[2], qg[3]);
        mma_bf16_16816(sa, qf, b0, b1);
        mma_bf16_16816(sb, qg, b2, b3);
      }
      if (ks < ks_n) {                                  // an odd last step: the upper two matrices re-read the lower ones
        uint32_t qf[4], b0, b1, b2, b3;
        ldsm_x4(kb_addr + ks * 32 - (ai >> 1) * 32, b0, b1, b2, b3);
        ldsm_x4(qa_addr + ks * 32, qf[0], qf[1], qf[2], qf[3]);
        mma_bf16_16816(sa, qf, b0, b1);
      }
    }
    float sc[4];
    const int key0 = blk * kLaKeys + wq * 8 + 2 * (lane & 3);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + (e & 1);
      const bool seen = key <= (e < 2 ? lim0 : lim1);
      const float v = seen ? (sa[e] + sb[e]) * a.scale_log2 : -INFINITY;
      sc[e] = v;
      if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if ((lane & 3) == 0) {
      rm[wq * 16 + t0] = mx0;
      rm[wq * 16 + t1] = mx1;
    }
    __syncthreads();
    float mn0 = m0, mn1 = m1;
#pragma unroll
    for (int w = 0; w < kLaTileWarps; ++w) {
      mn0 = fmaxf(mn0, rm[w * 16 + t0]);
      mn1 = fmaxf(mn1, rm[w * 16 + t1]);
    }
    // a range's first block has a key that every pair sees (key 0, or any key of a single row), so both maxima are finite
    const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    sc[0] = exp2f(sc[0] - mn0); sc[1] = exp2f(sc[1] - mn0);
    sc[2] = exp2f(sc[2] - mn1); sc[3] = exp2f(sc[3] - mn1);
    {
      const uint32_t colb = (uint32_t)(wq * 8 + 2 * (lane & 3)) * 2u;
      st_shared_u32(p_base + t0 * kLaPPitch + colb, pack_bf16(sc[0], sc[1]));
      st_shared_u32(p_base + t1 * kLaPPitch + colb, pack_bf16(sc[2], sc[3]));
    }
    l0 = l0 * a0 + (sc[0] + sc[1]);
    l1 = l1 * a1 + (sc[2] + sc[3]);
#pragma unroll
    for (int t = 0; t < NT; ++t) { o[t][0] *= a0; o[t][1] *= a0; o[t][2] *= a1; o[t][3] *= a1; }
    __syncthreads();                                    // the probability tiles are written

    // O[16][this warp's R/4 columns] += P (16 x 32) V (32 x R/4)
    if (tile_live) {
#pragma unroll
      for (int kk = 0; kk < kLaKeys / 16; ++kk) {
        uint32_t pa[4];
        ldsm_x4(p_base + a_row * kLaPPitch + (2 * kk + (ai >> 1)) * 16, pa[0], pa[1], pa[2], pa[3]);
        const uint32_t v_addr = k_base + (kk * 16 + v_tok) * pitch + (col_chunk0 + (ai >> 1)) * 16;
#pragma unroll
        for (int c = 0; c < NT; c += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_addr + c * 16, b0, b1, b2, b3);
          mma_bf16_16816(o[c], pa, b0, b1);
          mma_bf16_16816(o[c + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();                                    // this key buffer and the probability tiles are free again
    if (!two && blk + 1 < n_blk) {
      issue(blk + 1);
      cp_async_commit();
    }
  }
  cp_async_wait<0>();

  // ---- partial sums of the tile's four warps, the sink, the division
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if ((lane & 3) == 0) {
    rl[wq * 16 + t0] = l0;
    rl[wq * 16 + t1] = l1;
  }
  __syncthreads();
  float den0 = 0.f, den1 = 0.f;
#pragma unroll
  for (int w = 0; w < kLaTileWarps; ++w) {
    den0 += rl[w * 16 + t0];
    den1 += rl[w * 16 + t1];
  }
  const int qi0 = r0 / HB, hh0 = h0 + r0 % HB, qi1 = r1 / HB, hh1 = h0 + r1 % HB;
  const bool ok0 = qi0 < nq && hh0 < a.H, ok1 = qi1 < nq && hh1 < a.H;
  if (a.tile_seq == nullptr && a.nsplit > 1) {         // park (O, m, l) of this key range; the merge kernel finishes
    const int cbs = wq * (R / 4) + 2 * (lane & 3);
    float* w0 = a.ws + (((size_t)s * a.H + hh0) * a.nsplit + blockIdx.z) * (R + 2);
    float* w1 = a.ws + (((size_t)s * a.H + hh1) * a.nsplit + blockIdx.z) * (R + 2);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (ok0) { w0[cbs + t * 8] = o[t][0]; w0[cbs + t * 8 + 1] = o[t][1]; }
      if (ok1) { w1[cbs + t * 8] = o[t][2]; w1[cbs + t * 8 + 1] = o[t][3]; }
    }
    if (wq == 0 && (lane & 3) == 0) {
      if (ok0) { w0[R] = m0; w0[R + 1] = den0; }
      if (ok1) { w1[R] = m1; w1[R + 1] = den1; }
    }
    return;
  }
  if (a.sink != nullptr) {
    if (ok0) den0 += exp2f(a.sink[hh0] * 1.4426950408889634f - m0);
    if (ok1) den1 += exp2f(a.sink[hh1] * 1.4426950408889634f - m1);
  }
  const float inv0 = den0 > 0.f ? 1.f / den0 : 0.f, inv1 = den1 > 0.f ? 1.f / den1 : 0.f;
  const int cb = wq * (R / 4) + 2 * (lane & 3);
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    if (ok0)
      *reinterpret_cast<uint32_t*>(a.out + (grow0 + qi0) * a.ldo + (size_t)hh0 * R + cb + t * 8) =
          pack_bf16(o[t][0] * inv0, o[t][1] * inv0);
    if (ok1)
      *reinterpret_cast<uint32_t*>(a.out + (grow0 + qi1) * a.ldo + (size_t)hh1 * R + cb + t * 8) =
          pack_bf16(o[t][2] * inv1, o[t][3] * inv1);
  }
}

// out[b][h] = sum_s O_s 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink_h log2 e - M)),  M = max_s m_s; empty ranges
// (m_s = -inf) are skipped.
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ ws, const float* __restrict__ sink, bf16* out, int64_t ldo, int H,
                         int R, int nsplit) {
  const int b = blockIdx.x, h = blockIdx.y;
  const float* p = ws + ((size_t)b * H + h) * nsplit * (R + 2);
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, p[(size_t)s * (R + 2) + R]);
  float den = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = p[(size_t)s * (R + 2) + R];
    if (ms > -INFINITY) den += p[(size_t)s * (R + 2) + R + 1] * exp2f(ms - M);
  }
  if (sink != nullptr && M > -INFINITY) den += exp2f(sink[h] * 1.4426950408889634f - M);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = p[(size_t)s * (R + 2) + R];
      if (ms > -INFINITY) acc += p[(size_t)s * (R + 2) + d] * exp2f(ms - M);
    }
    out[(size_t)b * ldo + (size_t)h * R + d] = __float2bfloat16_rn(acc * inv);
  }
}

static size_t la_smem_bytes(int W, int nbuf) {
  const size_t pitch = (size_t)W * 2 + 16;
  return kLaRows * pitch + nbuf * kLaKeys * pitch + kLaRows * kLaPPitch + 2 * kLaWarps * 16 * sizeof(float);
}

// two buffers while two CTAs still fit an SM's shared memory with them, else one
static int la_nbuf(int W) { return la_smem_bytes(W, 2) <= 100 * 1024 ? 2 : 1; }

static int la_log2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

static int la_heads_per_cta(int H) {
  int hb = 1;
  while (hb * 2 <= H && hb < kLaRows) hb *= 2;
  return hb;
}

template <int NT>
static int la_launch(const LaArgs& a, dim3 grid, cudaStream_t s) {
  const size_t smem = la_smem_bytes(a.W, a.nbuf);
  static size_t attr = 0;
  if (smem > attr) {
    cudaError_t e = cudaFuncSetAttribute(latent_attn_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      b200_set_error("latent_attn: cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
      return B200_ERR_CUDA;
    }
    attr = smem;
  }
  latent_attn_mma_kernel<NT><<<grid, kLaWarps * 32, smem, s>>>(a);
  return b200_check_launch("b200_latent_attn");
}

static int la_dispatch(const LaArgs& a, dim3 grid, cudaStream_t s) {
  switch (a.R / 32) {
    case 2: return la_launch<2>(a, grid, s);
    case 4: return la_launch<4>(a, grid, s);
    case 6: return la_launch<6>(a, grid, s);
    case 8: return la_launch<8>(a, grid, s);
    case 12: return la_launch<12>(a, grid, s);
    case 16: return la_launch<16>(a, grid, s);
    default:
      b200_set_error("latent_attn: latent width %d is not covered (64, 128, 192, 256, 384, 512)", a.R);
      return B200_ERR_UNSUPPORTED;
  }
}

}  // namespace b200

using namespace b200;

// 1 when the tensor-core kernel takes this shape (bf16 only; the caller checks the element type).
extern "C" int b200_latent_attn_covers(int H, int R, int dr) {
  const int W = R + dr;
  if (H <= 0 || R <= 0 || dr < 0 || W % 16 != 0) return 0;
  if (!(R == 64 || R == 128 || R == 192 || R == 256 || R == 384 || R == 512)) return 0;
  return la_smem_bytes(W, la_nbuf(W)) <= 220 * 1024 ? 1 : 0;
}

static int la_check(const void* qa, int64_t ldq, const void* cache, int64_t ldo, int H, int R, int dr) {
  B200_REQUIRE(b200_latent_attn_covers(H, R, dr), "latent_attn: shape H=%d R=%d dr=%d is not covered", H, R, dr);
  B200_REQUIRE(ldq % 8 == 0 && (reinterpret_cast<uintptr_t>(qa) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
                   ldo % 2 == 0,
               "latent_attn: 16-byte aligned query and cache rows required");
  return B200_OK;
}

extern "C" int b200_latent_attn_prefill(const void* qa, int64_t ldq, const void* cache, int page,
                                        const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                                        const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0,
                                        int n_tiles, int tile_rows, const float* sink, void* out, int64_t ldo, int H, int R,
                                        int dr, float scale, void* stream) {
  if (int rc = la_check(qa, ldq, cache, ldo, H, R, dr)) return rc;
  B200_REQUIRE(tile_rows > 0 && tile_rows % 16 == 0, "latent_attn_prefill: tiles of %d rows (multiples of 16)", tile_rows);
  B200_REQUIRE(page > 0 && (page & (page - 1)) == 0, "latent_attn_prefill: the page size %d is not a power of two", page);
  if (n_tiles <= 0) return B200_OK;
  const int hb = la_heads_per_cta(H);
  const int qr = kLaRows / hb < 16 ? kLaRows / hb : 16;       // query rows per CTA: a divisor of the 16-row tile pieces
  LaArgs a{(const bf16*)qa, ldq, (const bf16*)cache, page, block_table, max_blocks, cu_q, ctx_lens, tile_seq, tile_q0, nullptr,
           sink, (bf16*)out, ldo, H, R + dr, R, hb, qr, scale * 1.4426950408889634f, la_log2(page), 1, nullptr, la_nbuf(R + dr)};
  dim3 grid(n_tiles, (H + hb - 1) / hb, tile_rows / qr);
  return la_dispatch(a, grid, (cudaStream_t)stream);
}

// Key ranges per row worth launching for B rows of H heads whose sequences are at most max_len long: enough CTAs for
// two per SM, at least 256 keys per range, at most 16 ranges.
extern "C" int b200_latent_attn_decode_splits(int B, int H, int max_len) {
  const int hb = la_heads_per_cta(H);
  const int ctas = B * ((H + hb - 1) / hb);
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  int n = ctas > 0 ? (2 * sms) / ctas : 1;
  const int by_len = (max_len + 255) / 256;
  if (n > by_len) n = by_len;
  if (n > 16) n = 16;
  return n < 1 ? 1 : n;
}

extern "C" size_t b200_latent_attn_decode_workspace_bytes(int B, int H, int R, int nsplit) {
  return nsplit > 1 ? (size_t)B * H * nsplit * (R + 2) * sizeof(float) : 0;
}

extern "C" int b200_latent_attn_decode(const void* qa, int64_t ldq, const void* cache, int page,
                                       const int32_t* block_table, int max_blocks, const int32_t* seq_lens, int B,
                                       const float* sink, void* out, int64_t ldo, int H, int R, int dr, float scale,
                                       int nsplit, void* workspace, void* stream) {
  if (int rc = la_check(qa, ldq, cache, ldo, H, R, dr)) return rc;
  B200_REQUIRE(page > 0 && (page & (page - 1)) == 0, "latent_attn_decode: the page size %d is not a power of two", page);
  B200_REQUIRE(nsplit >= 1 && nsplit <= 16 && (nsplit == 1 || workspace != nullptr), "latent_attn_decode: %d key ranges need a workspace", nsplit);
  if (B <= 0) return B200_OK;
  const int hb = la_heads_per_cta(H);
  LaArgs a{(const bf16*)qa, ldq, (const bf16*)cache, page, block_table, max_blocks, nullptr, nullptr, nullptr, nullptr, seq_lens,
           sink, (bf16*)out, ldo, H, R + dr, R, hb, 1, scale * 1.4426950408889634f, la_log2(page), nsplit, (float*)workspace,
           la_nbuf(R + dr)};
  dim3 grid(B, (H + hb - 1) / hb, nsplit);
  if (int rc = la_dispatch(a, grid, (cudaStream_t)stream)) return rc;
  if (nsplit > 1) {
    latent_attn_merge_kernel<<<dim3(B, H), 128, 0, (cudaStream_t)stream>>>((const float*)workspace, sink, (bf16*)out, ldo, H, R,
                                                                          nsplit);
    return b200_check_launch("b200_latent_attn_decode(merge)");
  }
  return B200_OK;
}
