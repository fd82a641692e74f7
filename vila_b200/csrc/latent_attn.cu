// Latent attention over a paged cache that stores ONE latent row c_j per token (no per-head keys
// or values): every query head attends to the same rows, keys and values are both c_j.  The
// per-head key expansion is folded into the query beforehand (q'_h = W_uk,h^T q_h) and the value
// expansion is applied to the result afterwards (o_h = W_uv,h sum_j p_j c_j), so the cache traffic
// per token is R numbers instead of H * (dim + vdim).
//   softmax with a sink: the running (max, sum) pair starts at (sink_h, 1) instead of (-inf, 0),
//   which puts exp(sink_h) into the denominator exactly once, with no key and no value.
// Scores, softmax and accumulation are fp32.  Two kernels:
//   latent_attn_tile_kernel   up to 16 consecutive rows of one sequence per CTA (prompt portions)
//   latent_attn_decode_kernel one row per CTA, all 256 threads spread over keys (decoded tokens)
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int BQ = 16;   // query rows per tile
constexpr int BKEY = 32; // keys per iteration
constexpr float kNegBig = -1e30f;

__device__ __forceinline__ size_t cache_row(const int32_t* pt, int page, int j) {
  return static_cast<size_t>(pt[j / page]) * page + (j % page);
}

// thread (i = tid / 16, l = tid % 16): scores of query i for keys l and l + 16 of the block, then the
// accumulator columns l, l + 16, ... of query i.
template <int KK>
__global__ void __launch_bounds__(kThreads) latent_attn_tile_kernel(const vila_latent_attn_params p) {
  extern __shared__ float sm[];
  const int R = p.R, RS = R + 1;
  float* Qs = sm;                 // [BQ][R]
  float* Cs = Qs + BQ * R;        // [BKEY][R + 1]
  float* Ps = Cs + BKEY * RS;     // [BQ][BKEY]
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x, i = tid >> 4, l = tid & 15;
  const int h = blockIdx.y;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row0 = tile[0], n = tile[1], pos0 = tile[2], slot = tile[3];
  const int32_t* pt = p.page_tables + static_cast<size_t>(slot) * p.pt_stride;
  const size_t ldq = static_cast<size_t>(p.H) * R;
  for (int idx = tid; idx < BQ * R; idx += kThreads) {
    const int qi = idx / R, k = idx % R;
    Qs[idx] = qi < n ? p.q[(row0 + qi) * ldq + static_cast<size_t>(h) * R + k] * p.scale : 0.f;
  }
  float m = p.sink ? p.sink[h] : kNegBig;
  float lsum = p.sink ? 1.0f : 0.0f;
  float acc[KK];
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) acc[kk] = 0.f;
  const int nkeys = pos0 + n;
  const int my_last = pos0 + i;  // last visible key of query i
  for (int j0 = 0; j0 < nkeys; j0 += BKEY) {
    __syncthreads();  // Qs ready (first pass) / previous block consumed
    for (int idx = tid; idx < BKEY * R; idx += kThreads) {
      const int jj = idx / R, k = idx % R, j = j0 + jj;
      Cs[jj * RS + k] = j < nkeys ? ld_any(p.cache, p.cache_dtype, cache_row(pt, p.page, j) * R + k) : 0.f;
    }
    __syncthreads();
    float s0 = 0.f, s1 = 0.f;
    const float* qr = Qs + i * R;
    const float* c0 = Cs + l * RS;
    const float* c1 = Cs + (l + 16) * RS;
    for (int k = 0; k < R; ++k) {
      const float qv = qr[k];
      s0 = fmaf(qv, c0[k], s0);
      s1 = fmaf(qv, c1[k], s1);
    }
    const bool v0 = i < n && j0 + l <= my_last, v1 = i < n && j0 + l + 16 <= my_last;
    s0 = v0 ? s0 : kNegBig;
    s1 = v1 ? s1 : kNegBig;
    float bm = fmaxf(s0, s1);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
    const float m_new = fmaxf(m, bm);
    const float alpha = expf(m - m_new);
    const float p0 = v0 ? expf(s0 - m_new) : 0.f, p1 = v1 ? expf(s1 - m_new) : 0.f;
    float ps = p0 + p1;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    lsum = lsum * alpha + ps;
    m = m_new;
    Ps[i * BKEY + l] = p0;
    Ps[i * BKEY + l + 16] = p1;
    __syncthreads();
    const float* pr = Ps + i * BKEY;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = l + 16 * kk;
      if (k < R) {
        float a = acc[kk] * alpha;
#pragma unroll 8
        for (int jj = 0; jj < BKEY; ++jj) a = fmaf(pr[jj], Cs[jj * RS + k], a);
        acc[kk] = a;
      }
    }
  }
  if (i < n) {
    const size_t row = row0 + i;
    float g = 1.0f / lsum;
    if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, row * p.ldg + h));
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = l + 16 * kk;
      if (k < R) st_any(p.out, p.out_dtype, row * ldq + static_cast<size_t>(h) * R + k, acc[kk] * g);
    }
  }
}

// One query row per CTA.  Per block of 32 keys: 8 threads share a key's dot product, warp 0 updates
// the running softmax, then thread (k = tid % RP, jg = tid / RP) adds the keys jj = jg (mod G) into
// column k.  The G partial accumulators of a column are summed in a fixed order at the end.
template <int KK>
__global__ void __launch_bounds__(kThreads) latent_attn_decode_kernel(const vila_latent_attn_params p, int RP) {
  extern __shared__ float sm[];
  const int R = p.R, RS = R + 1;
  float* Qs = sm;               // [R]
  float* Cs = Qs + R;           // [BKEY][R + 1]
  float* Ps = Cs + BKEY * RS;   // [BKEY] + alpha + (m, l)
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row0 = tile[0], pos0 = tile[2], slot = tile[3];
  const int32_t* pt = p.page_tables + static_cast<size_t>(slot) * p.pt_stride;
  const size_t ldq = static_cast<size_t>(p.H) * R;
  for (int k = tid; k < R; k += kThreads) Qs[k] = p.q[row0 * ldq + static_cast<size_t>(h) * R + k] * p.scale;
  // key groups per column; at most BKEY so that the final [G][R] exchange fits into Cs
  const int G = RP >= kThreads ? 1 : (kThreads / RP < BKEY ? kThreads / RP : BKEY);
  const int jg = RP >= kThreads ? 0 : tid / RP;
  const int kcol = RP >= kThreads ? tid : (jg < G ? tid % RP : R);  // R: this thread owns no column
  float acc[KK];
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) acc[kk] = 0.f;
  float m = p.sink ? p.sink[h] : kNegBig;   // meaningful in warp 0 only
  float lsum = p.sink ? 1.0f : 0.0f;
  const int nkeys = pos0 + 1;
  const int jj_s = tid >> 3, sub = tid & 7;
  for (int j0 = 0; j0 < nkeys; j0 += BKEY) {
    __syncthreads();
    for (int idx = tid; idx < BKEY * R; idx += kThreads) {
      const int jj = idx / R, k = idx % R, j = j0 + jj;
      Cs[jj * RS + k] = j < nkeys ? ld_any(p.cache, p.cache_dtype, cache_row(pt, p.page, j) * R + k) : 0.f;
    }
    __syncthreads();
    float s = 0.f;
    for (int k = sub; k < R; k += 8) s = fmaf(Qs[k], Cs[jj_s * RS + k], s);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (sub == 0) Ps[jj_s] = j0 + jj_s < nkeys ? s : kNegBig;
    __syncthreads();
    if (tid < 32) {
      const float sc = Ps[tid];
      const float m_new = fmaxf(m, warp_max(sc));
      const float alpha = expf(m - m_new);
      const float pv = sc > 0.5f * kNegBig ? expf(sc - m_new) : 0.f;
      lsum = lsum * alpha + warp_sum(pv);
      m = m_new;
      Ps[tid] = pv;
      if (tid == 0) Ps[BKEY] = alpha;
    }
    __syncthreads();
    const float alpha = Ps[BKEY];
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = kcol + kThreads * kk;
      if (k < R && (RP >= kThreads || kcol < R)) {
        float a = acc[kk] * alpha;
        for (int jj = jg; jj < BKEY; jj += G) a = fmaf(Ps[jj], Cs[jj * RS + k], a);
        acc[kk] = a;
      }
    }
  }
  __syncthreads();
  if (tid == 0) Ps[BKEY + 1] = lsum;
  // cross-group reduction through Cs (reused): [G][R]
  if (G > 1) {
    if (kcol < R) Cs[jg * R + kcol] = acc[0];
    __syncthreads();
    if (jg == 0 && kcol < R) {
      float a = 0.f;
      for (int g2 = 0; g2 < G; ++g2) a += Cs[g2 * R + kcol];
      acc[0] = a;
    }
  } else {
    __syncthreads();
  }
  if (jg == 0) {
    float g = 1.0f / Ps[BKEY + 1];
    if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, static_cast<size_t>(row0) * p.ldg + h));
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = kcol + kThreads * kk;
      if (k < R && (RP >= kThreads || kcol < R))
        st_any(p.out, p.out_dtype, row0 * ldq + static_cast<size_t>(h) * R + k, acc[kk] * g);
    }
  }
}

template <typename K>
int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024)
    VB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  return 0;
}

}  // namespace

int latent_attention(const vila_latent_attn_params& p, cudaStream_t stream) {
  if (p.ntiles <= 0) return 0;
  VB_CHECK(p.R >= 1 && p.R <= 512, "latent_attention: latent width %d not in [1, 512]", p.R);
  VB_CHECK(p.H >= 1 && p.H <= 65535 && p.page >= 1, "latent_attention: H=%d page=%d", p.H, p.page);
  const dim3 grid(p.ntiles, p.H), block(kThreads);
  if (p.decode) {
    int rp = 1;
    while (rp < p.R) rp <<= 1;
    const size_t smem = sizeof(float) * (p.R + BKEY * (p.R + 1) + BKEY + 2);
    if (p.R <= 256) {
      if (set_smem(latent_attn_decode_kernel<1>, smem)) return 2;
      VB_CUDA(launch_pdl(latent_attn_decode_kernel<1>, grid, block, smem, stream, p, rp));
    } else {
      if (set_smem(latent_attn_decode_kernel<2>, smem)) return 2;
      VB_CUDA(launch_pdl(latent_attn_decode_kernel<2>, grid, block, smem, stream, p, rp));
    }
    return 0;
  }
  const size_t smem = sizeof(float) * (BQ * p.R + BKEY * (p.R + 1) + BQ * BKEY);
#define VB_LAT_TILE(KK)                                                                    \
  do {                                                                                     \
    if (set_smem(latent_attn_tile_kernel<KK>, smem)) return 2;                             \
    VB_CUDA(launch_pdl(latent_attn_tile_kernel<KK>, grid, block, smem, stream, p));        \
  } while (0)
  if (p.R <= 32) VB_LAT_TILE(2);
  else if (p.R <= 64) VB_LAT_TILE(4);
  else if (p.R <= 128) VB_LAT_TILE(8);
  else if (p.R <= 256) VB_LAT_TILE(16);
  else VB_LAT_TILE(32);
#undef VB_LAT_TILE
  return 0;
}

}  // namespace vb
