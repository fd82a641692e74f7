// Causal short convolution over time on the channels of ragged rows, with the input added back, and the
// per-sequence state that lets a sequence be fed in portions: the last taps - 1 inputs of every
// sequence live in its state slot (fp32 [slots, taps - 1, cols], oldest first).
//   out[t, c] = h[t, c] + sum_j w[c, j] * h[t - (taps - 1) + j, c]
// A tap that reaches before the portion reads the state, one that reaches before position 0 reads zero
// (so a reused slot's stale contents are never seen).  All arithmetic is fp32, in tap order.
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTaps = 16;

__global__ void __launch_bounds__(kThreads)
short_conv_rows_kernel(const float* __restrict__ h, const void* __restrict__ w, int w_dt,
                       const float* __restrict__ state, const int32_t* __restrict__ seqs,
                       const int32_t* __restrict__ row_seq, void* __restrict__ out, int o_dt, int rows, int cols,
                       int taps) {
  const int t = blockIdx.x;
  const int* sq = seqs + 4 * row_seq[t];
  const int row0 = sq[0], pos0 = sq[2], slot = sq[3];
  const int back = taps - 1;
  const int pos = pos0 + (t - row0);
  const float* st = state + static_cast<size_t>(slot) * back * cols;
  for (int c = blockIdx.y * kThreads + threadIdx.x; c < cols; c += gridDim.y * kThreads) {
    const float cur = h[static_cast<size_t>(t) * cols + c];
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int d = back - j;          // this tap looks d positions back
      if (pos - d < 0) continue;
      float v;
      if (d == 0) v = cur;
      else if (t - d >= row0) v = h[static_cast<size_t>(t - d) * cols + c];
      else v = st[static_cast<size_t>(back - (row0 - (t - d))) * cols + c];   // position pos0 - k is state row back - k
      acc = fmaf(ld_any(w, w_dt, static_cast<size_t>(c) * taps + j), v, acc);
    }
    st_any(out, o_dt, static_cast<size_t>(t) * cols + c, cur + acc);
  }
}

// New state row j holds position end - back + j (end = first position after the portion): a row of the
// portion, an older state row (read at an index above the one being written: the loop runs upwards in
// j, one thread per channel, so nothing is overwritten before it is read), or zero before position 0.
__global__ void __launch_bounds__(kThreads)
short_conv_state_kernel(const float* __restrict__ h, float* __restrict__ state, const int32_t* __restrict__ seqs,
                        int cols, int taps) {
  const int* sq = seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int back = taps - 1;
  float* st = state + static_cast<size_t>(slot) * back * cols;
  for (int c = blockIdx.y * kThreads + threadIdx.x; c < cols; c += gridDim.y * kThreads) {
    for (int j = 0; j < back; ++j) {
      const int p = pos0 + n - back + j;
      float v = 0.f;
      if (p >= pos0) v = h[static_cast<size_t>(row0 + (p - pos0)) * cols + c];
      else if (p >= 0) v = st[static_cast<size_t>(j + n) * cols + c];
      st[static_cast<size_t>(j) * cols + c] = v;
    }
  }
}


// ---- group norm + short convolution for up to two sublayers in one pass ------------------------------
// One CTA per row t.  Phase 1: the inverse root mean square of every piece of the rows t - back .. t that
// lie inside the portion (a warp per (row, piece); the rows come from L2, they were just written).  Phase
// 2: per channel, the taps of both sublayers from the normalised rows (x * inv) * norm weight, or from the
// sequence's state for rows before the portion.  Same arithmetic as the separate kernels.
__device__ __forceinline__ float piece_inv(const float* __restrict__ xr, int gc, float eps) {
  float ss = 0.f;
  if ((gc & 3) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int c = threadIdx.x & 31; c < (gc >> 2); c += 32) {
      const float4 v = __ldg(x4 + c);
      s0 = fmaf(v.x, v.x, s0); s1 = fmaf(v.y, v.y, s1); s2 = fmaf(v.z, v.z, s2); s3 = fmaf(v.w, v.w, s3);
    }
    ss = (s0 + s1) + (s2 + s3);
  } else {
    for (int c = threadIdx.x & 31; c < gc; c += 32) ss = fmaf(xr[c], xr[c], ss);
  }
  ss = warp_sum(ss);
  return 1.0f / sqrtf(ss / static_cast<float>(gc) + eps);
}

__global__ void __launch_bounds__(kThreads) norm_conv_rows_kernel(const vila_norm_conv_params p) {
  extern __shared__ float inv_s[];   // [rows in reach][groups]
  const int t = blockIdx.x, cols = p.cols, groups = p.groups, gc = cols / groups, taps = p.taps, back = taps - 1;
  const int* sq = p.seqs + 4 * p.row_seq[t];
  const int row0 = sq[0], pos0 = sq[2], slot = sq[3];
  const int pos = pos0 + (t - row0);
  const int n_in = min(back, t - row0);          // predecessors inside the portion
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int pair = warp; pair < (n_in + 1) * groups; pair += kThreads / 32) {
    const int k = pair / groups, piece = pair - k * groups;
    const float r = piece_inv(p.x + static_cast<size_t>(t - k) * cols + static_cast<size_t>(piece) * gc, gc, p.eps);
    if (lane == 0) inv_s[pair] = r;
  }
  __syncthreads();
  const size_t soff = static_cast<size_t>(slot) * back * cols;
  for (int c = threadIdx.x; c < cols; c += kThreads) {
    const int piece = c / gc;
    float w[2], acc[2] = {0.f, 0.f}, cur[2] = {0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 2; ++k) w[k] = k < p.nsub ? p.norm_w[k][c] + p.w_offset : 0.f;
    for (int d = 0; d <= back; ++d) {            // this tap looks d positions back; weight column back - d
      if (pos - d < 0) break;
      const bool inside = d <= n_in;
      const float xn = inside ? p.x[static_cast<size_t>(t - d) * cols + c] * inv_s[d * groups + piece] : 0.f;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (k < p.nsub) {
          const float v = inside ? xn * w[k]
                                 : p.state[k][soff + static_cast<size_t>(back - (d - (t - row0))) * cols + c];
          if (d == 0) cur[k] = v;
          acc[k] = fmaf(ld_any(p.conv_w[k], p.conv_w_dtype, static_cast<size_t>(c) * taps + (back - d)), v, acc[k]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k)
      if (k < p.nsub) st_any(p.out[k], p.out_dtype, static_cast<size_t>(t) * cols + c, cur[k] + acc[k]);
  }
}

// The same pass for the common layout (fp32 convolution weights, channel count and piece width multiples of 4,
// 2 .. 4 taps): a thread owns 4 consecutive channels, the taps are unrolled, rows are read with 16-byte loads.
template <int TAPS, int NSUB>
__global__ void __launch_bounds__(kThreads) norm_conv_rows_vec_kernel(const vila_norm_conv_params p) {
  extern __shared__ float inv_s[];   // [rows in reach][groups]
  constexpr int back = TAPS - 1;
  const int t = blockIdx.x, cols = p.cols, groups = p.groups, gc = cols / groups;
  const int* sq = p.seqs + 4 * p.row_seq[t];
  const int row0 = sq[0], pos0 = sq[2], slot = sq[3];
  const int pos = pos0 + (t - row0);
  const int n_in = min(back, t - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int pair = warp; pair < (n_in + 1) * groups; pair += kThreads / 32) {
    const int k = pair / groups, piece = pair - k * groups;
    const float r = piece_inv(p.x + static_cast<size_t>(t - k) * cols + static_cast<size_t>(piece) * gc, gc, p.eps);
    if (lane == 0) inv_s[pair] = r;
  }
  __syncthreads();
  const float* xrow[TAPS];
  const float* srow[NSUB][TAPS];
  bool live[TAPS], inside[TAPS];
#pragma unroll
  for (int d = 0; d < TAPS; ++d) {
    live[d] = pos - d >= 0;
    inside[d] = d <= n_in;
    xrow[d] = p.x + static_cast<size_t>(inside[d] ? t - d : t) * cols;
#pragma unroll
    for (int k = 0; k < NSUB; ++k)
      srow[k][d] = (live[d] && !inside[d])
                       ? p.state[k] + (static_cast<size_t>(slot) * back + (back - (d - (t - row0)))) * cols
                       : nullptr;
  }
  for (int c = threadIdx.x << 2; c < cols; c += kThreads << 2) {
    const int piece = c / gc;
    float nw[NSUB][4], acc[NSUB][4], cur[NSUB][4];
#pragma unroll
    for (int k = 0; k < NSUB; ++k) {
      const float4 w4 = __ldg(reinterpret_cast<const float4*>(p.norm_w[k] + c));
      nw[k][0] = w4.x + p.w_offset; nw[k][1] = w4.y + p.w_offset; nw[k][2] = w4.z + p.w_offset; nw[k][3] = w4.w + p.w_offset;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[k][e] = cur[k][e] = 0.f;
    }
#pragma unroll
    for (int d = 0; d < TAPS; ++d) {
      if (!live[d]) continue;
      float xn[4] = {0.f, 0.f, 0.f, 0.f};
      if (inside[d]) {
        const float4 xv = *reinterpret_cast<const float4*>(xrow[d] + c);
        const float inv = inv_s[d * groups + piece];
        xn[0] = xv.x * inv; xn[1] = xv.y * inv; xn[2] = xv.z * inv; xn[3] = xv.w * inv;
      }
#pragma unroll
      for (int k = 0; k < NSUB; ++k) {
        float v[4];
        if (inside[d]) {
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = xn[e] * nw[k][e];
        } else {
          const float4 sv = *reinterpret_cast<const float4*>(srow[k][d] + c);
          v[0] = sv.x; v[1] = sv.y; v[2] = sv.z; v[3] = sv.w;
        }
        const float* cw = static_cast<const float*>(p.conv_w[k]) + static_cast<size_t>(c) * TAPS + (back - d);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (d == 0) cur[k][e] = v[e];
          acc[k][e] = fmaf(__ldg(cw + e * TAPS), v[e], acc[k][e]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < NSUB; ++k) {
      const size_t o = static_cast<size_t>(t) * cols + c;
      const float r0 = cur[k][0] + acc[k][0], r1 = cur[k][1] + acc[k][1], r2 = cur[k][2] + acc[k][2], r3 = cur[k][3] + acc[k][3];
      if (p.out_dtype == VILA_DT_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(p.out[k]) + o) = make_float4(r0, r1, r2, r3);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
        uint2 u;
        u.x = *reinterpret_cast<unsigned int*>(&lo);
        u.y = *reinterpret_cast<unsigned int*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out[k]) + o) = u;
      }
    }
  }
}

// ---- the streaming form: statistics first, then CTAs that own a channel slice of a block of rows -------
// group_inv_kernel: inv[row, piece] (a warp per pair).  norm_conv_slice_kernel: grid (row blocks, channel
// slices of 4 * 256 channels); a thread keeps the convolution and norm weights of its 4 channels in
// registers for all rows of the block, so the weights are read once per CTA instead of once per row, and
// the predecessor rows a tap needs were read by the same thread one row earlier (L1).
__global__ void __launch_bounds__(kThreads) group_inv_kernel(const vila_norm_conv_params p) {
  const int gc = p.cols / p.groups;
  const int pair = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (pair >= p.rows * p.groups) return;
  const int row = pair / p.groups, piece = pair - row * p.groups;
  const float r = piece_inv(p.x + static_cast<size_t>(row) * p.cols + static_cast<size_t>(piece) * gc, gc, p.eps);
  if ((threadIdx.x & 31) == 0) p.inv[pair] = r;
}

template <int TAPS, int NSUB>
__global__ void __launch_bounds__(kThreads) norm_conv_slice_kernel(const vila_norm_conv_params p, int RB) {
  constexpr int back = TAPS - 1;
  const int cols = p.cols, groups = p.groups, gc = cols / groups;
  const int c = (blockIdx.y * kThreads + threadIdx.x) << 2;
  if (c >= cols) return;
  const int piece = c / gc;
  const int t0 = blockIdx.x * RB, t1 = min(p.rows, t0 + RB);
  float nw[NSUB][4], cw[NSUB][4][TAPS];
#pragma unroll
  for (int k = 0; k < NSUB; ++k) {
    const float4 w4 = __ldg(reinterpret_cast<const float4*>(p.norm_w[k] + c));
    nw[k][0] = w4.x + p.w_offset; nw[k][1] = w4.y + p.w_offset; nw[k][2] = w4.z + p.w_offset; nw[k][3] = w4.w + p.w_offset;
    const float* w = static_cast<const float*>(p.conv_w[k]) + static_cast<size_t>(c) * TAPS;
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
      for (int j = 0; j < TAPS; ++j) cw[k][e][j] = __ldg(w + e * TAPS + j);
  }
  for (int t = t0; t < t1; ++t) {
    const int* sq = p.seqs + 4 * p.row_seq[t];
    const int row0 = sq[0], pos0 = sq[2], slot = sq[3];
    const int pos = pos0 + (t - row0);
    const int n_in = min(back, t - row0);
    float acc[NSUB][4], cur[NSUB][4];
#pragma unroll
    for (int k = 0; k < NSUB; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[k][e] = cur[k][e] = 0.f;
#pragma unroll
    for (int d = 0; d < TAPS; ++d) {
      if (pos - d < 0) continue;
      const bool inside = d <= n_in;
      float xn[4] = {0.f, 0.f, 0.f, 0.f};
      if (inside) {
        const float4 xv = *reinterpret_cast<const float4*>(p.x + static_cast<size_t>(t - d) * cols + c);
        const float inv = p.inv[(t - d) * groups + piece];
        xn[0] = xv.x * inv; xn[1] = xv.y * inv; xn[2] = xv.z * inv; xn[3] = xv.w * inv;
      }
#pragma unroll
      for (int k = 0; k < NSUB; ++k) {
        float v[4];
        if (inside) {
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = xn[e] * nw[k][e];
        } else {
          const float4 sv = *reinterpret_cast<const float4*>(
              p.state[k] + (static_cast<size_t>(slot) * back + (back - (d - (t - row0)))) * cols + c);
          v[0] = sv.x; v[1] = sv.y; v[2] = sv.z; v[3] = sv.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (d == 0) cur[k][e] = v[e];
          acc[k][e] = fmaf(cw[k][e][back - d], v[e], acc[k][e]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < NSUB; ++k) {
      const size_t o = static_cast<size_t>(t) * cols + c;
      const float r0 = cur[k][0] + acc[k][0], r1 = cur[k][1] + acc[k][1], r2 = cur[k][2] + acc[k][2], r3 = cur[k][3] + acc[k][3];
      if (p.out_dtype == VILA_DT_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(p.out[k]) + o) = make_float4(r0, r1, r2, r3);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
        uint2 u;
        u.x = *reinterpret_cast<unsigned int*>(&lo);
        u.y = *reinterpret_cast<unsigned int*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out[k]) + o) = u;
      }
    }
  }
}

// One CTA per sequence: its last taps - 1 normalised inputs, for both sublayers.
__global__ void __launch_bounds__(kThreads) norm_conv_state_kernel(const vila_norm_conv_params p) {
  extern __shared__ float inv_s[];   // [rows kept][groups]
  const int cols = p.cols, groups = p.groups, gc = cols / groups, back = p.taps - 1;
  const int* sq = p.seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int keep = min(back, n);                 // rows of the portion that enter the state: the last `keep`
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int pair = warp; pair < keep * groups; pair += kThreads / 32) {
    const int k = pair / groups, piece = pair - k * groups;     // k-th of the kept rows: row0 + n - keep + k
    const int row = row0 + n - keep + k;
    const float r = p.inv ? p.inv[row * groups + piece]
                          : piece_inv(p.x + static_cast<size_t>(row) * cols + static_cast<size_t>(piece) * gc, gc, p.eps);
    if (lane == 0) inv_s[pair] = r;
  }
  __syncthreads();
  const size_t soff = static_cast<size_t>(slot) * back * cols;
  for (int c = blockIdx.y * kThreads + threadIdx.x; c < cols; c += gridDim.y * kThreads) {
    const int piece = c / gc;
    for (int j = 0; j < back; ++j) {
      const int q = pos0 + n - back + j;          // position held by new state row j
      const bool fresh = q >= pos0;
      const int k = j - (back - keep);            // index among the kept rows
      const float xn = fresh ? p.x[static_cast<size_t>(row0 + n - keep + k) * cols + c] * inv_s[k * groups + piece] : 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u < p.nsub) {
          float v = 0.f;
          if (fresh) v = xn * (p.norm_w[u][c] + p.w_offset);
          else if (q >= 0) v = p.state[u][soff + static_cast<size_t>(j + n) * cols + c];
          p.state[u][soff + static_cast<size_t>(j) * cols + c] = v;
        }
      }
    }
  }
}

}  // namespace

int short_conv_rows(const float* h, const void* w, int w_dt, const float* state, const int32_t* seqs,
                    const int32_t* row_seq, void* out, int o_dt, int rows, int cols, int taps,
                    cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  VB_CHECK(taps >= 1 && taps <= kMaxTaps && (taps == 1 || state != nullptr), "short_conv_rows: taps=%d", taps);
  const dim3 grid(rows, (cols + 4 * kThreads - 1) / (4 * kThreads));
  VB_CUDA(launch_serial(short_conv_rows_kernel, grid, dim3(kThreads), 0, stream, h, w, w_dt, state, seqs,
                        row_seq, out, o_dt, rows, cols, taps));
  return 0;
}

int short_conv_state(const float* h, float* state, const int32_t* seqs, int nseq, int cols, int taps,
                     cudaStream_t stream) {
  if (nseq <= 0 || cols <= 0 || taps <= 1) return 0;
  VB_CHECK(taps <= kMaxTaps, "short_conv_state: taps=%d", taps);
  const dim3 grid(nseq, (cols + 4 * kThreads - 1) / (4 * kThreads));
  VB_CUDA(launch_serial(short_conv_state_kernel, grid, dim3(kThreads), 0, stream, h, state, seqs, cols, taps));
  return 0;
}

int norm_conv_rows(const vila_norm_conv_params& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.cols <= 0) return 0;
  VB_CHECK(p.taps >= 1 && p.taps <= kMaxTaps && p.groups >= 1 && p.cols % p.groups == 0 && (p.nsub == 1 || p.nsub == 2),
           "norm_conv_rows: taps=%d groups=%d cols=%d nsub=%d", p.taps, p.groups, p.cols, p.nsub);
  for (int k = 0; k < p.nsub; ++k)
    VB_CHECK(p.norm_w[k] && p.conv_w[k] && p.out[k] && (p.taps == 1 || p.state[k]), "norm_conv_rows: sublayer %d lacks a tensor", k);
  const size_t smem = sizeof(float) * p.taps * p.groups;
  VB_CHECK(smem <= 48 * 1024, "norm_conv_rows: groups=%d", p.groups);
  bool aligned = p.conv_w_dtype == VILA_DT_F32 && p.cols % 4 == 0 && (p.cols / p.groups) % 4 == 0 && p.taps >= 2 &&
                 p.taps <= 4 && reinterpret_cast<uintptr_t>(p.x) % 16 == 0;
  for (int k = 0; k < p.nsub; ++k)
    aligned = aligned && reinterpret_cast<uintptr_t>(p.norm_w[k]) % 16 == 0 && reinterpret_cast<uintptr_t>(p.out[k]) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(p.state[k]) % 16 == 0;
  if (aligned && p.inv != nullptr && p.rows >= 256) {
    // many rows: statistics, then channel-slice CTAs that stream a block of rows with the weights in registers
    const int slices = (p.cols + 4 * kThreads - 1) / (4 * kThreads);
    int rb = p.rows * slices / (2 * 148);          // about two CTAs per SM
    rb = rb < 4 ? 4 : (rb > 32 ? 32 : rb);
    const dim3 sgrid((p.rows + rb - 1) / rb, slices);
    VB_CUDA(launch_serial(group_inv_kernel, dim3((p.rows * p.groups + 7) / 8), dim3(kThreads), 0, stream, p));
#define VB_NS(T, N) VB_CUDA(launch_serial(norm_conv_slice_kernel<T, N>, sgrid, dim3(kThreads), 0, stream, p, rb))
    if (p.nsub == 2) {
      if (p.taps == 2) VB_NS(2, 2);
      else if (p.taps == 3) VB_NS(3, 2);
      else VB_NS(4, 2);
    } else {
      if (p.taps == 2) VB_NS(2, 1);
      else if (p.taps == 3) VB_NS(3, 1);
      else VB_NS(4, 1);
    }
#undef VB_NS
    if (p.taps > 1 && p.nseq > 0)
      VB_CUDA(launch_serial(norm_conv_state_kernel, dim3(p.nseq, (p.cols + kThreads - 1) / kThreads), dim3(kThreads), smem, stream, p));
    return 0;
  }
#define VB_NC(T, N) VB_CUDA(launch_serial(norm_conv_rows_vec_kernel<T, N>, dim3(p.rows), dim3(kThreads), smem, stream, p))
  if (aligned && p.nsub == 2) {
    if (p.taps == 2) VB_NC(2, 2);
    else if (p.taps == 3) VB_NC(3, 2);
    else VB_NC(4, 2);
  } else if (aligned) {
    if (p.taps == 2) VB_NC(2, 1);
    else if (p.taps == 3) VB_NC(3, 1);
    else VB_NC(4, 1);
  } else {
    VB_CUDA(launch_serial(norm_conv_rows_kernel, dim3(p.rows), dim3(kThreads), smem, stream, p));
  }
#undef VB_NC
  if (p.taps > 1 && p.nseq > 0) {
    vila_norm_conv_params q = p;
    q.inv = nullptr;   // no statistics pass ran on this path: the state kernel computes its own
    VB_CUDA(launch_serial(norm_conv_state_kernel, dim3(p.nseq, (p.cols + kThreads - 1) / kThreads), dim3(kThreads), smem, stream, q));
  }
  return 0;
}

}  // namespace vb
