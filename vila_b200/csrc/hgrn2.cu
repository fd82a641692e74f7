// HGRN2-style gated linear recurrence (linear attention whose forget gate also sets the input gate):
//   S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,   o_t = S_t^T q_t,   S: [dim, vdim] per head, fp32.
// The state of a sequence lives in a slot of a caller-owned pool between steps; a step advances it by
// the rows the step brings (a prompt portion of any length, or one decoded token).
// Grid (sequence, head, 32-column slice of vdim); thread (c = tid / 8, r = tid % 8) keeps the rows
// r, r + 8, ... of column c in registers, the 8 row groups of a column sit in adjacent lanes and the
// dot product with q_t is finished with three shuffles.  Gates are evaluated in fp32 while a chunk of
// 16 tokens is staged in shared memory: q = silu(zq), f = lower + (1 - lower) sigmoid(zf + bias).
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256, kCols = 32, kRowGroups = 8, kChunk = 16;

template <int KPT>  // rows per thread: dim <= 8 * KPT
__global__ void __launch_bounds__(kThreads) hgrn2_scan_kernel(const vila_hgrn2_params p) {
  extern __shared__ float sm[];
  const int dim = p.dim, vdim = p.vdim;
  float* q_s = sm;                    // [kChunk][dim]
  float* f_s = q_s + kChunk * dim;    // [kChunk][dim]
  float* v_s = f_s + kChunk * dim;    // [kChunk][kCols]
  const int tid = threadIdx.x, r = tid & 7, c = tid >> 3;
  const int* sq = p.seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int h = blockIdx.y;
  const int col = blockIdx.z * kCols + c;
  const bool col_ok = col < vdim;
  float* st = p.state + (static_cast<size_t>(slot) * p.H + h) * dim * vdim;
  float S[KPT];
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    const int i = r + kRowGroups * k;
    S[k] = (pos0 > 0 && col_ok && i < dim) ? st[static_cast<size_t>(i) * vdim + col] : 0.f;
  }
  for (int t0 = 0; t0 < n; t0 += kChunk) {
    const int nt = min(kChunk, n - t0);
    __syncthreads();
    for (int idx = tid; idx < nt * dim; idx += kThreads) {
      const int t = idx / dim, i = idx % dim;
      const size_t base = static_cast<size_t>(row0 + t0 + t) * p.ldp;
      const int ch = h * dim + i;
      const float zq = ld_any(p.proj, p.proj_dtype, base + p.q_off + ch);
      const float zf = ld_any(p.proj, p.proj_dtype, base + p.f_off + ch) + (p.f_bias ? p.f_bias[ch] : 0.f);
      const float lo = p.lower ? p.lower[ch] : 0.f;
      q_s[t * dim + i] = silu_exact_f(zq);
      f_s[t * dim + i] = lo + (1.0f - lo) * sigmoid_f(zf);
    }
    for (int idx = tid; idx < nt * kCols; idx += kThreads) {
      const int t = idx / kCols, cc = idx % kCols, gc = blockIdx.z * kCols + cc;
      v_s[idx] = gc < vdim ? ld_any(p.proj, p.proj_dtype, static_cast<size_t>(row0 + t0 + t) * p.ldp + p.v_off +
                                                              h * vdim + gc)
                           : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = v_s[t * kCols + c];
      const float* ft = f_s + t * dim;
      const float* qt = q_s + t * dim;
      float part = 0.f;
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        const int i = r + kRowGroups * k;
        if (i < dim) {
          const float f = ft[i];
          S[k] = fmaf(f, S[k], (1.0f - f) * v);
          part = fmaf(S[k], qt[i], part);
        }
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      if (r == 0 && col_ok)
        p.out[static_cast<size_t>(row0 + t0 + t) * p.H * vdim + h * vdim + col] = part;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int k = 0; k < KPT; ++k) {
      const int i = r + kRowGroups * k;
      if (i < dim) st[static_cast<size_t>(i) * vdim + col] = S[k];
    }
  }
}

}  // namespace

int hgrn2_scan(const vila_hgrn2_params& p, cudaStream_t stream) {
  if (p.nseq <= 0) return 0;
  VB_CHECK(p.dim >= 1 && p.dim <= 256 && p.vdim >= 1 && p.H >= 1, "hgrn2_scan: H=%d dim=%d (<= 256) vdim=%d",
           p.H, p.dim, p.vdim);
  const dim3 grid(p.nseq, p.H, (p.vdim + kCols - 1) / kCols), block(kThreads);
  VB_CHECK(grid.y <= 65535 && grid.z <= 65535, "hgrn2_scan: grid too large");
  const size_t smem = sizeof(float) * (2 * kChunk * p.dim + kChunk * kCols);
#define VB_HGRN(KPT) VB_CUDA(launch_serial(hgrn2_scan_kernel<KPT>, grid, block, smem, stream, p))
  if (p.dim <= 16) VB_HGRN(2);
  else if (p.dim <= 32) VB_HGRN(4);
  else if (p.dim <= 64) VB_HGRN(8);
  else if (p.dim <= 128) VB_HGRN(16);
  else VB_HGRN(32);
#undef VB_HGRN
  return 0;
}

}  // namespace vb
