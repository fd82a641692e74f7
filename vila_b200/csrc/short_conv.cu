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

}  // namespace vb
