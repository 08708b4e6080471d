// Fused dequantise-and-matvec over Q8_0 / Q4_K / Q6_K rows against int8-quantised
// activations (batch 1..8 columns per pass).
//
// Arithmetic follows Camelid's CPU dots — integer block dots, then f32 scaling:
//   Q8_0: q8_0_dot_rows            (src/inference.rs:26166-26200)
//   Q4_K: q4_k_dot_scalar          (src/diffusion_gemma/refmath.rs:504-562)
//   Q6_K: q6_k_wire_row_dot        (src/inference.rs:25535-25581)
// The integer parts are exact; the f32 partial sums are accumulated per lane and combined by
// a warp shuffle tree, so a result can differ from the CPU's block-ordered sum in the last
// bits (never in the integer parts).
//
// This file holds the direct-load kernel: one warp owns kRows consecutive output rows, a lane
// owns 16-byte units of the row's code stream, issues kUnroll independent 128-bit streaming
// loads per row before touching them, unpacks in registers and feeds dp4a.  It accepts every
// shape; the staged kernel in gemv_pipe.cu is the fast path for the shapes it supports.
#include "gemv_rows.cuh"

namespace cmld {

constexpr int kRows = 2;    // rows per warp
constexpr int kUnroll = 4;  // 16-byte units in flight per lane and row
constexpr int kWarpsPerBlock = 4;
constexpr int kRowsPerBlock = kRows * kWarpsPerBlock;
constexpr int kMaxJobs = 4;

struct GemvJobs {
  GemvJob job[kMaxJobs];
  int32_t first_block[kMaxJobs + 1];
  int32_t n;
};

template <int B>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) gemv_kernel(const GemvJobs jobs, const uint8_t *__restrict__ act) {
  int ji = 0;
#pragma unroll
  for (int k = 1; k < kMaxJobs; ++k)
    if (k < jobs.n && (int)blockIdx.x >= jobs.first_block[k]) ji = k;
  const GemvJob &J = jobs.job[ji];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t r0 = ((int64_t)(blockIdx.x - jobs.first_block[ji]) * kWarpsPerBlock + warp) * kRows;
  if (r0 >= J.rows) return;
  const uint8_t *row[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) row[r] = J.w + (r0 + r < J.rows ? r0 + r : r0) * J.stride;
  float acc[kRows][B];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) acc[r][b] = 0.0f;
  const int64_t astride = act_row_stride(J.cols);
  if (J.qt == CMLD_Q4_K) rows_q4_k<B, kRows, kUnroll, false>(row, J.cols, act, astride, lane, acc);
  else if (J.qt == CMLD_Q6_K) rows_q6_k<B, kRows, kUnroll, false>(row, J.cols, act, astride, lane, acc);
  else rows_q8_0<B, kRows, kUnroll, false>(row, J.cols, act, astride, lane, acc);
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float v = warp_sum(acc[r][b]);
      if (lane == 0 && r0 + r < J.rows) {
        const int64_t o = (int64_t)b * J.y_stride + r0 + r;
        J.y[o] = J.residual ? __fadd_rn(J.residual[o], v) : v;
      }
    }
}

template <int B>
static int32_t launch_b(const GemvJobs &jobs, int blocks, const uint8_t *act, cudaStream_t s) {
  gemv_kernel<B><<<blocks, kWarpsPerBlock * 32, 0, s>>>(jobs, act);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// All jobs of one launch share `cols` and read the same activation buffer (Q8_0 jobs its
// Q8_0 codes, K-quant jobs its Q8_K codes; the caller passes the matching buffer, which for
// a mixed group means separate launches).  batch > 8 runs in passes of up to 8 columns.
int32_t launch_gemv(const GemvJob *jobs_in, int n_jobs, const uint8_t *act, int32_t batch, cudaStream_t s) {
  if (n_jobs < 1 || n_jobs > kMaxJobs) return fail(CMLD_ERR_INVALID, "gemv: %d jobs in one launch", n_jobs);
  for (int b0 = 0; b0 < batch; b0 += 8) {
    const int nb = batch - b0 < 8 ? batch - b0 : 8;
    GemvJobs jobs;
    jobs.n = n_jobs;
    int blocks = 0;
    for (int k = 0; k < n_jobs; ++k) {
      jobs.job[k] = jobs_in[k];
      jobs.job[k].y += (int64_t)b0 * jobs_in[k].y_stride;
      if (jobs.job[k].residual) jobs.job[k].residual += (int64_t)b0 * jobs_in[k].y_stride;
      jobs.first_block[k] = blocks;
      blocks += (int)((jobs_in[k].rows + kRowsPerBlock - 1) / kRowsPerBlock);
      if (jobs_in[k].cols != jobs_in[0].cols) return fail(CMLD_ERR_SHAPE, "gemv: jobs of one launch must share cols");
    }
    jobs.first_block[n_jobs] = blocks;
    if (blocks == 0) continue;
    const uint8_t *a = act + (int64_t)b0 * act_row_stride(jobs_in[0].cols);
    switch (nb) {
      case 1: CMLD_TRY(launch_b<1>(jobs, blocks, a, s)); break;
      case 2: CMLD_TRY(launch_b<2>(jobs, blocks, a, s)); break;
      case 3: CMLD_TRY(launch_b<3>(jobs, blocks, a, s)); break;
      case 4: CMLD_TRY(launch_b<4>(jobs, blocks, a, s)); break;
      case 5: CMLD_TRY(launch_b<5>(jobs, blocks, a, s)); break;
      case 6: CMLD_TRY(launch_b<6>(jobs, blocks, a, s)); break;
      case 7: CMLD_TRY(launch_b<7>(jobs, blocks, a, s)); break;
      default: CMLD_TRY(launch_b<8>(jobs, blocks, a, s)); break;
    }
  }
  return CMLD_OK;
}

}  // namespace cmld
