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
// Mapping: HBM-bound, no tensor cores.  One warp owns kRows consecutive output rows; a lane
// owns 16-byte units of the row's code stream (unit u of every row sits at byte 16u, so a
// warp load is 512 contiguous bytes), issues kUnroll independent 128-bit streaming loads per
// row before touching them, unpacks in registers and feeds dp4a.
#include "common.cuh"

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

__device__ __forceinline__ int dot16(const uint4 &a, const int4 &b) {
  int s = __dp4a((int)a.x, b.x, 0);
  s = __dp4a((int)a.y, b.y, s);
  s = __dp4a((int)a.z, b.z, s);
  return __dp4a((int)a.w, b.w, s);
}

template <int B>
__device__ __forceinline__ void rows_q8_0(const uint8_t *const (&row)[kRows], int64_t cols, const uint8_t *act,
                                          int64_t act_stride, int lane, float (&acc)[kRows][B]) {
  const int units = (int)(cols >> 4);
  const int64_t sc_off = act_scale_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * kUnroll) {
    uint4 wv[kRows][kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
#pragma unroll
      for (int r = 0; r < kRows; ++r) wv[r][i] = u < units ? ld_stream16(row[r] + (int64_t)u * 16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      const int blk = u >> 1;
      float ws[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) ws[r] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(row[r] + cols) + blk));
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xv = __ldg(reinterpret_cast<const int4 *>(a) + u);
        const float xs = __ldg(reinterpret_cast<const float *>(a + sc_off) + blk);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int isum = dot16(wv[r][i], xv);
          acc[r][b] = __fadd_rn(acc[r][b], __fmul_rn(__fmul_rn((float)isum, ws[r]), xs));
        }
      }
    }
  }
}

template <int B>
__device__ __forceinline__ void rows_q4_k(const uint8_t *const (&row)[kRows], int64_t cols, const uint8_t *act,
                                          int64_t act_stride, int lane, float (&acc)[kRows][B]) {
  const int nsb = (int)(cols >> 8);
  const int units = nsb * 8;
  const int64_t sc_off = act_scale_off(cols), bs_off = act_bsum_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * kUnroll) {
    uint4 wv[kRows][kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
#pragma unroll
      for (int r = 0; r < kRows; ++r) wv[r][i] = u < units ? ld_stream16(row[r] + (int64_t)u * 16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      const int sb = u >> 3, t = u & 7, j = t >> 1, h = t & 1;
      // This lane's 16 bytes hold values 64j+16h.. (low nibbles) and 64j+32+16h.. (high nibbles)
      // of superblock sb; for the mins term the lane owns 32-value group t.
      float dw[kRows], dmw[kRows];
      int scl[kRows], sch[kRows], mt[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint4 meta = __ldg(reinterpret_cast<const uint4 *>(row[r] + (int64_t)nsb * 128) + sb);
        dw[r] = f16_bits_to_f32((uint16_t)(meta.x & 0xffff));
        dmw[r] = f16_bits_to_f32((uint16_t)(meta.x >> 16));
        int m_unused;
        q4k_scale_min(2 * j, meta.y, meta.z, meta.w, scl[r], m_unused);
        q4k_scale_min(2 * j + 1, meta.y, meta.z, meta.w, sch[r], m_unused);
        int sc_unused;
        q4k_scale_min(t, meta.y, meta.z, meta.w, sc_unused, mt[r]);
      }
      uint4 lo[kRows], hi[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint4 w = wv[r][i];
        lo[r] = make_uint4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu);
        hi[r] = make_uint4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, (w.z >> 4) & 0x0f0f0f0fu,
                           (w.w >> 4) & 0x0f0f0f0fu);
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xlo = __ldg(reinterpret_cast<const int4 *>(a + sb * 256 + 64 * j + 16 * h));
        const int4 xhi = __ldg(reinterpret_cast<const int4 *>(a + sb * 256 + 64 * j + 32 + 16 * h));
        const float xd = __ldg(reinterpret_cast<const float *>(a + sc_off) + sb);
        const int bs2 = __ldg(reinterpret_cast<const int *>(a + bs_off) + sb * 8 + t);  // two i16 sums of group t
        const int bsum = (int)(short)(bs2 & 0xffff) + (bs2 >> 16);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int s = dot16(lo[r], xlo) * scl[r] + dot16(hi[r], xhi) * sch[r];
          const int p = bsum * mt[r];
          const float d = __fmul_rn(xd, dw[r]), dmin = __fmul_rn(xd, dmw[r]);
          acc[r][b] = __fmaf_rn(d, (float)s, __fmaf_rn(-dmin, (float)p, acc[r][b]));
        }
      }
    }
  }
}

template <int B>
__device__ __forceinline__ void rows_q6_k(const uint8_t *const (&row)[kRows], int64_t cols, const uint8_t *act,
                                          int64_t act_stride, int lane, float (&acc)[kRows][B]) {
  const int nsb = (int)(cols >> 8);
  const int units = nsb * 8;
  const int64_t sc_off = act_scale_off(cols), bs_off = act_bsum_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * kUnroll) {
    uint4 wl[kRows][kUnroll], wh[kRows][kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
      const int sb = u >> 3, t = u & 7;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (u < units) {
          wl[r][i] = ld_stream16(row[r] + (int64_t)u * 16);
          // qh bytes for l = 16c.. of half h: shared by the two lanes s' = 0,1
          wh[r][i] = __ldg(reinterpret_cast<const uint4 *>(row[r] + (int64_t)nsb * 128 + sb * 64 + 32 * (t >> 2) + 16 * (t & 1)));
        } else {
          wl[r][i] = wh[r][i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      // unit t of superblock sb: half h, ql sub-run s' (streams s' and s'+2), l = 16c..16c+15
      const int sb = u >> 3, t = u & 7, h = t >> 2, sp = (t >> 1) & 1, c = t & 1;
      const int jlo = 8 * h + 2 * sp + c;  // 16-value group of the low-nibble stream; high stream is jlo + 4
      float dw[kRows];
      int slo[kRows], shi[kRows];
      uint4 qlo[kRows], qhi[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        dw[r] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(row[r] + (int64_t)nsb * 208) + sb));
        const int8_t *sc = reinterpret_cast<const int8_t *>(row[r] + (int64_t)nsb * 192 + sb * 16);
        slo[r] = __ldg(sc + jlo);
        shi[r] = __ldg(sc + jlo + 4);
        const uint4 l4 = wl[r][i], h4 = wh[r][i];
        const int sh_lo = 2 * sp, sh_hi = 2 * sp + 4;
        qlo[r] = make_uint4((l4.x & 0x0f0f0f0fu) | (((h4.x >> sh_lo) & 0x03030303u) << 4),
                            (l4.y & 0x0f0f0f0fu) | (((h4.y >> sh_lo) & 0x03030303u) << 4),
                            (l4.z & 0x0f0f0f0fu) | (((h4.z >> sh_lo) & 0x03030303u) << 4),
                            (l4.w & 0x0f0f0f0fu) | (((h4.w >> sh_lo) & 0x03030303u) << 4));
        qhi[r] = make_uint4(((l4.x >> 4) & 0x0f0f0f0fu) | (((h4.x >> sh_hi) & 0x03030303u) << 4),
                            ((l4.y >> 4) & 0x0f0f0f0fu) | (((h4.y >> sh_hi) & 0x03030303u) << 4),
                            ((l4.z >> 4) & 0x0f0f0f0fu) | (((h4.z >> sh_hi) & 0x03030303u) << 4),
                            ((l4.w >> 4) & 0x0f0f0f0fu) | (((h4.w >> sh_hi) & 0x03030303u) << 4));
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xlo = __ldg(reinterpret_cast<const int4 *>(a + sb * 256 + jlo * 16));
        const int4 xhi = __ldg(reinterpret_cast<const int4 *>(a + sb * 256 + (jlo + 4) * 16));
        const float xd = __ldg(reinterpret_cast<const float *>(a + sc_off) + sb);
        const short *bs = reinterpret_cast<const short *>(a + bs_off) + sb * 16;
        const int blo = __ldg(bs + jlo), bhi = __ldg(bs + jlo + 4);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          // codes are stored +32: sum (q-32)*x = dot(q,x) - 32*sum(x)
          const int s = slo[r] * (dot16(qlo[r], xlo) - 32 * blo) + shi[r] * (dot16(qhi[r], xhi) - 32 * bhi);
          acc[r][b] = __fadd_rn(acc[r][b], __fmul_rn(__fmul_rn(dw[r], xd), (float)s));
        }
      }
    }
  }
}

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
  if (J.qt == CMLD_Q4_K) rows_q4_k<B>(row, J.cols, act, astride, lane, acc);
  else if (J.qt == CMLD_Q6_K) rows_q6_k<B>(row, J.cols, act, astride, lane, acc);
  else rows_q8_0<B>(row, J.cols, act, astride, lane, acc);
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
