// Reference-order kernels (engine flag CMLD_FLAG_EXACT_ORDER).
//
// The fast kernels combine f32 partial sums with shuffle trees.  Camelid's CPU path adds them one
// after another — blocks of a row in order, attention positions in order — and because every
// matvec operand is then quantised to int8, a 1e-6 difference can land on the other side of a
// rounding boundary.  These kernels keep the CPU's order of every f32 operation, so that with the
// bit-exact quantisers, the host-computed RoPE table and the restated expf, a decode step returns
// the CPU path's bits.  They are slower (one lane walks each row's terms) and exist for parity
// work, not for the benchmark.
//
//   matvec:    q8_0_dot_rows (src/inference.rs:26191-26199), q4_k_dot_scalar
//              (src/diffusion_gemma/refmath.rs:504-562), q6_k_wire_row_dot (src/inference.rs:25535-25581)
//   attention: attention_context_for_head_into_with_kernels (src/inference.rs:30287-30466) with
//              dot_product (src/tensor/mod.rs:3464-3480)
#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

constexpr int kExactWarps = 4;

// One warp per output row.  Lanes compute the exact per-block pieces in parallel into shared memory;
// then the row's terms are added in block order.
template <int QT>
__global__ void __launch_bounds__(kExactWarps * 32) gemv_exact_kernel(GemvJob J, const uint8_t *__restrict__ act, int batch,
                                                                      int smem_per_warp) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t r = (int64_t)blockIdx.x * kExactWarps + warp;
  if (r >= J.rows) return;
  const uint8_t *row = J.w + r * J.stride;
  float *sf = reinterpret_cast<float *>(smem + (size_t)warp * smem_per_warp);
  int *si = reinterpret_cast<int *>(sf);
  const int64_t cols = J.cols, astride = act_row_stride(cols);
  for (int b = 0; b < batch; ++b) {
    const uint8_t *a = act + b * astride;
    const int8_t *xq = reinterpret_cast<const int8_t *>(a);
    const float *xs = reinterpret_cast<const float *>(a + act_scale_off(cols));
    float result = 0.0f;
    if (QT == CMLD_Q8_0) {
      const int nb = (int)(cols >> 5);
      for (int blk = lane; blk < nb; blk += 32) {
        const int8_t *wq = reinterpret_cast<const int8_t *>(row) + blk * 32;
        int isum = 0;
        for (int j = 0; j < 32; ++j) isum += (int)wq[j] * (int)xq[blk * 32 + j];
        const float ws = f16_bits_to_f32(reinterpret_cast<const uint16_t *>(row + cols)[blk]);
        sf[blk] = __fmul_rn(__fmul_rn((float)isum, ws), xs[blk]);
      }
      __syncwarp();
      if (lane == 0) {
        float s = 0.0f;
        for (int blk = 0; blk < nb; ++blk) s = __fadd_rn(s, sf[blk]);
        result = s;
      }
    } else if (QT == CMLD_Q4_K) {
      const int nsb = (int)(cols >> 8);
      for (int sb = lane; sb < nsb; sb += 32) {
        const uint8_t *blk = row + sb * 144;
        const uint32_t *meta = reinterpret_cast<const uint32_t *>(blk);
        const float dw = f16_bits_to_f32((uint16_t)(meta[0] & 0xffff)), dmw = f16_bits_to_f32((uint16_t)(meta[0] >> 16));
        const int8_t *y = xq + sb * 256;
        long long prod = 0, s12 = 0;
        for (int g = 0; g < 8; ++g) {
          int sc, m;
          q4k_scale_min(g, meta[1], meta[2], meta[3], sc, m);
          int bs = 0, dot = 0;
          const uint8_t *qs = blk + 16 + 32 * (g >> 1);
          for (int t = 0; t < 32; ++t) {
            const int yv = y[32 * g + t];
            bs += yv;
            const int nib = (g & 1) ? (qs[t] >> 4) : (qs[t] & 15);
            dot += nib * yv;
          }
          prod += (long long)bs * m;
          s12 += (long long)dot * sc;
        }
        const float xd = xs[sb];
        sf[4 * sb + 0] = __fmul_rn(xd, dw);
        sf[4 * sb + 1] = (float)s12;
        sf[4 * sb + 2] = __fmul_rn(xd, dmw);
        sf[4 * sb + 3] = (float)prod;
      }
      __syncwarp();
      if (lane == 0) {
        float sumf = 0.0f;
        for (int sb = 0; sb < nsb; ++sb) {
          sumf = __fmaf_rn(-sf[4 * sb + 2], sf[4 * sb + 3], sumf);
          sumf = __fmaf_rn(sf[4 * sb + 0], sf[4 * sb + 1], sumf);
        }
        result = sumf;
      }
    } else {  // Q6_K
      const int nsb = (int)(cols >> 8);
      const int l = lane & 7;
      for (int sb = lane >> 3; sb < nsb; sb += 4) {
        const uint8_t *blk = row + sb * 208;
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
        const int8_t *y = xq + sb * 256;
        int aux = 0;
        for (int j = 0; j < 16; ++j) {
          int part = 0;
          for (int half = 0; half < 2; ++half) {
            const int e = 16 * j + 8 * half + l;
            const int h = e >> 7, stream = (e >> 5) & 3, ll = e & 31;
            const uint8_t lb = blk[64 * h + (stream & 1) * 32 + ll];
            const int lo = (stream & 2) ? (lb >> 4) : (lb & 15);
            const int q = (lo | (((blk[128 + 32 * h + ll] >> (2 * stream)) & 3) << 4)) - 32;
            part += (int)y[e] * q;
          }
          aux += (int)sc[j] * part;
        }
        si[sb * 8 + l] = aux;
      }
      __syncwarp();
      float sums = 0.0f;
      if (lane < 8) {
        for (int sb = 0; sb < nsb; ++sb) {
          const float dd = __fmul_rn(f16_bits_to_f32(reinterpret_cast<const uint16_t *>(row + (int64_t)nsb * 208)[sb]), xs[sb]);
          sums = __fadd_rn(sums, __fmul_rn(dd, (float)si[sb * 8 + lane]));
        }
      }
      float tot = 0.0f;
      for (int k = 0; k < 8; ++k) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, sums, k));
      result = tot;
    }
    if (lane == 0) {
      const int64_t o = (int64_t)b * J.y_stride + r;
      J.y[o] = J.residual ? __fadd_rn(J.residual[o], result) : result;
    }
    __syncwarp();
  }
}

int32_t launch_gemv_exact(const GemvJob &J, const uint8_t *act, int32_t batch, cudaStream_t s) {
  const int nb = (int)(J.cols >> 5), nsb = (int)(J.cols >> 8);
  const int per_warp = J.qt == CMLD_Q8_0 ? nb * 4 : (J.qt == CMLD_Q4_K ? nsb * 16 : nsb * 32);
  const int per_warp16 = (per_warp + 15) & ~15;
  const unsigned grid = (unsigned)((J.rows + kExactWarps - 1) / kExactWarps);
  const size_t smem = (size_t)per_warp16 * kExactWarps;
  if (J.qt == CMLD_Q8_0) gemv_exact_kernel<CMLD_Q8_0><<<grid, kExactWarps * 32, smem, s>>>(J, act, batch, per_warp16);
  else if (J.qt == CMLD_Q4_K) gemv_exact_kernel<CMLD_Q4_K><<<grid, kExactWarps * 32, smem, s>>>(J, act, batch, per_warp16);
  else if (J.qt == CMLD_Q6_K) gemv_exact_kernel<CMLD_Q6_K><<<grid, kExactWarps * 32, smem, s>>>(J, act, batch, per_warp16);
  else return fail(CMLD_ERR_UNSUPPORTED, "gemv_exact: type %d", J.qt);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// One CTA per (row, query head); q already rotated, K/V already in the cache (the separate
// RoPE + KV-append kernel ran before).  Scores, their sum and the weighted values are
// accumulated in the CPU's order: a single accumulator over d, then over positions.
constexpr int kExactAttnThreads = 256;

__global__ void __launch_bounds__(kExactAttnThreads) attn_exact_kernel(AttnArgs a) {
  extern __shared__ float s_sc[];  // [n_pos] scores, then probabilities
  __shared__ float s_q[128];
  __shared__ float s_bcast[2];
  const int head = blockIdx.x, b = blockIdx.y;
  const int hd = a.head_dim;
  const int n_pos = a.positions[b] + 1;
  const int slot = a.slots[b];
  const int kvh = head / (a.n_heads / a.n_kv_heads);
  const __half *kbase = a.k_cache + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * hd;
  const __half *vbase = a.v_cache + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * hd;
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) s_q[d] = q[d];
  __syncthreads();
  // Tree verification: a position at or above tree_base takes part only if the row's mask names that node.  A
  // position left out is skipped in every sum below, so what remains is the linear decode of the node's own path.
  const uint32_t *mask = a.tree_mask ? a.tree_mask + (int64_t)b * a.tree_words : nullptr;
  auto live = [&](int p) -> bool {
    if (!mask || p < a.tree_base) return true;
    const int j = p - a.tree_base;
    return (mask[j >> 5] >> (j & 31)) & 1u;
  };
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x) {
    if (!live(p)) {
      s_sc[p] = -INFINITY;
      continue;
    }
    const __half *kr = kbase + (int64_t)p * hd;
    float s = 0.0f;
    for (int d = 0; d < hd; ++d) s = __fadd_rn(s, __fmul_rn(s_q[d], __half2float(kr[d])));
    s_sc[p] = __fmul_rn(s, a.scale);
  }
  __syncthreads();
  // maximum (order does not matter), then exp and the in-order sum by one thread
  float m = -INFINITY;
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x) m = fmaxf(m, s_sc[p]);
  m = warp_max(m);
  __shared__ float s_red[kExactAttnThreads / 32];
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = s_red[0];
    for (int w = 1; w < kExactAttnThreads / 32; ++w) mm = fmaxf(mm, s_red[w]);
    s_bcast[0] = mm;
  }
  __syncthreads();
  m = s_bcast[0];
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x)
    if (live(p)) s_sc[p] = expf_exact(__fsub_rn(s_sc[p], m));
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.0f;
    for (int p = 0; p < n_pos; ++p)
      if (live(p)) sum = __fadd_rn(sum, s_sc[p]);
    s_bcast[1] = __fdiv_rn(1.0f, sum);
  }
  __syncthreads();
  const float inv = s_bcast[1];
  float *out = a.out + (int64_t)b * a.q_stride + (int64_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.0f;
    for (int p = 0; p < n_pos; ++p)
      if (live(p)) o = __fadd_rn(o, __fmul_rn(__fmul_rn(s_sc[p], inv), __half2float(vbase[(int64_t)p * hd + d])));
    out[d] = o;
  }
}

int32_t launch_attention_exact(const AttnArgs &a, cudaStream_t s) {
  if (a.head_dim > 128) return fail(CMLD_ERR_SHAPE, "attention (reference order): head_dim %d > 128", a.head_dim);
  const size_t smem = (size_t)a.max_pos * 4;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    CMLD_CUDA(cudaFuncSetAttribute(attn_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::min<size_t>(smem, 200 * 1024)));
    configured = smem;
  }
  if (smem > 200 * 1024) return fail(CMLD_ERR_SHAPE, "attention (reference order): max_pos %lld too large", (long long)a.max_pos);
  dim3 grid((unsigned)a.n_heads, (unsigned)a.batch);
  attn_exact_kernel<<<grid, kExactAttnThreads, smem, s>>>(a);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
