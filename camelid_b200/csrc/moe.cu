// Mixtral-style top-k mixture-of-experts FFN for the decode step.
//
// CPU form (mixtral_moe_ffn, src/inference.rs:14142-14280 in the Camelid tree): router logits =
// f32 router . normed hidden; softmax_top_k (src/inference.rs:13940-13991): order by (logit
// desc, index asc), keep k, softmax over the kept logits, re-order by (weight desc, index asc);
// each selected expert runs gate/up -> SwiGLU -> down and `out += expert_out * weight` in that
// order; then the residual add.  Expert matrices that are not Q8_0 are multiplied as
// dequantised f32 weights against the *unquantised* f32 activation (the reference loads
// them as f32, src/inference.rs:832-846, and uses the plain dot of expert_matrix_view,
// :14109-14123) — so the expert matvec here keeps f32 activations: sum_i x_i * w_i is
// evaluated per 32- or 16-value group as scale * sum(x_i * code_i) - min * sum(x_i), which
// is the same real number with different f32 rounding points.
#include <algorithm>
#include <string>
#include <vector>

#include "actquant.cuh"

namespace cmld {

int32_t weight_upload(Weight &w, int32_t qt, int64_t rows, int64_t cols, const void *wire, uint64_t nbytes, cudaStream_t s);
void weight_free(Weight &w);

constexpr int kMaxExperts = 64;
constexpr int kMoeCols = 4;  // activation columns per pass of the expert matvec
constexpr int kMoeRows = 4;
constexpr int kMoeWarps = 4;

// total_cmp key of an f32 (Rust f32::total_cmp).
__device__ __forceinline__ int total_key(float f) {
  const int b = __float_as_int(f);
  return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}

// One CTA per token row: router logits, then top-k selection by thread 0.
__global__ void __launch_bounds__(256) moe_route_kernel(const float *__restrict__ x, const float *__restrict__ router, int hidden,
                                                        int n_exp, int k, int32_t *__restrict__ sel_idx, float *__restrict__ sel_w) {
  __shared__ float logits[kMaxExperts];
  __shared__ __align__(16) float prod[8][1024];
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *xr = x + (int64_t)b * hidden;
  // logits_e = ((0 + x0*r0) + x1*r1) + ...: the CPU's one-accumulator dot (dot_product_row,
  // src/inference.rs:29382-29409).  One warp per expert: the products of a 1024-value chunk are formed by all lanes
  // from coalesced loads (a product does not depend on the order), then lane 0 adds them in index order.
  for (int e = warp; e < n_exp; e += 8) {
    const float *r = router + (int64_t)e * hidden;
    float s = 0.0f;
    for (int i0 = 0; i0 < hidden; i0 += 1024) {
      const int cnt = min(1024, hidden - i0);
      for (int i = lane * 4; i < cnt; i += 128) {
        if (i + 4 <= cnt && ((hidden & 3) == 0)) {
          const float4 xv = __ldg(reinterpret_cast<const float4 *>(xr + i0 + i)), rv = __ldg(reinterpret_cast<const float4 *>(r + i0 + i));
          *reinterpret_cast<float4 *>(&prod[warp][i]) = make_float4(__fmul_rn(xv.x, rv.x), __fmul_rn(xv.y, rv.y), __fmul_rn(xv.z, rv.z), __fmul_rn(xv.w, rv.w));
        } else {
          for (int j = i; j < min(i + 4, cnt); ++j) prod[warp][j] = __fmul_rn(xr[i0 + j], r[i0 + j]);
        }
      }
      __syncwarp();
      if (lane == 0) {
        int i = 0;
        for (; i + 4 <= cnt; i += 4) {
          const float4 p4 = *reinterpret_cast<const float4 *>(&prod[warp][i]);
          s = __fadd_rn(s, p4.x);
          s = __fadd_rn(s, p4.y);
          s = __fadd_rn(s, p4.z);
          s = __fadd_rn(s, p4.w);
        }
        for (; i < cnt; ++i) s = __fadd_rn(s, prod[warp][i]);
      }
      __syncwarp();
    }
    if (lane == 0) logits[e] = s;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  int idx[kMaxExperts];
  float w[kMaxExperts];
  bool used[kMaxExperts];
  for (int e = 0; e < n_exp; ++e) used[e] = false;
  for (int s = 0; s < k; ++s) {  // selection sort: largest total_cmp key, lowest index on ties
    int best = -1;
    for (int e = 0; e < n_exp; ++e)
      if (!used[e] && (best < 0 || total_key(logits[e]) > total_key(logits[best]))) best = e;
    used[best] = true;
    idx[s] = best;
  }
  float mx = -INFINITY;
  for (int s = 0; s < k; ++s) mx = fmaxf(mx, logits[idx[s]]);
  float sum = 0.0f;
  for (int s = 0; s < k; ++s) {
    const float v = logits[idx[s]];
    w[s] = isfinite(v) ? expf_exact(__fsub_rn(v, mx)) : 0.0f;
    sum = __fadd_rn(sum, w[s]);
  }
  for (int s = 0; s < k; ++s) w[s] = sum > 0.0f ? __fdiv_rn(w[s], sum) : __fdiv_rn(1.0f, (float)k);
  for (int s = 1; s < k; ++s) {  // stable insertion by (weight desc, index asc)
    const int ci = idx[s];
    const float cw = w[s];
    int j = s - 1;
    while (j >= 0 && (total_key(w[j]) < total_key(cw) || (total_key(w[j]) == total_key(cw) && idx[j] > ci))) {
      idx[j + 1] = idx[j];
      w[j + 1] = w[j];
      --j;
    }
    idx[j + 1] = ci;
    w[j + 1] = cw;
  }
  for (int s = 0; s < k; ++s) {
    sel_idx[b * k + s] = idx[s];
    sel_w[b * k + s] = w[s];
  }
}

// Bucket the batch*k assignments by expert, in ascending assignment order.
__global__ void moe_group_kernel(const int32_t *__restrict__ sel_idx, int n_assign, int n_exp, int32_t *__restrict__ counts,
                                 int32_t *__restrict__ lists, int32_t *__restrict__ pos) {
  const int e = threadIdx.x;
  if (e >= n_exp) return;
  int n = 0;
  for (int a = 0; a < n_assign; ++a)
    if (sel_idx[a] == e) {
      if (pos) pos[a] = n;  // where assignment a sits in its expert's list
      lists[e * n_assign + n++] = a;
    }
  counts[e] = n;
}

// ------------------------------------------------------------------ expert matvecs on the tensor cores
//
// The reference multiplies the experts' dequantised weights with the UNQUANTISED f32 activation.  To keep that
// precision on the int8 tensor-core kernel, an activation vector x is written as the sum of three Q8_K vectors:
// x1 = Q8_K(x), x2 = Q8_K(x - x1), x3 = Q8_K(x - x1 - x2).  Every stage shrinks the remainder by about 1/254,
// so what is left after three is below 1e-7 of the block's largest value: the size of an f32 rounding error of the
// dot product itself.  The matvec runs over the three rows as if they were three tokens (exact integer dots, one
// f32 scale step per superblock) and the three results are added.  Rows of expert e (local index) live at
// [e*cap + 3*j + p] for the j-th assignment of its list, in the standard quantised-activation row layout.

struct Quant3Args {
  const float *x;        // source rows (mode 0: [token][cols]; mode 1: g3 / u3 result rows, 3 per assignment)
  const float *x2;       // mode 1: the "up" result rows
  int32_t mode;          // 0: x[token]; 1: SwiGLU(sum of 3 gate rows, sum of 3 up rows)
  int32_t cols, k, n_assign, first_expert, expert_step, cap;
  const int32_t *counts, *lists;
  uint8_t *act;          // [local expert][cap] rows of act_row_stride(cols) bytes
};

__global__ void __launch_bounds__(256) moe_quant3_kernel(const Quant3Args a) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int j = blockIdx.x, e_local = blockIdx.y, e = a.first_expert + e_local * a.expert_step;
  if (j >= a.counts[e]) return;
  const int asg = a.lists[e * a.n_assign + j];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t astride = act_row_stride(a.cols);
  const int64_t row0 = (int64_t)e_local * a.cap + 3 * j;
  const int n_chunks = a.cols >> 8;
  for (int ch = blockIdx.z * 8 + warp; ch < n_chunks; ch += 8 * gridDim.z) {
    const int e0 = ch * 256 + lane * 8;
    float v[8];
    if (a.mode == 0) {
      const float *src = a.x + (int64_t)(asg / a.k) * a.cols + e0;
      const float4 p = __ldcg(reinterpret_cast<const float4 *>(src)), q = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
      v[0] = p.x, v[1] = p.y, v[2] = p.z, v[3] = p.w, v[4] = q.x, v[5] = q.y, v[6] = q.z, v[7] = q.w;
    } else {
      float g[8], u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = u[i] = 0.0f;
#pragma unroll
      for (int p3 = 0; p3 < 3; ++p3) {  // the three partial results, added in order
        const float *gs = a.x + (row0 + p3) * a.cols + e0, *us = a.x2 + (row0 + p3) * a.cols + e0;
        const float4 g0 = __ldcg(reinterpret_cast<const float4 *>(gs)), g1 = __ldcg(reinterpret_cast<const float4 *>(gs) + 1);
        const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(us)), u1 = __ldcg(reinterpret_cast<const float4 *>(us) + 1);
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          g[i] = __fadd_rn(g[i], gv[i]);
          u[i] = __fadd_rn(u[i], uv[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = swiglu(g[i], u[i]);
    }
#pragma unroll
    for (int p3 = 0; p3 < 3; ++p3) {
      int q[8];
      float d;
      q8k_quantise_chunk(v, lane, q, d);
      uint8_t *row = a.act + (row0 + p3) * astride;
      *reinterpret_cast<uint2 *>(row + e0) = pack8(q);
      int s16 = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
      s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
      if ((lane & 1) == 0) reinterpret_cast<short *>(row + act_bsum_off(a.cols))[ch * 16 + (lane >> 1)] = (short)s16;
      if (lane == 0) reinterpret_cast<float *>(row + act_scale_off(a.cols))[ch] = d;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fsub_rn(v[i], __fmul_rn(d, (float)q[i]));  // what this stage did not capture
    }
  }
}

// h[b] (+)= sum_s w[b][s] * (sum of the three result rows of assignment (b, s)), in selection order from zero.
__global__ void moe_combine3_kernel(float *__restrict__ h, const float *__restrict__ y3, const float *__restrict__ sel_w,
                                    const int32_t *__restrict__ sel_idx, const int32_t *__restrict__ pos, int hidden, int k,
                                    int first_expert, int expert_step, int cap, int add_residual) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int b = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < hidden; c += gridDim.x * blockDim.x) {
    float out = 0.0f;
    for (int s = 0; s < k; ++s) {
      const int e = sel_idx[b * k + s];
      if ((e - first_expert) % expert_step != 0 || e < first_expert) continue;  // expert held by another rank
      const int64_t row = (int64_t)((e - first_expert) / expert_step) * cap + 3 * pos[b * k + s];
      const float *y = y3 + row * hidden + c;
      const float v = __fadd_rn(__fadd_rn(__ldcg(y), __ldcg(y + hidden)), __ldcg(y + 2 * hidden));
      out = __fadd_rn(out, __fmul_rn(v, sel_w[b * k + s]));
    }
    h[(int64_t)b * hidden + c] = add_residual ? __fadd_rn(h[(int64_t)b * hidden + c], out) : out;
  }
}

// float(code) of byte `sel` of w without an int->float conversion: place the byte in the
// mantissa of 2^23 and subtract 2^23 (exact for 0..255).
__device__ __forceinline__ float byte_to_float(uint32_t w, int sel) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | sel)) - 8388608.0f;
}

struct MoeGemvArgs {
  const uint8_t *w;  // expert slabs, device layout, rows_per_expert rows each
  int32_t qt;
  int64_t rows_per_expert, cols, stride;
  const float *x;   // activation rows
  int64_t x_stride;
  int32_t x_div;    // activation row of assignment a is a / x_div (k for gate/up, 1 for down)
  float *y;         // [n_assign][rows_per_expert]
  const int32_t *counts, *lists;
  int32_t n_assign;
  int32_t first_expert, expert_step;  // experts held locally: first_expert + i*expert_step
  const uint8_t *w2 = nullptr;        // ordered kernel: a second slab of the same shape and type (gate and up in one launch,
  float *y2 = nullptr;                // grid.z = 2), results into y2
};

template <int QT>
__global__ void __launch_bounds__(kMoeWarps * 32) moe_gemv_kernel(MoeGemvArgs a) {
  const int e_local = blockIdx.y;
  const int e = a.first_expert + e_local * a.expert_step;
  const int n = a.counts[e];
  if (n == 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t r0 = ((int64_t)blockIdx.x * kMoeWarps + warp) * kMoeRows;
  if (r0 >= a.rows_per_expert) return;
  const uint8_t *row[kMoeRows];
#pragma unroll
  for (int r = 0; r < kMoeRows; ++r)
    row[r] = a.w + ((int64_t)e_local * a.rows_per_expert + (r0 + r < a.rows_per_expert ? r0 + r : r0)) * a.stride;
  const int nsb = (int)(a.cols >> 8);
  const int units = nsb * 8;
  for (int c0 = 0; c0 < n; c0 += kMoeCols) {
    const float *xc[kMoeCols];
    int asg[kMoeCols];
#pragma unroll
    for (int c = 0; c < kMoeCols; ++c) {
      asg[c] = a.lists[e * a.n_assign + min(c0 + c, n - 1)];
      xc[c] = a.x + (int64_t)(asg[c] / a.x_div) * a.x_stride;
    }
    float acc[kMoeRows][kMoeCols];
#pragma unroll
    for (int r = 0; r < kMoeRows; ++r)
#pragma unroll
      for (int c = 0; c < kMoeCols; ++c) acc[r][c] = 0.0f;
    for (int u = lane; u < units; u += 32) {
      const int sb = u >> 3, t = u & 7;
      uint4 wq[kMoeRows];
#pragma unroll
      for (int r = 0; r < kMoeRows; ++r)
        wq[r] = ld_stream16(row[r] + (QT == CMLD_Q4_K ? (int64_t)sb * 144 + 16 + t * 16 : (int64_t)sb * 208 + t * 16));
      if (QT == CMLD_Q4_K) {
        const int j = t >> 1, h = t & 1;
        const int xo = sb * 256 + 64 * j + 16 * h;
        float dl[kMoeRows], dh[kMoeRows], ml[kMoeRows], mh[kMoeRows];
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r) {
          const uint4 meta = __ldg(reinterpret_cast<const uint4 *>(row[r] + (int64_t)sb * 144));
          const float d = f16_bits_to_f32((uint16_t)(meta.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(meta.x >> 16));
          int s0, m0, s1, m1;
          q4k_scale_min(2 * j, meta.y, meta.z, meta.w, s0, m0);
          q4k_scale_min(2 * j + 1, meta.y, meta.z, meta.w, s1, m1);
          dl[r] = __fmul_rn(d, (float)s0);
          dh[r] = __fmul_rn(d, (float)s1);
          ml[r] = __fmul_rn(dmin, (float)m0);
          mh[r] = __fmul_rn(dmin, (float)m1);
        }
        float dotl[kMoeRows][kMoeCols], doth[kMoeRows][kMoeCols], sxl[kMoeCols], sxh[kMoeCols];
#pragma unroll
        for (int c = 0; c < kMoeCols; ++c) {
          sxl[c] = sxh[c] = 0.0f;
#pragma unroll
          for (int r = 0; r < kMoeRows; ++r) dotl[r][c] = doth[r][c] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float fl[kMoeRows][4], fh[kMoeRows][4];
#pragma unroll
          for (int r = 0; r < kMoeRows; ++r) {
            const uint32_t w = k == 0 ? wq[r].x : (k == 1 ? wq[r].y : (k == 2 ? wq[r].z : wq[r].w));
            const uint32_t lo = w & 0x0f0f0f0fu, hi = (w >> 4) & 0x0f0f0f0fu;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              fl[r][i] = byte_to_float(lo, i);
              fh[r][i] = byte_to_float(hi, i);
            }
          }
#pragma unroll
          for (int c = 0; c < kMoeCols; ++c) {
            const float4 xl = __ldg(reinterpret_cast<const float4 *>(xc[c] + xo + 4 * k));
            const float4 xh = __ldg(reinterpret_cast<const float4 *>(xc[c] + xo + 32 + 4 * k));
            sxl[c] += (xl.x + xl.y) + (xl.z + xl.w);
            sxh[c] += (xh.x + xh.y) + (xh.z + xh.w);
#pragma unroll
            for (int r = 0; r < kMoeRows; ++r) {
              dotl[r][c] = __fmaf_rn(fl[r][0], xl.x, __fmaf_rn(fl[r][1], xl.y, __fmaf_rn(fl[r][2], xl.z, __fmaf_rn(fl[r][3], xl.w, dotl[r][c]))));
              doth[r][c] = __fmaf_rn(fh[r][0], xh.x, __fmaf_rn(fh[r][1], xh.y, __fmaf_rn(fh[r][2], xh.z, __fmaf_rn(fh[r][3], xh.w, doth[r][c]))));
            }
          }
        }
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r)
#pragma unroll
          for (int c = 0; c < kMoeCols; ++c)
            acc[r][c] += (dl[r] * dotl[r][c] - ml[r] * sxl[c]) + (dh[r] * doth[r][c] - mh[r] * sxh[c]);
      } else {  // Q6_K
        const int h = t >> 2, sp = (t >> 1) & 1, cc = t & 1;
        const int jlo = 8 * h + 2 * sp + cc;
        const int xo = sb * 256 + jlo * 16;
        float dl[kMoeRows], dh[kMoeRows];
        uint4 qh4[kMoeRows];
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r) {
          qh4[r] = __ldg(reinterpret_cast<const uint4 *>(row[r] + (int64_t)sb * 208 + 128 + 32 * h + 16 * cc));
          const float d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(row[r] + (int64_t)nsb * 208) + sb));
          const int8_t *sc = reinterpret_cast<const int8_t *>(row[r] + (int64_t)sb * 208 + 192);
          dl[r] = __fmul_rn(d, (float)__ldg(sc + jlo));
          dh[r] = __fmul_rn(d, (float)__ldg(sc + jlo + 4));
        }
        float dotl[kMoeRows][kMoeCols], doth[kMoeRows][kMoeCols], sxl[kMoeCols], sxh[kMoeCols];
#pragma unroll
        for (int c = 0; c < kMoeCols; ++c) {
          sxl[c] = sxh[c] = 0.0f;
#pragma unroll
          for (int r = 0; r < kMoeRows; ++r) dotl[r][c] = doth[r][c] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float fl[kMoeRows][4], fh[kMoeRows][4];
#pragma unroll
          for (int r = 0; r < kMoeRows; ++r) {
            const uint32_t w = k == 0 ? wq[r].x : (k == 1 ? wq[r].y : (k == 2 ? wq[r].z : wq[r].w));
            const uint32_t q = k == 0 ? qh4[r].x : (k == 1 ? qh4[r].y : (k == 2 ? qh4[r].z : qh4[r].w));
            const uint32_t lo = (w & 0x0f0f0f0fu) | (((q >> (2 * sp)) & 0x03030303u) << 4);
            const uint32_t hi = ((w >> 4) & 0x0f0f0f0fu) | (((q >> (2 * sp + 4)) & 0x03030303u) << 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              fl[r][i] = byte_to_float(lo, i);
              fh[r][i] = byte_to_float(hi, i);
            }
          }
#pragma unroll
          for (int c = 0; c < kMoeCols; ++c) {
            const float4 xl = __ldg(reinterpret_cast<const float4 *>(xc[c] + xo + 4 * k));
            const float4 xh = __ldg(reinterpret_cast<const float4 *>(xc[c] + xo + 64 + 4 * k));
            sxl[c] += (xl.x + xl.y) + (xl.z + xl.w);
            sxh[c] += (xh.x + xh.y) + (xh.z + xh.w);
#pragma unroll
            for (int r = 0; r < kMoeRows; ++r) {
              dotl[r][c] = __fmaf_rn(fl[r][0], xl.x, __fmaf_rn(fl[r][1], xl.y, __fmaf_rn(fl[r][2], xl.z, __fmaf_rn(fl[r][3], xl.w, dotl[r][c]))));
              doth[r][c] = __fmaf_rn(fh[r][0], xh.x, __fmaf_rn(fh[r][1], xh.y, __fmaf_rn(fh[r][2], xh.z, __fmaf_rn(fh[r][3], xh.w, doth[r][c]))));
            }
          }
        }
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r)
#pragma unroll
          for (int c = 0; c < kMoeCols; ++c)
            acc[r][c] += dl[r] * (dotl[r][c] - 32.0f * sxl[c]) + dh[r] * (doth[r][c] - 32.0f * sxh[c]);
      }
    }
#pragma unroll
    for (int r = 0; r < kMoeRows; ++r)
#pragma unroll
      for (int c = 0; c < kMoeCols; ++c) {
        const float v = warp_sum(acc[r][c]);
        if (lane == 0 && r0 + r < a.rows_per_expert && c0 + c < n) a.y[(int64_t)asg[c] * a.rows_per_expert + r0 + r] = v;
      }
  }
}

// ------------------------------------------------------------------ expert matvec in the CPU path's order
//
// The reference holds non-Q8_0 expert tensors as dequantised f32 and multiplies them with the f32 activation by
// its one-accumulator dot (expert_matrix_view else-branch, src/inference.rs:14109-14123; dot_product_row,
// :29382-29409): y[r] = ((0 + x0*w0) + x1*w1) + ... with w_i the dequantised weight (Q4KBlock::dequantize /
// Q6KBlock::dequantize, src/tensor/mod.rs:5903-5924 and :6039-6066).  One thread owns one output row and walks
// its weights in index order, dequantising on the way; up to kOrdCols assignments of the expert share the
// dequantised weight (independent chains, which also cover each other's addition latency).
// The weights reach a lane through a private ring in shared memory that the lane's warp fills with cp.async: the 32
// rows of a warp are 32 separate byte ranges, and a load instruction whose lanes each touch another row costs 32
// cache-line lookups, so the warp copies a superblock step of its 32 rows with lanes walking consecutive 16-byte
// pieces (9 or 13 per row) and each lane then reads its own row from the ring (row pitch 144 / 208 bytes: an odd
// number of 16-byte units, conflict-free).
constexpr int kOrdCols = 4;
constexpr int kOrdWarps = 2;   // small CTAs: the few rows of the active experts spread over all SMs
constexpr int kOrdThreads = kOrdWarps * 32;
constexpr int kOrdStages = 3;

__device__ __forceinline__ void ord_cp16(void *dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// One pass over the row for NC assignments of the expert (NC columns share each dequantised weight; their chains are
// independent and cover each other's addition latency).
template <int QT, int NC, class Issue>
__device__ __forceinline__ void ord_pass(const MoeGemvArgs &a, float *yout, int e, int c0, int nsb, const uint8_t *ring, const uint8_t *row, int lane,
                                         int64_t r, bool row_ok, Issue &&issue) {
  constexpr int SB = QT == CMLD_Q4_K ? 144 : 208;
  const float *xc[NC];
  int asg[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    asg[c] = a.lists[e * a.n_assign + c0 + c];
    xc[c] = a.x + (int64_t)(asg[c] / a.x_div) * a.x_stride;
  }
  float acc[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) acc[c] = 0.0f;
  __syncwarp();  // the ring is free: every lane is done with the previous pass
  for (int sb = 0; sb < kOrdStages - 1; ++sb) issue(sb);
  for (int sb = 0; sb < nsb; ++sb) {
    issue(sb + kOrdStages - 1);  // into the stage step sb-1 used: every lane left it at the __syncwarp below
    asm volatile("cp.async.wait_group %0;" ::"n"(kOrdStages - 1) : "memory");
    __syncwarp();  // the other lanes' pieces of step sb are visible
    const uint8_t *stage = ring + (sb % kOrdStages) * (32 * SB + kOrdCols * 1024);
    const uint8_t *blk = stage + lane * SB;
    const float *xs = reinterpret_cast<const float *>(stage + 32 * SB);  // [assignment][256]
    if (QT == CMLD_Q4_K) {
      const uint4 meta = *reinterpret_cast<const uint4 *>(blk);
      const float d = f16_bits_to_f32((uint16_t)(meta.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(meta.x >> 16));
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * p), q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * p);
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int hl = 0; hl < 2; ++hl) {  // low nibbles = values 64p..64p+31, high nibbles = the next 32
          int sc, m;
          q4k_scale_min(2 * p + hl, meta.y, meta.z, meta.w, sc, m);
          const float dsc = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)m);
          const int xo = 64 * p + 32 * hl;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t nib = hl ? (qw[k] >> 4) & 0x0f0f0f0fu : qw[k] & 0x0f0f0f0fu;
            float w4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w4[i] = __fsub_rn(__fmul_rn(dsc, byte_to_float(nib, i)), dm);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              const float4 xv = *reinterpret_cast<const float4 *>(xs + c * 256 + xo + 4 * k);
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.x, w4[0]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.y, w4[1]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.z, w4[2]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.w, w4[3]));
            }
          }
        }
      }
    } else {  // Q6_K: values 128h + 32*stream + l, stream 0/1 = low nibbles of ql[64h + 32*stream' ..], 2/3 = high nibbles
      const float d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(row + (int64_t)nsb * 208) + sb));
      const uint4 scw = *reinterpret_cast<const uint4 *>(blk + 192);
      const uint32_t scs[4] = {scw.x, scw.y, scw.z, scw.w};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 h0 = *reinterpret_cast<const uint4 *>(blk + 128 + 32 * h), h1 = *reinterpret_cast<const uint4 *>(blk + 144 + 32 * h);
        const uint32_t qh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int stream = 0; stream < 4; ++stream) {
          const uint4 l0 = *reinterpret_cast<const uint4 *>(blk + 64 * h + 32 * (stream & 1)),
                      l1 = *reinterpret_cast<const uint4 *>(blk + 64 * h + 32 * (stream & 1) + 16);
          const uint32_t ql[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int j = 8 * h + 2 * stream + (k >> 2);  // scale index of values 16j..16j+15
            const float dsc = __fmul_rn(d, (float)(int)(int8_t)(scs[j >> 2] >> (8 * (j & 3))));
            const uint32_t lo = (stream & 2) ? (ql[k] >> 4) & 0x0f0f0f0fu : ql[k] & 0x0f0f0f0fu;
            const uint32_t q6 = lo | (((qh[k] >> (2 * stream)) & 0x03030303u) << 4);
            float w4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w4[i] = __fmul_rn(dsc, byte_to_float(q6, i) - 32.0f);
            const int xo = 128 * h + 32 * stream + 4 * k;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              const float4 xv = *reinterpret_cast<const float4 *>(xs + c * 256 + xo);
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.x, w4[0]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.y, w4[1]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.z, w4[2]));
              acc[c] = __fadd_rn(acc[c], __fmul_rn(xv.w, w4[3]));
            }
          }
        }
      }
    }
    __syncwarp();  // every lane is done with this stage before a later copy overwrites it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (row_ok) {
#pragma unroll
    for (int c = 0; c < NC; ++c)
      yout[(int64_t)asg[c] * a.rows_per_expert + r] = acc[c];
  }
}

template <int QT>
__global__ void __launch_bounds__(kOrdThreads) moe_gemv_ordered_kernel(MoeGemvArgs a) {
  extern __shared__ __align__(16) uint8_t ord_smem[];
  constexpr int SB = QT == CMLD_Q4_K ? 144 : 208, SEG = SB / 16;
  const int e_local = blockIdx.y;
  const int e = a.first_expert + e_local * a.expert_step;
  const int n = a.counts[e];
  if (n == 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = ((int64_t)blockIdx.x * kOrdWarps + warp) * 32;  // this warp's first row
  if (r0 >= a.rows_per_expert) return;
  const int64_t r = r0 + lane;
  const bool row_ok = r < a.rows_per_expert;
  const uint8_t *w0 = (blockIdx.z ? a.w2 : a.w) + (int64_t)e_local * a.rows_per_expert * a.stride;
  float *yout = blockIdx.z ? a.y2 : a.y;
  const int nsb = (int)(a.cols >> 8);
  constexpr int STAGE = 32 * SB + kOrdCols * 1024;  // the warp's 32 superblocks, then 256 activation values per assignment
  uint8_t *ring = ord_smem + warp * (kOrdStages * STAGE);
  const float *xc_issue[kOrdCols] = {nullptr, nullptr, nullptr, nullptr};
  int nc_issue = 0;
  // piece c of a step: row c / SEG of the warp, 16-byte unit c % SEG of that row's superblock
  auto issue = [&](int sb) {
    if (sb < nsb) {
      uint8_t *dst = ring + (sb % kOrdStages) * STAGE;
      for (int c = lane; c < nc_issue * 64; c += 32)  // the activation chunk of every live assignment: 64 pieces each
        ord_cp16(dst + 32 * SB + c * 16, xc_issue[c >> 6] + sb * 256 + (c & 63) * 4);
#pragma unroll
      for (int j = 0; j < (32 * SEG + 31) / 32; ++j) {
        const int c = lane + 32 * j;
        if (c < 32 * SEG) {
          const int64_t rr = min(r0 + c / SEG, a.rows_per_expert - 1);
          ord_cp16(dst + c * 16, w0 + rr * a.stride + (int64_t)sb * SB + (c % SEG) * 16);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const uint8_t *row = w0 + min(r, a.rows_per_expert - 1) * a.stride;  // this lane's row (Q6_K: its f16 scales behind the blocks)
  for (int c0 = 0; c0 < n; c0 += kOrdCols) {
    nc_issue = min(kOrdCols, n - c0);
    for (int c = 0; c < nc_issue; ++c) xc_issue[c] = a.x + (int64_t)(a.lists[e * a.n_assign + c0 + c] / a.x_div) * a.x_stride;
    switch (nc_issue) {
      case 1: ord_pass<QT, 1>(a, yout, e, c0, nsb, ring, row, lane, r, row_ok, issue); break;
      case 2: ord_pass<QT, 2>(a, yout, e, c0, nsb, ring, row, lane, r, row_ok, issue); break;
      case 3: ord_pass<QT, 3>(a, yout, e, c0, nsb, ring, row, lane, r, row_ok, issue); break;
      default: ord_pass<QT, 4>(a, yout, e, c0, nsb, ring, row, lane, r, row_ok, issue); break;
    }
  }
}

// h[b] += sum_s down[b*k+s] * w[b][s], accumulated in selection order from zero, as the CPU does.
__global__ void moe_combine_kernel(float *__restrict__ h, const float *__restrict__ down, const float *__restrict__ sel_w,
                                   const int32_t *__restrict__ sel_idx, int hidden, int k, int first_expert, int expert_step,
                                   int add_residual) {
  const int b = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < hidden; c += gridDim.x * blockDim.x) {
    float out = 0.0f;
    for (int s = 0; s < k; ++s) {
      const int e = sel_idx[b * k + s];
      if (expert_step > 1 && (e - first_expert) % expert_step != 0) continue;  // expert held by another rank
      out = __fadd_rn(out, __fmul_rn(down[((int64_t)b * k + s) * hidden + c], sel_w[b * k + s]));
    }
    h[(int64_t)b * hidden + c] = add_residual ? __fadd_rn(h[(int64_t)b * hidden + c], out) : out;
  }
}

}  // namespace cmld

using namespace cmld;

namespace cmld {

int32_t moe_route(const float *normed, const float *router, int hidden, int n_exp, int k, int batch, int32_t *sel_idx,
                  float *sel_w, int32_t *counts, int32_t *lists, cudaStream_t s, int32_t *pos) {
  if (n_exp > kMaxExperts) return fail(CMLD_ERR_SHAPE, "more than %d experts", kMaxExperts);
  moe_route_kernel<<<batch, 256, 0, s>>>(normed, router, hidden, n_exp, k, sel_idx, sel_w);
  CMLD_CUDA(cudaGetLastError());
  moe_group_kernel<<<1, kMaxExperts, 0, s>>>(sel_idx, batch * k, n_exp, counts, lists, pos);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t moe_expert_gemv(const Weight &slab, int64_t rows_per_expert, int n_local_experts, int first_expert, int expert_step,
                        const float *x, int64_t x_stride, int x_div, float *y, const int32_t *counts, const int32_t *lists,
                        int n_assign, cudaStream_t s) {
  MoeGemvArgs a{slab.data, slab.qt, rows_per_expert, slab.cols, slab.stride, x, x_stride, x_div, y, counts, lists, n_assign,
                first_expert, expert_step};
  dim3 grid((unsigned)((rows_per_expert + kMoeRows * kMoeWarps - 1) / (kMoeRows * kMoeWarps)), (unsigned)n_local_experts);
  if (slab.qt == CMLD_Q4_K) moe_gemv_kernel<CMLD_Q4_K><<<grid, kMoeWarps * 32, 0, s>>>(a);
  else if (slab.qt == CMLD_Q6_K) moe_gemv_kernel<CMLD_Q6_K><<<grid, kMoeWarps * 32, 0, s>>>(a);
  else return fail(CMLD_ERR_UNSUPPORTED, "expert tensors must be Q4_K or Q6_K");
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t moe_expert_gemv_ordered(const Weight &slab, int64_t rows_per_expert, int n_local_experts, int first_expert, int expert_step,
                                const float *x, int64_t x_stride, int x_div, float *y, const int32_t *counts, const int32_t *lists,
                                int n_assign, cudaStream_t s, const Weight *slab2, float *y2) {
  MoeGemvArgs a{slab.data, slab.qt, rows_per_expert, slab.cols, slab.stride, x, x_stride, x_div, y, counts, lists, n_assign,
                first_expert, expert_step};
  if (slab2) {
    if (slab2->qt != slab.qt || slab2->cols != slab.cols || slab2->stride != slab.stride || !y2) return fail(CMLD_ERR_SHAPE, "paired expert slabs differ in shape or type");
    a.w2 = slab2->data;
    a.y2 = y2;
  }
  if (slab.cols % 256) return fail(CMLD_ERR_SHAPE, "expert tensor width %lld is not a multiple of 256", (long long)slab.cols);
  dim3 grid((unsigned)((rows_per_expert + kOrdThreads - 1) / kOrdThreads), (unsigned)n_local_experts, slab2 ? 2u : 1u);
  static bool attr4 = false, attr6 = false;
  if (slab.qt == CMLD_Q4_K) {
    const int smem = kOrdWarps * kOrdStages * (32 * 144 + kOrdCols * 1024);
    if (!attr4) {
      CMLD_CUDA(cudaFuncSetAttribute(moe_gemv_ordered_kernel<CMLD_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr4 = true;
    }
    moe_gemv_ordered_kernel<CMLD_Q4_K><<<grid, kOrdThreads, smem, s>>>(a);
  } else if (slab.qt == CMLD_Q6_K) {
    const int smem = kOrdWarps * kOrdStages * (32 * 208 + kOrdCols * 1024);
    if (!attr6) {
      CMLD_CUDA(cudaFuncSetAttribute(moe_gemv_ordered_kernel<CMLD_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr6 = true;
    }
    moe_gemv_ordered_kernel<CMLD_Q6_K><<<grid, kOrdThreads, smem, s>>>(a);
  } else {
    return fail(CMLD_ERR_UNSUPPORTED, "expert tensors must be Q4_K or Q6_K");
  }
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t moe_combine(float *h, const float *down, const float *sel_w, const int32_t *sel_idx, int hidden, int k, int batch,
                    int first_expert, int expert_step, bool add_residual, cudaStream_t s) {
  dim3 grid((unsigned)((hidden + 255) / 256), (unsigned)batch);
  moe_combine_kernel<<<grid, 256, 0, s>>>(h, down, sel_w, sel_idx, hidden, k, first_expert, expert_step, add_residual ? 1 : 0);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// Three-stage Q8_K rows of the experts' operands.  mode 0: from the token rows x[token][cols]; mode 1: from the
// gate/up result rows (SwiGLU of their sums).
int32_t moe_quant3(const float *x, const float *x2, int mode, int cols, int k, int n_assign, int n_local, int first_expert,
                   int expert_step, int cap, const int32_t *counts, const int32_t *lists, uint8_t *act, cudaStream_t s) {
  if (cols % 256) return fail(CMLD_ERR_SHAPE, "expert operand width %d is not a multiple of 256", cols);
  Quant3Args a{x, x2, mode, cols, k, n_assign, first_expert, expert_step, cap, counts, lists, act};
  const int z = std::max(1, std::min(8, (cols >> 8) / 8));  // CTAs that share one row's chunks
  moe_quant3_kernel<<<dim3((unsigned)n_assign, (unsigned)n_local, (unsigned)z), 256, 0, s>>>(a);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t moe_combine3(float *h, const float *y3, const float *sel_w, const int32_t *sel_idx, const int32_t *pos, int hidden, int k,
                     int batch, int first_expert, int expert_step, int cap, bool add_residual, cudaStream_t s) {
  dim3 grid((unsigned)((hidden + 255) / 256), (unsigned)batch);
  moe_combine3_kernel<<<grid, 256, 0, s>>>(h, y3, sel_w, sel_idx, pos, hidden, k, first_expert, std::max(1, expert_step), cap,
                                           add_residual ? 1 : 0);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
