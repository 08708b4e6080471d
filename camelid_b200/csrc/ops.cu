// Per-token work around the matvecs: RMSNorm / SwiGLU fused with activation quantisation,
// RoPE fused with the f16 KV-cache write, and greedy argmax.
#include "actquant.cuh"
#include "exact_sum.cuh"

namespace cmld {

// ------------------------------------------------------------------ norm / SwiGLU -> quantised activation
//
// One CTA per batch row.  v = (x*scale)*w (rms_norm_into, src/tensor/mod.rs:2740-2764 in the
// Camelid tree), or v = g/(1+exp(-g))*u (src/inference.rs:13231-13236), or v = x.  The
// mean-square has the bits of the CPU's sequential sum.  v is then quantised the way the CPU
// quantises a matvec operand:
//   Q8_K (quantize_q8_k_blocks, src/inference.rs:23121-23152): first max |v| of each 256 keeps
//        its sign, iscale = -127/max, q = min(127, rne(iscale*v)), d = 1/iscale;
//   Q8_0 (quantize_q8_0_block, src/inference.rs:22510-22528): d = amax/127 kept as its f16
//        rounding, q = round-half-away(v * (1/d_unrounded)) clamped to [-128,127].
constexpr int kNormThreads = 256;
constexpr int kNormMaxExact = 8192;  // widest row whose squares are summed by all warps (exact_sum.cuh); wider rows by one thread

template <int MODE>  // 0 plain, 1 rmsnorm, 2 swiglu
__global__ void __launch_bounds__(kNormThreads) norm_quant_kernel(NormQuantArgs a) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float *x = a.x + (int64_t)b * a.cols;
  const float *x2 = MODE == 2 ? a.x2 + (int64_t)b * a.cols : nullptr;
  float scale = 1.0f;
  if (MODE == 1) {
    __shared__ float s_scale;
    // the CPU's order: one accumulator, squares added in index order (rms_norm_into, src/tensor/mod.rs:2755)
    if ((a.cols & 255) == 0 && a.cols <= kNormMaxExact) {
      // the same bits from all the warps (exact_sum.cuh)
      extern __shared__ __align__(16) uint8_t dyn_smem[];  // cols floats, then the exact sum's workspace
      float *sq = reinterpret_cast<float *>(dyn_smem);
      for (int64_t i = threadIdx.x; i < a.cols; i += kNormThreads) sq[i] = __fmul_rn(x[i], x[i]);
      const float t = xsum::cta_sum<kNormThreads / 32>(sq, (int)a.cols, warp, lane, 1, dyn_smem + a.cols * 4);
      if (threadIdx.x == 0) s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)a.cols), a.eps)));
    } else if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int64_t i = 0; i < a.cols; ++i) t = __fadd_rn(t, __fmul_rn(x[i], x[i]));
      s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)a.cols), a.eps)));
    }
    __syncthreads();
    scale = s_scale;
  }
  const int64_t n_chunks = (a.cols + 255) >> 8;
  const int64_t astride = act_row_stride(a.cols);
  // every CTA of a row repeats the mean-square (cheap) and quantises its own 256-value chunks
  for (int64_t ch = (int64_t)blockIdx.x * nwarps + warp; ch < n_chunks; ch += (int64_t)gridDim.x * nwarps) {
    const int64_t e0 = ch * 256 + lane * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t e = e0 + i;
      float t = 0.0f;
      if (e < a.cols) {
        if (MODE == 1) t = __fmul_rn(__fmul_rn(x[e], scale), a.weight[e]);
        else if (MODE == 2) {
          const float g = x[e];
          t = swiglu(g, x2[e]);
        } else t = x[e];
        if (a.out) a.out[(int64_t)b * a.cols + e] = t;
      }
      v[i] = t;
    }
    if (a.act_q8_k && e0 < a.cols) {
      uint8_t *act = a.act + b * astride;
      float amax = 0.0f, mx = 0.0f;
      int idx = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (fabsf(v[i]) > amax) {
          amax = fabsf(v[i]);
          mx = v[i];
          idx = lane * 8 + i;
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oa > amax || (oa == amax && oi < idx)) {
          amax = oa;
          mx = om;
          idx = oi;
        }
      }
      int q[8];
      float d = 0.0f;
      if (amax == 0.0f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = 0;
      } else {
        const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = min(127, __float2int_rn(__fmul_rn(iscale, v[i])));
        d = __fdiv_rn(1.0f, iscale);
      }
      uint2 packed;
      packed.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
      packed.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
      *reinterpret_cast<uint2 *>(act + e0) = packed;
      int s = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if ((lane & 1) == 0) reinterpret_cast<short *>(act + act_bsum_off(a.cols))[ch * 16 + (lane >> 1)] = (short)s;
      if (lane == 0) reinterpret_cast<float *>(act + act_scale_off(a.cols))[ch] = d;
    }
    if (a.act_q8_0) {
      uint8_t *act = (a.act_q8_k ? a.act2 : a.act) + b * astride;
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const float du = __fdiv_rn(amax, 127.0f);
      const float inv = du == 0.0f ? 0.0f : __fdiv_rn(1.0f, du);
      if (e0 < a.cols) {
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = (int)fminf(fmaxf(roundf(__fmul_rn(v[i], inv)), -128.0f), 127.0f);
        uint2 packed;
        packed.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
        packed.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
        *reinterpret_cast<uint2 *>(act + e0) = packed;
        if ((lane & 3) == 0)
          reinterpret_cast<float *>(act + act_scale_off(a.cols))[e0 >> 5] = f16_bits_to_f32(f32_to_f16_bits(du));
      }
    }
  }
}

int32_t launch_norm_quant(const NormQuantArgs &a, cudaStream_t s) {
  if (a.cols % 32 != 0) return fail(CMLD_ERR_SHAPE, "activation width %lld is not a multiple of 32", (long long)a.cols);
  if (a.act_q8_k && a.cols % 256 != 0)
    return fail(CMLD_ERR_SHAPE, "Q8_K activation width %lld is not a multiple of 256", (long long)a.cols);
  if (a.batch <= 0) return CMLD_OK;
  const int mode = a.x2 ? 2 : (a.weight ? 1 : 0);
  const int64_t n_chunks = (a.cols + 255) >> 8;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)((n_chunks + kNormThreads / 32 - 1) / (kNormThreads / 32)), (unsigned)a.batch);
  cfg.blockDim = dim3(kNormThreads);
  cfg.stream = s;
  if (mode == 1 && a.cols % 256 == 0 && a.cols <= kNormMaxExact) cfg.dynamicSmemBytes = (size_t)a.cols * 4 + xsum::workspace_bytes((int)a.cols);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  static bool carveout_set = false;
  if (!carveout_set) {
    prefer_max_smem_carveout(norm_quant_kernel<0>);
    prefer_max_smem_carveout(norm_quant_kernel<1>);
    prefer_max_smem_carveout(norm_quant_kernel<2>);
    CMLD_CUDA(cudaFuncSetAttribute(norm_quant_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kNormMaxExact * 4 + xsum::workspace_bytes(kNormMaxExact)));
    carveout_set = true;
  }
  if (mode == 0) CMLD_CUDA(cudaLaunchKernelEx(&cfg, norm_quant_kernel<0>, a));
  else if (mode == 1) CMLD_CUDA(cudaLaunchKernelEx(&cfg, norm_quant_kernel<1>, a));
  else CMLD_CUDA(cudaLaunchKernelEx(&cfg, norm_quant_kernel<2>, a));
  return CMLD_OK;
}

// ------------------------------------------------------------------ RoPE + KV write
//
// apply_rope_to_row (src/inference/rope.rs:495-530): x0' = x0*c - x1*s, x1' = x0*s + x1*c on
// pairs (2i,2i+1) (Llama) or (i, i+rope_dim/2) (split-half); then K and V are rounded to f16
// into the cache at the row's position (store_kv_head_row, src/inference/kv_cache.rs:846-876).
__global__ void rope_kv_kernel(RopeKvArgs a) {
  const int b = blockIdx.y;
  const int half = a.rope_dim / 2;
  const int hd = a.head_dim;
  const int n_qp = a.n_heads * half, n_kp = a.n_kv_heads * half;
  const int n_kpass = a.n_kv_heads * (hd - a.rope_dim);
  const int n_v = a.n_kv_heads * hd;
  const int total = n_qp + n_kp + n_kpass + n_v;
  const int pos = a.positions[b];
  const int slot = a.slots[b];
  if (pos < 0 || pos >= a.max_pos) return;
  const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
  const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
  float *q = a.q + (int64_t)b * a.q_stride;
  const float *k = a.k + (int64_t)b * a.kv_stride;
  const float *v = a.v + (int64_t)b * a.kv_stride;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    if (i < n_qp + n_kp) {
      const bool is_q = i < n_qp;
      const int j = is_q ? i : i - n_qp;
      const int h = j / half, p = j % half;
      const int d0 = a.split_half ? p : 2 * p, d1 = a.split_half ? p + half : 2 * p + 1;
      const float c = ct[p], s = st[p];
      if (is_q) {
        const float x0 = q[h * hd + d0], x1 = q[h * hd + d1];
        q[h * hd + d0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        q[h * hd + d1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
      } else {
        const float x0 = k[h * hd + d0], x1 = k[h * hd + d1];
        __half *dst = a.k_cache + (((int64_t)slot * a.n_kv_heads + h) * a.max_pos + pos) * hd;
        dst[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        dst[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
      }
    } else if (i < n_qp + n_kp + n_kpass) {
      const int j = i - n_qp - n_kp;
      const int h = j / (hd - a.rope_dim), d = a.rope_dim + j % (hd - a.rope_dim);
      a.k_cache[(((int64_t)slot * a.n_kv_heads + h) * a.max_pos + pos) * hd + d] = __float2half_rn(k[h * hd + d]);
    } else {
      const int j = i - n_qp - n_kp - n_kpass;
      const int h = j / hd, d = j % hd;
      a.v_cache[(((int64_t)slot * a.n_kv_heads + h) * a.max_pos + pos) * hd + d] = __float2half_rn(v[h * hd + d]);
    }
  }
}

int32_t launch_rope_kv(const RopeKvArgs &a, cudaStream_t s) {
  const int half = a.rope_dim / 2;
  const int total = a.n_heads * half + a.n_kv_heads * half + a.n_kv_heads * (a.head_dim - a.rope_dim) +
                    a.n_kv_heads * a.head_dim;
  dim3 grid((unsigned)((total + 255) / 256), (unsigned)a.batch);
  rope_kv_kernel<<<grid, 256, 0, s>>>(a);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// ------------------------------------------------------------------ greedy argmax
//
// greedy_sample (src/inference.rs:8904-8917): strict '>', so the lowest index of the maximum
// wins.  Stage 1: kArgmaxBlocks CTAs per row each reduce a contiguous slice; the CTA that
// takes the last ticket reduces the partials and, for the on-device token loop, feeds the
// result back (next token, position + 1, history).
constexpr int kArgmaxBlocks = 64;
constexpr int kArgmaxThreads = 256;
int argmax_blocks() { return kArgmaxBlocks; }

__device__ __forceinline__ void argmax_combine(float &v, int &i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

__global__ void __launch_bounds__(kArgmaxThreads)
    argmax_kernel(const float *__restrict__ x, int64_t n, float *part_val, int32_t *part_idx, uint32_t *ticket,
                  int32_t *out_idx, int32_t *next_tokens, int32_t *positions, int32_t *history, int32_t *hist_len,
                  int32_t batch, unsigned long long *key_out, int32_t idx_offset) {
  const int b = blockIdx.y;
  const float *row = x + (int64_t)b * n;
  const int64_t per = (n + gridDim.x - 1) / gridDim.x;
  const int64_t lo = blockIdx.x * per, hi = min(n, lo + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v > bv) {
      bv = v;
      bi = (int)i;
    }
  }
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ int si[kArgmaxThreads / 32];
  __shared__ bool last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) argmax_combine(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w) argmax_combine(bv, bi, sv[w], si[w]);
    part_val[b * gridDim.x + blockIdx.x] = bv;
    part_idx[b * gridDim.x + blockIdx.x] = bi;
    __threadfence();
    last = atomicAdd(&ticket[b], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (warp == 0) {
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (int k = lane; k < (int)gridDim.x; k += 32)
      argmax_combine(v, i, __ldcg(&part_val[b * gridDim.x + k]), __ldcg(&part_idx[b * gridDim.x + k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_combine(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
    if (lane == 0) {
      if (i == 0x7fffffff) i = 0;  // all-NaN or -inf row
      ticket[b] = 0;
      if (key_out) {
        // order-preserving bits of the value above, inverted global index below: an unsigned max over
        // the shards picks the largest value and, among equals, the lowest index
        uint32_t u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        key_out[b] = ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)(i + idx_offset));
        return;
      }
      out_idx[b] = i;
      if (next_tokens) {
        next_tokens[b] = i;
        positions[b] += 1;
        const int step = hist_len[b];
        history[(int64_t)step * batch + b] = i;
        hist_len[b] = step + 1;
      }
    }
  }
}

// history: [max_steps][batch] ids; hist_len lives right after the tickets: ticket[batch..2*batch).
int32_t launch_argmax(const float *x, int64_t n, int32_t batch, float *part_val, int32_t *part_idx, uint32_t *ticket,
                      int32_t *out_idx, int32_t *next_tokens, int32_t *positions, int32_t *history, cudaStream_t s,
                      unsigned long long *key_out, int32_t idx_offset) {
  static bool carveout_set = false;
  if (!carveout_set) {
    prefer_max_smem_carveout(argmax_kernel);
    prefer_max_smem_carveout(rope_kv_kernel);
    carveout_set = true;
  }
  dim3 grid(kArgmaxBlocks, (unsigned)batch);
  argmax_kernel<<<grid, kArgmaxThreads, 0, s>>>(x, n, part_val, part_idx, ticket, out_idx, next_tokens, positions, history,
                                                reinterpret_cast<int32_t *>(ticket) + batch, batch, key_out, idx_offset);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// ------------------------------------------------------------------ helpers of the sharded step

__global__ void residual_add_kernel(float *__restrict__ h, const float *__restrict__ delta, int64_t n) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    h[i] = __fadd_rn(h[i], delta[i]);
}

int32_t launch_residual_add(float *h, const float *delta, int64_t n, bool pdl, cudaStream_t s) {
  (void)pdl;  // follows a collective: ordinary stream order
  residual_add_kernel<<<(unsigned)std::min<int64_t>((n + 255) / 256, 1024), 256, 0, s>>>(h, delta, n);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// After the all-reduce(max) of the packed keys: token = inverted low word; feed it back.
__global__ void argmax_finish_kernel(const unsigned long long *__restrict__ keys, int32_t batch, int32_t *out_idx,
                                     int32_t *next_tokens, int32_t *positions, int32_t *history, int32_t *hist_len) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int i = (int)(0xffffffffu - (uint32_t)(keys[b] & 0xffffffffull));
  out_idx[b] = i;
  if (next_tokens) {
    next_tokens[b] = i;
    positions[b] += 1;
    const int step = hist_len[b];
    history[(int64_t)step * batch + b] = i;
    hist_len[b] = step + 1;
  }
}

int32_t launch_argmax_finish(const unsigned long long *keys, int32_t batch, int32_t *out_idx, int32_t *next_tokens,
                             int32_t *positions, int32_t *history, uint32_t *ticket_base, cudaStream_t s) {
  argmax_finish_kernel<<<(batch + 63) / 64, 64, 0, s>>>(keys, batch, out_idx, next_tokens, positions, history,
                                                        reinterpret_cast<int32_t *>(ticket_base) + batch);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// all-gather output [rank][batch][per_rank] -> [batch][rank * per_rank]
__global__ void gather_permute_kernel(const float *__restrict__ g, float *__restrict__ out, int ranks, int batch, int64_t per_rank) {
  const int64_t total = (int64_t)ranks * batch * per_rank;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / (batch * per_rank), rem = i % (batch * per_rank);
    const int64_t b = rem / per_rank, v = rem % per_rank;
    out[(b * ranks + r) * per_rank + v] = g[i];
  }
}

int32_t launch_gather_permute(const float *gathered, float *out, int32_t ranks, int32_t batch, int64_t per_rank, cudaStream_t s) {
  const int64_t total = (int64_t)ranks * batch * per_rank;
  gather_permute_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 2048), 256, 0, s>>>(gathered, out, ranks, batch, per_rank);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld

// ------------------------------------------------------------------ stand-alone receive of a peer sum
namespace cmld {

// h[b][c] = sum over ranks (in rank order) of the partial rows in the local slot, once every rank's
// arrival word has reached the expected count.  The same arithmetic as the matvec kernel's
// receiving prologue, for a step that ends on a sublayer instead of feeding another matvec.
__global__ void peer_reduce_kernel(const GemvPeer rx, int32_t batch, int32_t hidden, int32_t *status) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if ((int)threadIdx.x < rx.rx_n) peer_wait(rx.rx_flag + threadIdx.x, __ldcg(rx.rx_epoch), rx.timeout_ns, status);
  __syncthreads();
  const int64_t rank_stride = (int64_t)kPeerRows * hidden;
  const int64_t n4 = (int64_t)batch * hidden / 4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 s = __ldcg(reinterpret_cast<const float4 *>(rx.rx_part) + i);
    for (int r = 1; r < rx.rx_n; ++r) {
      const float4 t = __ldcg(reinterpret_cast<const float4 *>(rx.rx_part + r * rank_stride) + i);
      s.x = __fadd_rn(s.x, t.x), s.y = __fadd_rn(s.y, t.y), s.z = __fadd_rn(s.z, t.z), s.w = __fadd_rn(s.w, t.w);
    }
    reinterpret_cast<float4 *>(rx.rx_out)[i] = s;
  }
}

int32_t launch_peer_reduce(const GemvPeer &rx, int32_t batch, int32_t hidden, int32_t *status, bool pdl, cudaStream_t s) {
  if (rx.rx_n < 1 || !rx.rx_out || !status || hidden % 4) return fail(CMLD_ERR_INVALID, "peer_reduce: bad arguments");
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)std::min<int64_t>(((int64_t)batch * hidden / 4 + 255) / 256, 64));
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, peer_reduce_kernel, rx, batch, hidden, status));
  return CMLD_OK;
}


// ---------------------------------------------------------------- self-test of the exact sum

// out[0] = the sum of n non-negative terms by xsum::cta_sum; out[1] = the same event list walked again with the check
// in front of every step and every second run forced to fail it (replayed term by term).  Both must be the
// sequential sum's bits.
__global__ void __launch_bounds__(kNormThreads) exact_sum_selftest_kernel(const float *terms, int n, float *out) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  float *sq = reinterpret_cast<float *>(dyn_smem);
  uint8_t *ws = dyn_smem + (size_t)n * 4;
  for (int i = threadIdx.x; i < n; i += kNormThreads) sq[i] = terms[i];
  const float s = xsum::cta_sum<kNormThreads / 32>(sq, n, threadIdx.x >> 5, threadIdx.x & 31, 1, ws);
  if (threadIdx.x == 0) {
    out[0] = s;
    out[1] = xsum::rewalk_with_forced_replays(sq, n, ws);
  }
}

int32_t launch_exact_sum_selftest(const float *terms, int32_t n, float *out, cudaStream_t s) {
  if (n <= 0 || n % 256 || n > kNormMaxExact) return fail(CMLD_ERR_SHAPE, "exact sum self-test: n must be a multiple of 256, at most %d", kNormMaxExact);
  const size_t smem = (size_t)n * 4 + xsum::workspace_bytes(n);
  static bool configured = false;
  if (!configured) {
    CMLD_CUDA(cudaFuncSetAttribute(exact_sum_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kNormMaxExact * 4 + xsum::workspace_bytes(kNormMaxExact)));
    configured = true;
  }
  exact_sum_selftest_kernel<<<1, kNormThreads, smem, s>>>(terms, n, out);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
