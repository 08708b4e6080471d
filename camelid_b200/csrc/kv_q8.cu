// KV cache held as Q8_0 blocks (kv_scatter_q8_0 / attention_decode_q8_0 of the reference's CUDA lane,
// src/cuda_resident.rs:5366-5480; the arithmetic is that of its CPU lane, src/tensor/kv_quant.rs): per 32 values
// of a head one f16 scale d = amax/127 and 32 int8 codes (34 bytes), half the bytes of the f16 cache.
//
//   append : RoPE(q) in place; RoPE(k) and v quantised block by block — one warp per block, a lane per value, the
//            block maximum by shuffles (a maximum does not depend on the order) — and stored at the row's position.
//   attend : one CTA per (query head, row).  score_p = (sum over blocks of (sum_i q_i*code_i) * d) * scale with the
//            inner sums in index order (vec_dot_row_q8_0, scalar form); softmax as the f16 path (maximum, exp, sum in
//            position order); out_i = fma(prob_p * d, code_i, out_i) position after position (axpy_row_q8_0).
// Cache layout per layer: [slot][kv_head][max_pos][head_dim/32] blocks of {u16 scale, i8 codes[32]}.
#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

namespace {

constexpr int kQ8Block = 34;

__global__ void __launch_bounds__(256) rope_kv_q8_kernel(RopeKvArgs a, uint8_t *kq, uint8_t *vq) {
  const int b = blockIdx.y;
  const int half = a.rope_dim / 2, hd = a.head_dim, nb = hd / 32;
  const int pos = a.positions[b], slot = a.slots[b];
  if (pos < 0 || pos >= a.max_pos) return;
  const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
  const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
  float *q = a.q + (int64_t)b * a.q_stride;
  const float *k = a.k + (int64_t)b * a.kv_stride, *v = a.v + (int64_t)b * a.kv_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = 2 * a.n_kv_heads * nb;  // K blocks, then V blocks
  for (int u = blockIdx.x * 8 + warp; u < n_units; u += gridDim.x * 8) {
    const bool is_v = u >= a.n_kv_heads * nb;
    const int j = is_v ? u - a.n_kv_heads * nb : u, h = j / nb, blk = j % nb, d = blk * 32 + lane;
    float x;
    if (is_v) {
      x = v[h * hd + d];
    } else if (d >= a.rope_dim) {
      x = k[h * hd + d];
    } else {
      // apply_rope_to_row (src/inference/rope.rs:495-530): x0' = x0*c - x1*s, x1' = x0*s + x1*c
      int p, d0, d1;
      bool first;
      if (a.split_half) {
        first = d < half;
        p = first ? d : d - half;
        d0 = p, d1 = p + half;
      } else {
        first = (d & 1) == 0;
        p = d >> 1;
        d0 = 2 * p, d1 = 2 * p + 1;
      }
      const float x0 = k[h * hd + d0], x1 = k[h * hd + d1], c = ct[p], s = st[p];
      x = first ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    // quantize_block_q8_0 (src/tensor/kv_quant.rs:123-143)
    float amax = fabsf(x);
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float dd = __fdiv_rn(amax, 127.0f), id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
    const float r = fminf(fmaxf(roundf(__fmul_rn(x, id)), -127.0f), 127.0f);
    uint8_t *dst = (is_v ? vq : kq) + ((((int64_t)slot * a.n_kv_heads + h) * a.max_pos + pos) * nb + blk) * kQ8Block;
    if (lane == 0) *reinterpret_cast<uint16_t *>(dst) = f32_to_f16_bits(dd);
    dst[2 + lane] = (uint8_t)(int8_t)r;
  }
  // RoPE(q) in place, by the threads of the first CTAs of the row
  const int n_qp = a.n_heads * half;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_qp; i += gridDim.x * blockDim.x) {
    const int h = i / half, p = i % half;
    const int d0 = a.split_half ? p : 2 * p, d1 = a.split_half ? p + half : 2 * p + 1;
    const float c = ct[p], s = st[p], x0 = q[h * hd + d0], x1 = q[h * hd + d1];
    q[h * hd + d0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    q[h * hd + d1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
  }
}

constexpr int kQ8AttnThreads = 256;

__global__ void __launch_bounds__(kQ8AttnThreads) attn_q8_kernel(AttnArgs a, const uint8_t *kq, const uint8_t *vq) {
  extern __shared__ float s_sc[];  // [n_pos] scores, then exponentials
  __shared__ float s_q[128];
  __shared__ float s_red[kQ8AttnThreads / 32];
  __shared__ float s_bcast[2];
  const int head = blockIdx.x, b = blockIdx.y, hd = a.head_dim, nb = hd / 32;
  const int n_pos = a.positions[b] + 1, slot = a.slots[b];
  const int kvh = head / (a.n_heads / a.n_kv_heads);
  const uint8_t *kbase = kq + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * nb * kQ8Block;
  const uint8_t *vbase = vq + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * nb * kQ8Block;
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) s_q[d] = q[d];
  __syncthreads();
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x) {
    const uint8_t *row = kbase + (int64_t)p * nb * kQ8Block;
    float total = 0.0f;
    for (int blk = 0; blk < nb; ++blk) {
      const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(row + blk * kQ8Block));
      const int8_t *codes = reinterpret_cast<const int8_t *>(row + blk * kQ8Block + 2);
      float sum = 0.0f;
      for (int i = 0; i < 32; ++i) sum = __fadd_rn(sum, __fmul_rn(s_q[blk * 32 + i], (float)codes[i]));
      total = __fadd_rn(total, __fmul_rn(sum, d));
    }
    s_sc[p] = __fmul_rn(total, a.scale);
  }
  __syncthreads();
  float m = -INFINITY;
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x) m = fmaxf(m, s_sc[p]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = s_red[0];
    for (int w = 1; w < kQ8AttnThreads / 32; ++w) mm = fmaxf(mm, s_red[w]);
    s_bcast[0] = mm;
  }
  __syncthreads();
  m = s_bcast[0];
  for (int p = threadIdx.x; p < n_pos; p += blockDim.x) s_sc[p] = expf_exact(__fsub_rn(s_sc[p], m));
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.0f;
    for (int p = 0; p < n_pos; ++p) sum = __fadd_rn(sum, s_sc[p]);
    s_bcast[1] = __fdiv_rn(1.0f, sum);
  }
  __syncthreads();
  const float inv = s_bcast[1];
  float *out = a.out + (int64_t)b * a.q_stride + (int64_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    const int blk = d >> 5, i = d & 31;
    float o = 0.0f;
    for (int p = 0; p < n_pos; ++p) {
      const uint8_t *blkp = vbase + ((int64_t)p * nb + blk) * kQ8Block;
      const float dv = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blkp));
      o = __fmaf_rn(__fmul_rn(__fmul_rn(s_sc[p], inv), dv), (float)reinterpret_cast<const int8_t *>(blkp + 2)[i], o);
    }
    out[d] = o;
  }
}

// f32 rows [kv_head][n_pos][hd] <-> blocks, slot 0 (seed_layer / read_kv_layer)
__global__ void kv_q8_convert_kernel(uint8_t *cache, float *host_layout, int n_kv, int64_t max_pos, int64_t n_pos, int hd, bool to_cache) {
  const int nb = hd / 32, lane = threadIdx.x & 31;
  const int64_t n_blocks = (int64_t)n_kv * n_pos * nb;
  for (int64_t u = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); u < n_blocks; u += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t kh = u / (n_pos * nb), rem = u % (n_pos * nb), p = rem / nb, blk = rem % nb;
    uint8_t *dst = cache + ((kh * max_pos + p) * nb + blk) * kQ8Block;
    float *f = host_layout + (kh * n_pos + p) * hd + blk * 32 + lane;
    if (to_cache) {
      const float x = *f;
      float amax = fabsf(x);
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float dd = __fdiv_rn(amax, 127.0f), id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
      if (lane == 0) *reinterpret_cast<uint16_t *>(dst) = f32_to_f16_bits(dd);
      dst[2 + lane] = (uint8_t)(int8_t)fminf(fmaxf(roundf(__fmul_rn(x, id)), -127.0f), 127.0f);
    } else {
      // dequantize_block_q8_0 (:145-151): code * d
      *f = __fmul_rn((float)reinterpret_cast<const int8_t *>(dst + 2)[lane], f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(dst)));
    }
  }
}

}  // namespace

int64_t kv_q8_layer_bytes(int64_t seqs, int n_kv, int64_t max_pos, int hd) { return seqs * n_kv * max_pos * (hd / 32) * kQ8Block; }

int32_t launch_rope_kv_q8(const RopeKvArgs &a, uint8_t *kq, uint8_t *vq, cudaStream_t s) {
  if (a.head_dim % 32) return fail(CMLD_ERR_SHAPE, "Q8_0 KV cache: head_dim %d is not a multiple of 32", a.head_dim);
  const int units = 2 * a.n_kv_heads * (a.head_dim / 32);
  dim3 grid((unsigned)std::max(1, (units + 7) / 8), (unsigned)a.batch);
  rope_kv_q8_kernel<<<grid, 256, 0, s>>>(a, kq, vq);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t launch_attention_q8(const AttnArgs &a, const uint8_t *kq, const uint8_t *vq, cudaStream_t s) {
  if (a.head_dim > 128 || a.head_dim % 32) return fail(CMLD_ERR_SHAPE, "Q8_0 KV attention: head_dim %d", a.head_dim);
  if (a.tree_mask) return fail(CMLD_ERR_UNSUPPORTED, "tree verification over a Q8_0 KV cache is not supported");
  const size_t smem = (size_t)a.max_pos * 4;
  static size_t configured = 0;
  if (smem > 200 * 1024) return fail(CMLD_ERR_SHAPE, "Q8_0 KV attention: max_pos %lld too large", (long long)a.max_pos);
  if (smem > 48 * 1024 && smem > configured) {
    CMLD_CUDA(cudaFuncSetAttribute(attn_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid((unsigned)a.n_heads, (unsigned)a.batch);
  attn_q8_kernel<<<grid, kQ8AttnThreads, smem, s>>>(a, kq, vq);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t launch_kv_q8_convert(uint8_t *cache, float *rows, int n_kv, int64_t max_pos, int64_t n_pos, int hd, bool to_cache, cudaStream_t s) {
  const int64_t n_blocks = (int64_t)n_kv * n_pos * (hd / 32);
  const unsigned blocks = (unsigned)std::min<int64_t>((n_blocks + 7) / 8, 4096);
  kv_q8_convert_kernel<<<std::max(1u, blocks), 256, 0, s>>>(cache, rows, n_kv, max_pos, n_pos, hd, to_cache);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
