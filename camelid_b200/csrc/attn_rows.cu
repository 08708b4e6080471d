// Reference-order attention for steps of several rows (batched decode, prompt chunks): one CTA per (row, KV head)
// serving all G query heads of the group, so that 32 rows x 8 KV heads fill the machine with independent CTAs
// instead of queueing clusters of eight.  The same f32 operations in the same order as the one-row kernels
// (attention_context_for_head, src/inference.rs:30287-30466):
//   score_p  = (sum over d, in order, of q_d * k_pd) * scale          one thread per (position, head), K tiles staged
//                                                                     with cp.async (row pitch 272 B: the eight
//                                                                     positions of a warp fall on distinct banks, the
//                                                                     G heads of a position share the row)
//   e_p      = expf(score_p - max)                                    glibc's expf restated
//   sum      = e_0 + e_1 + ... in position order                      one thread per head
//   w_p      = e_p * (1 / sum)
//   out_d    = ((0 + w_0 * v_0d) + w_1 * v_1d) + ...                   one thread per (head, d), V tiles staged likewise
// q is already rotated and the step's K/V rows are already in the cache (the RoPE + append kernel ran before).
#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

namespace {

constexpr int kRowsThreads = 512;
constexpr int kRowsTile = 128;  // positions per staged tile

__device__ __forceinline__ void rows_cp16(void *dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int G, int HD>
__global__ void __launch_bounds__(kRowsThreads) attn_rows_kernel(AttnArgs a, int cap) {
  extern __shared__ __align__(16) uint8_t rows_smem[];
  constexpr int PITCH = HD * 2 + 16;  // bytes between staged rows
  constexpr int QP = HD + 4;          // floats between the heads' query rows
  float *q_s = reinterpret_cast<float *>(rows_smem);                      // [G][QP]
  float *sc = q_s + G * QP;                                               // [G][cap]
  uint8_t *tiles = reinterpret_cast<uint8_t *>(sc + (int64_t)G * cap);    // [2][kRowsTile][PITCH]
  __shared__ float s_red[G][kRowsThreads / 32];
  __shared__ float s_head[G][2];  // maximum, 1 / sum
  const int kvh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_pos = a.positions[b] + 1, slot = a.slots[b];
  const __half *kbase = a.k_cache + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const __half *vbase = a.v_cache + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  for (int i = tid; i < G * HD; i += kRowsThreads) q_s[(i / HD) * QP + i % HD] = q[i];
  const int n_tiles = (n_pos + kRowsTile - 1) / kRowsTile;
  auto stage = [&](const __half *base, int t) {
    if (t < n_tiles) {
      const int p0 = t * kRowsTile, cnt = min(kRowsTile, n_pos - p0);
      uint8_t *dst = tiles + (t & 1) * (kRowsTile * PITCH);
      for (int c = tid; c < cnt * (HD / 8); c += kRowsThreads) {
        const int p = c / (HD / 8), j = c % (HD / 8);
        rows_cp16(dst + p * PITCH + j * 16, reinterpret_cast<const uint8_t *>(base + (int64_t)(p0 + p) * HD) + j * 16);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // ---- scores
  stage(kbase, 0);
  for (int t = 0; t < n_tiles; ++t) {
    stage(kbase, t + 1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();  // tile t (and, the first time, q) visible to all
    const int p0 = t * kRowsTile, cnt = min(kRowsTile, n_pos - p0);
    const uint8_t *tile = tiles + (t & 1) * (kRowsTile * PITCH);
    for (int u = tid; u < cnt * G; u += kRowsThreads) {
      const int p = u / G, g = u % G;  // the heads of a position sit in neighbouring lanes and share its row
      const uint8_t *kr = tile + p * PITCH;
      const float *qg = q_s + g * QP;
      float s = 0.0f;
#pragma unroll 4
      for (int j = 0; j < HD / 8; ++j) {
        const uint4 kw = *reinterpret_cast<const uint4 *>(kr + j * 16);
        const float4 q0 = *reinterpret_cast<const float4 *>(qg + 8 * j), q1 = *reinterpret_cast<const float4 *>(qg + 8 * j + 4);
        const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.x)), k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.y));
        const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.z)), k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.w));
        s = __fadd_rn(s, __fmul_rn(q0.x, k0.x));
        s = __fadd_rn(s, __fmul_rn(q0.y, k0.y));
        s = __fadd_rn(s, __fmul_rn(q0.z, k1.x));
        s = __fadd_rn(s, __fmul_rn(q0.w, k1.y));
        s = __fadd_rn(s, __fmul_rn(q1.x, k2.x));
        s = __fadd_rn(s, __fmul_rn(q1.y, k2.y));
        s = __fadd_rn(s, __fmul_rn(q1.z, k3.x));
        s = __fadd_rn(s, __fmul_rn(q1.w, k3.y));
      }
      sc[(int64_t)g * cap + p0 + p] = __fmul_rn(s, a.scale);
    }
    __syncthreads();  // everybody is done with tile t before the copy of tile t + 2 overwrites it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  stage(vbase, 0);  // the first value tile travels while the softmax is formed
  // ---- maxima (any order), exponentials, sums in position order, weights
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float m = -INFINITY;
    for (int p = tid; p < n_pos; p += kRowsThreads) m = fmaxf(m, sc[(int64_t)g * cap + p]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[g][warp] = m;
  }
  __syncthreads();
  if (tid < G) {
    float m = s_red[tid][0];
    for (int w = 1; w < kRowsThreads / 32; ++w) m = fmaxf(m, s_red[tid][w]);
    s_head[tid][0] = m;
  }
  __syncthreads();
  for (int i = tid; i < G * n_pos; i += kRowsThreads) {
    const int g = i / n_pos, p = i % n_pos;
    sc[(int64_t)g * cap + p] = expf_exact(__fsub_rn(sc[(int64_t)g * cap + p], s_head[g][0]));
  }
  __syncthreads();
  if (tid < G) {
    const float *e = sc + (int64_t)tid * cap;
    float sum = 0.0f;
    int p = 0;
    for (; p + 4 <= n_pos; p += 4) {
      const float4 e4 = *reinterpret_cast<const float4 *>(e + p);
      sum = __fadd_rn(sum, e4.x);
      sum = __fadd_rn(sum, e4.y);
      sum = __fadd_rn(sum, e4.z);
      sum = __fadd_rn(sum, e4.w);
    }
    for (; p < n_pos; ++p) sum = __fadd_rn(sum, e[p]);
    s_head[tid][1] = __fdiv_rn(1.0f, sum);
  }
  __syncthreads();
  for (int i = tid; i < G * n_pos; i += kRowsThreads) {
    const int g = i / n_pos, p = i % n_pos;
    sc[(int64_t)g * cap + p] = __fmul_rn(sc[(int64_t)g * cap + p], s_head[g][1]);
  }
  // ---- weighted values: a thread per (head, dimension) walks the positions
  float acc[(G * HD + kRowsThreads - 1) / kRowsThreads];
#pragma unroll
  for (int k = 0; k < (G * HD + kRowsThreads - 1) / kRowsThreads; ++k) acc[k] = 0.0f;
  for (int t = 0; t < n_tiles; ++t) {
    stage(vbase, t + 1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();  // tile t and (the first time) the weights visible to all
    const int p0 = t * kRowsTile, cnt = min(kRowsTile, n_pos - p0);
    const uint8_t *tile = tiles + (t & 1) * (kRowsTile * PITCH);
#pragma unroll
    for (int k = 0; k < (G * HD + kRowsThreads - 1) / kRowsThreads; ++k) {
      const int c = tid + k * kRowsThreads;
      if (c < G * HD) {
        const int g = c / HD, d = c % HD;
        const float *w = sc + (int64_t)g * cap + p0;
        const uint8_t *vcol = tile + d * 2;
        float o = acc[k];
        int p = 0;
        for (; p + 4 <= cnt; p += 4) {
          const float4 w4 = *reinterpret_cast<const float4 *>(w + p);
          o = __fadd_rn(o, __fmul_rn(w4.x, __half2float(*reinterpret_cast<const __half *>(vcol + (p + 0) * PITCH))));
          o = __fadd_rn(o, __fmul_rn(w4.y, __half2float(*reinterpret_cast<const __half *>(vcol + (p + 1) * PITCH))));
          o = __fadd_rn(o, __fmul_rn(w4.z, __half2float(*reinterpret_cast<const __half *>(vcol + (p + 2) * PITCH))));
          o = __fadd_rn(o, __fmul_rn(w4.w, __half2float(*reinterpret_cast<const __half *>(vcol + (p + 3) * PITCH))));
        }
        for (; p < cnt; ++p) o = __fadd_rn(o, __fmul_rn(w[p], __half2float(*reinterpret_cast<const __half *>(vcol + p * PITCH))));
        acc[k] = o;
      }
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  float *out = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
#pragma unroll
  for (int k = 0; k < (G * HD + kRowsThreads - 1) / kRowsThreads; ++k) {
    const int c = tid + k * kRowsThreads;
    if (c < G * HD) out[c] = acc[k];
  }
}

size_t rows_smem_bytes(int G, int HD, int cap) { return (size_t)G * (HD + 4) * 4 + (size_t)G * cap * 4 + 2 * (size_t)kRowsTile * (HD * 2 + 16); }

template <int G, int HD>
int32_t launch_rows(const AttnArgs &a, int cap, cudaStream_t s) {
  const size_t smem = rows_smem_bytes(G, HD, cap);
  static size_t configured = 0;
  if (smem > configured) {
    CMLD_CUDA(cudaFuncSetAttribute(attn_rows_kernel<G, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid((unsigned)a.n_kv_heads, (unsigned)a.batch);
  attn_rows_kernel<G, HD><<<grid, kRowsThreads, smem, s>>>(a, cap);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace

// cap: bound on positions[b] + 1 of every row of the step, a multiple of 4.
bool attention_rows_fits(int n_heads, int n_kv_heads, int head_dim, int64_t cap) {
  if (n_kv_heads < 1 || n_heads % n_kv_heads) return false;
  const int G = n_heads / n_kv_heads;
  if (!(G == 1 || G == 2 || G == 3 || G == 4 || G == 8) || !(head_dim == 64 || head_dim == 128)) return false;
  return cap > 0 && cap % 4 == 0 && rows_smem_bytes(G, head_dim, (int)cap) <= 200 * 1024;
}

int32_t launch_attention_rows(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  if (!attention_rows_fits(a.n_heads, a.n_kv_heads, a.head_dim, cap)) return CMLD_ERR_UNSUPPORTED;
  if (a.tree_mask || a.fuse_rope) return fail(CMLD_ERR_INVALID, "attention (rows): tree masks and fused RoPE are not supported here");
  const int G = a.n_heads / a.n_kv_heads, c = (int)cap;
#define CMLD_ROWS(GG)                                                                      \
  case GG: return a.head_dim == 128 ? launch_rows<GG, 128>(a, c, s) : launch_rows<GG, 64>(a, c, s);
  switch (G) {
    CMLD_ROWS(1)
    CMLD_ROWS(2)
    CMLD_ROWS(3)
    CMLD_ROWS(4)
    CMLD_ROWS(8)
  }
#undef CMLD_ROWS
  return CMLD_ERR_UNSUPPORTED;
}

}  // namespace cmld
