// Single-query grouped-query attention over the f16 KV cache with every f32 operation in the order of
// Camelid's CPU path (attention_context_for_head_into_with_kernels, src/inference.rs:30287-30466 with
// dot_product, src/tensor/mod.rs:3464-3480, in the Camelid tree), so the output has the CPU's bits:
//
//   score_p = (((0 + q0*k0) + q1*k1) + ...) * scale          one accumulator over the head dimension
//   m = max_p score_p;  e_p = expf(score_p - m);  S = ((e_0 + e_1) + ...)   one accumulator over positions
//   out_d = ((0 + (e_0/S)*v_0d) + (e_1/S)*v_1d) + ...        one accumulator over positions, per d
//
// The dependent chains are what they are — 4 cycles per addition — so the kernel is organised around
// having as many of them in flight as the arithmetic allows and nothing else on the critical path:
//   * one thread-block cluster of 8 CTAs per (sequence, kv head), serving the G query heads of the group;
//   * scores: positions are cut into 8 ranges, one per CTA; a thread owns one (position, head) chain over the
//     head dimension; K rows are staged by cp.async into shared memory at a bank-conflict-free pitch;
//   * softmax: range maxima meet through distributed shared memory; e_p is written straight into the
//     shared memory of the CTAs that need it; the sum over positions is a sequential f32 sum of non-negative
//     terms, computed with its exact bits by all warps of one CTA per head (exact_sum.cuh);
//   * output: the G*head_dim chains over positions are spread evenly over the 8 CTAs; a warp walks 32 of
//     them with the V slice it needs streamed through a private cp.async ring that was started when the
//     kernel began, so V arrives while the scores are still being computed.
// RoPE of q and k and the f16 KV append can be folded in (fuse_rope), as in the split-range kernel.
#include <cooperative_groups.h>

#include "common.cuh"
#include "exact_sum.cuh"
#include "expf_exact.cuh"

namespace cmld {

namespace cg = cooperative_groups;

constexpr int kOaThreads = 256;
constexpr int kOaWarps = kOaThreads / 32;
constexpr int kOaCluster = 8;
constexpr int kOaKBlock = 64;   // positions per staged K block
constexpr int kOaVChunk = 64;   // positions per V ring slot
constexpr int kOaVDepth = 8;    // ring slots per chain warp
constexpr int kOaVSlot = kOaVChunk * 64;  // bytes: 32 dims x f16 per position

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// RoPE pair partner and sign: x'[d] = x[d]*c + sgn * x[partner]*s  (src/inference/rope.rs:495-530)
__device__ __forceinline__ float oa_rope_elem(const float *x, int d, int rope_dim, int split_half, const float *ct, const float *st) {
  if (d >= rope_dim) return x[d];
  const int half = rope_dim >> 1;
  int p, partner;
  bool first;
  if (split_half) {
    first = d < half;
    p = first ? d : d - half;
    partner = first ? d + half : d - half;
  } else {
    first = (d & 1) == 0;
    p = d >> 1;
    partner = first ? d + 1 : d - 1;
  }
  const float c = ct[p], sn = st[p];
  return first ? __fsub_rn(__fmul_rn(x[d], c), __fmul_rn(x[partner], sn)) : __fadd_rn(__fmul_rn(x[partner], sn), __fmul_rn(x[d], c));
}

struct OaLayout {
  int cap_range;   // positions a CTA's range can hold
  int cap_pad;     // positions per weight array (multiple of 256)
  int n_warr;      // weight arrays per CTA (heads its chains touch)
  int off_q, off_k, off_klast, off_sc, off_w, off_ws, off_mx, off_inv, off_v, total;
};

__host__ __device__ inline OaLayout oa_layout(int G, int HD, int64_t cap) {
  OaLayout L;
  const int cpc = G * HD / kOaCluster;
  L.cap_range = (int)((cap + kOaCluster - 1) / kOaCluster);
  L.cap_pad = (int)((cap + 255) / 256 * 256);
  L.n_warr = (HD % cpc == 0) ? 1 : 2;
  int off = 0;
  L.off_q = off;
  off += G * HD * 4;
  L.off_k = off;
  off += 2 * kOaKBlock * (HD * 2 + 16);
  L.off_klast = off;
  off += HD * 2;
  L.off_sc = off;
  off += G * L.cap_range * 4;
  off = (off + 15) & ~15;
  L.off_w = off;
  off += L.n_warr * L.cap_pad * 4;
  L.off_ws = off;
  off += (L.cap_pad >> 8) * 16 + (L.cap_pad >> 3) * 8 + 16;
  L.off_mx = off;
  off += kOaCluster * 8 * 4;
  L.off_inv = off;
  off += 16;
  off = (off + 127) & ~127;
  L.off_v = off;
  off += ((cpc + 31) / 32) * kOaVDepth * kOaVSlot;
  L.total = off;
  return L;
}

template <int G, int HD>
__global__ void __launch_bounds__(kOaThreads, 1) attn_ordered_kernel(AttnArgs a, int64_t cap) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int CPC = G * HD / kOaCluster;   // chains of this CTA (consecutive (head, d) pairs of the kv group)
  constexpr int NCW = (CPC + 31) / 32;       // warps that walk chains
  constexpr int KP = HD * 2 + 16;            // K row pitch in shared memory
  const OaLayout L = oa_layout(G, HD, cap);
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = a.positions[b];
  const int n_pos = pos + 1;
  const int slot = a.slots[b];
  if (pos < 0 || pos >= a.max_pos || n_pos > cap) return;  // the same for every CTA of the cluster
  float(*s_q)[HD] = reinterpret_cast<float(*)[HD]>(smem + L.off_q);
  uint8_t *s_k = smem + L.off_k;
  __half *s_klast = reinterpret_cast<__half *>(smem + L.off_klast);
  float *s_sc = reinterpret_cast<float *>(smem + L.off_sc);   // [G][cap_range]
  float *s_w = reinterpret_cast<float *>(smem + L.off_w);     // [n_warr][cap_pad]
  uint8_t *s_ws = smem + L.off_ws;
  float *s_mx = reinterpret_cast<float *>(smem + L.off_mx);   // [cluster rank][8]
  float *s_inv = reinterpret_cast<float *>(smem + L.off_inv); // [n_warr] (+ one scratch float)
  uint8_t *s_v = smem + L.off_v;

  __half *kbase = const_cast<__half *>(a.k_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  __half *vbase = const_cast<__half *>(a.v_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const int n_pre = a.fuse_rope ? n_pos - 1 : n_pos;  // positions whose K/V rows are already in the cache

  // ---- chain bookkeeping: this CTA's chains are flat indices [c0, c0 + CPC) of (head, d) within the kv group
  const int c0 = crank * CPC;
  const int g_first = c0 / HD;  // first head this CTA's chains belong to

  // ---- V ring of the chain warps: start it now
  const int ch_start = c0 + warp * 32;  // first chain of this warp
  uint8_t *vring = s_v + warp * kOaVDepth * kOaVSlot;
  const int n_vchunks = (n_pre + kOaVChunk - 1) / kOaVChunk;
  auto issue_v = [&](int chunk) {
    if (chunk < n_vchunks) {
      uint8_t *dst = vring + (chunk % kOaVDepth) * kOaVSlot;
      const int gran = ((ch_start >> 3) + (lane & 3)) % (HD / 8);  // which 8 dims of the row this lane copies
#pragma unroll
      for (int i = 0; i < kOaVChunk / 8; ++i) {
        const int pp = (lane >> 2) + 8 * i, p = chunk * kOaVChunk + pp;
        if (p < n_pre) cp_async16(dst + pp * 64 + (lane & 3) * 16, vbase + (int64_t)p * HD + gran * 8);
      }
    }
    cp_async_commit();
  };
  if (warp < NCW) {
    for (int c = 0; c < kOaVDepth; ++c) issue_v(c);
  }

  // ---- q (rotated), and the row's own K/V: appended to the cache, K kept for the scores
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  // ranges: CTA r scores positions [r*len, (r+1)*len)
  const int len = (n_pos + kOaCluster - 1) / kOaCluster;
  const int lo = crank * len, hi = min(n_pos, lo + len);
  if (a.fuse_rope) {
    const int half = a.rope_dim >> 1;
    const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    for (int i = tid; i < G * HD; i += kOaThreads) s_q[i / HD][i % HD] = oa_rope_elem(q + (i / HD) * HD, i % HD, a.rope_dim, a.split_half, ct, st);
    if (pos >= lo && pos < hi) {
      const float *kn = a.k_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      const float *vn = a.v_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      for (int d = tid; d < HD; d += kOaThreads) {
        const __half kh = __float2half_rn(oa_rope_elem(kn, d, a.rope_dim, a.split_half, ct, st));
        s_klast[d] = kh;
        kbase[(int64_t)pos * HD + d] = kh;
        vbase[(int64_t)pos * HD + d] = __float2half_rn(vn[d]);
      }
    }
  } else {
    for (int i = tid; i < G * HD; i += kOaThreads) s_q[i / HD][i % HD] = q[i];
  }

  // ---- scores of this CTA's range, K staged block by block
  const int n_blocks = (hi - lo + kOaKBlock - 1) / kOaKBlock;
  auto issue_k = [&](int blk) {
    if (blk < n_blocks) {
      uint8_t *dst = s_k + (blk & 1) * kOaKBlock * KP;
      for (int i = tid; i < kOaKBlock * (HD / 8); i += kOaThreads) {
        const int pp = i / (HD / 8), gdx = i % (HD / 8), p = lo + blk * kOaKBlock + pp;
        if (p < hi && p < n_pre) cp_async16(dst + pp * KP + gdx * 16, kbase + (int64_t)p * HD + gdx * 8);
      }
    }
    cp_async_commit();
  };
  issue_k(0);
  for (int blk = 0; blk < n_blocks; ++blk) {
    issue_k(blk + 1);
    cp_async_wait<1>();
    __syncthreads();  // block blk has landed for everyone (the first pass also publishes s_q and s_klast)
    const uint8_t *kb = s_k + (blk & 1) * kOaKBlock * KP;
    for (int pair = tid; pair < kOaKBlock * G; pair += kOaThreads) {
      const int pp = pair % kOaKBlock, g = pair / kOaKBlock, p = lo + blk * kOaKBlock + pp;
      if (p < hi) {
        const uint4 *kr = p < n_pre ? reinterpret_cast<const uint4 *>(kb + pp * KP) : reinterpret_cast<const uint4 *>(s_klast);
        float s = 0.0f;
#pragma unroll 4
        for (int j = 0; j < HD / 8; ++j) {
          const uint4 raw = kr[j];
          const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
          const float4 qa = *reinterpret_cast<const float4 *>(&s_q[g][8 * j]), qb = *reinterpret_cast<const float4 *>(&s_q[g][8 * j + 4]);
          const float2 k0 = __half22float2(h2[0]), k1 = __half22float2(h2[1]), k2 = __half22float2(h2[2]), k3 = __half22float2(h2[3]);
          s = __fadd_rn(s, __fmul_rn(qa.x, k0.x));
          s = __fadd_rn(s, __fmul_rn(qa.y, k0.y));
          s = __fadd_rn(s, __fmul_rn(qa.z, k1.x));
          s = __fadd_rn(s, __fmul_rn(qa.w, k1.y));
          s = __fadd_rn(s, __fmul_rn(qb.x, k2.x));
          s = __fadd_rn(s, __fmul_rn(qb.y, k2.y));
          s = __fadd_rn(s, __fmul_rn(qb.z, k3.x));
          s = __fadd_rn(s, __fmul_rn(qb.w, k3.y));
        }
        s_sc[g * L.cap_range + (p - lo)] = __fmul_rn(s, a.scale);
      }
    }
    __syncthreads();  // the buffer is refilled two blocks later
  }
  if (n_blocks == 0) __syncthreads();
  cp_async_wait<0>();

  // ---- range maxima to every CTA
  if (warp < G) {
    float m = -INFINITY;
    for (int i = lane; i < hi - lo; i += 32) m = fmaxf(m, s_sc[warp * L.cap_range + i]);
    m = warp_max(m);
    if (lane < kOaCluster) cluster.map_shared_rank(s_mx, lane)[crank * 8 + warp] = m;
  }
  cluster.sync();
  // ---- e_p = expf(score - max) into the CTAs whose chains belong to the head
  for (int i = tid; i < G * (hi - lo); i += kOaThreads) {
    const int g = i / (hi - lo), pi = i % (hi - lo);
    float m = -INFINITY;
#pragma unroll
    for (int r = 0; r < kOaCluster; ++r) m = fmaxf(m, s_mx[r * 8 + g]);
    const float e = expf_exact(__fsub_rn(s_sc[g * L.cap_range + pi], m));
    const int r_lo = (g * HD) / CPC, r_hi = ((g + 1) * HD - 1) / CPC;
    for (int r = r_lo; r <= r_hi; ++r) {
      const int hl = g - (r * CPC) / HD;  // index of head g among the heads of CTA r's chains
      cluster.map_shared_rank(s_w, r)[hl * L.cap_pad + lo + pi] = e;
    }
  }
  cluster.sync();
  // ---- S = e_0 + e_1 + ... in order, by the first CTA that holds the head's weights; 1/S to all that hold them
  {
    int my_head = -1;  // the head whose sum this CTA computes
#pragma unroll
    for (int g = 0; g < G; ++g)
      if ((g * HD) / CPC == crank) my_head = g;
    if (my_head >= 0) {
      float *w = s_w + (my_head - g_first) * L.cap_pad;
      const int n_pad = (n_pos + 255) & ~255;
      for (int i = n_pos + tid; i < n_pad; i += kOaThreads) w[i] = 0.0f;  // adding +0 leaves a sum as it is
      const int nch = n_pad >> 8;
      const float ssum = xsum::cta_sum<kOaWarps>(w, n_pad, warp, lane, 1, reinterpret_cast<double *>(s_ws),
                                                reinterpret_cast<uint32_t *>(s_ws + nch * 8),
                                                reinterpret_cast<xsum::Item *>(s_ws + nch * 16), s_inv + 3);
      if (tid == 0) {
        const float inv = __fdiv_rn(1.0f, ssum);
        const int r_lo = (my_head * HD) / CPC, r_hi = ((my_head + 1) * HD - 1) / CPC;
        for (int r = r_lo; r <= r_hi; ++r) cluster.map_shared_rank(s_inv, r)[my_head - (r * CPC) / HD] = inv;
      }
    }
  }
  cluster.sync();
  // ---- prob_p = e_p * (1/S), in place
  for (int i = tid; i < L.n_warr * n_pos; i += kOaThreads) {
    const int hl = i / n_pos, p = i % n_pos;
    if (g_first + hl < G) s_w[hl * L.cap_pad + p] = __fmul_rn(s_w[hl * L.cap_pad + p], s_inv[hl]);
  }
  __syncthreads();
  // ---- out_d = sum over positions, in order
  if (warp < NCW) {
    const int chain = warp * 32 + lane;  // within this CTA
    const bool valid = chain < CPC;
    const int flat = c0 + (valid ? chain : 0), g = flat / HD, d = flat % HD;
    const float *pr = s_w + (g - g_first) * L.cap_pad;
    float o = 0.0f;
    for (int c = 0; c < n_vchunks; ++c) {
      cp_async_wait<kOaVDepth - 1>();
      __syncwarp();
      const uint8_t *vs = vring + (c % kOaVDepth) * kOaVSlot + 2 * lane;
      const int p0 = c * kOaVChunk, cnt = min(kOaVChunk, n_pre - p0);
      int pp = 0;
      for (; pp + 4 <= cnt; pp += 4) {
        const float4 w4 = *reinterpret_cast<const float4 *>(pr + p0 + pp);
        const float v0 = __half2float(*reinterpret_cast<const __half *>(vs + (pp + 0) * 64));
        const float v1 = __half2float(*reinterpret_cast<const __half *>(vs + (pp + 1) * 64));
        const float v2 = __half2float(*reinterpret_cast<const __half *>(vs + (pp + 2) * 64));
        const float v3 = __half2float(*reinterpret_cast<const __half *>(vs + (pp + 3) * 64));
        o = __fadd_rn(o, __fmul_rn(w4.x, v0));
        o = __fadd_rn(o, __fmul_rn(w4.y, v1));
        o = __fadd_rn(o, __fmul_rn(w4.z, v2));
        o = __fadd_rn(o, __fmul_rn(w4.w, v3));
      }
      for (; pp < cnt; ++pp) o = __fadd_rn(o, __fmul_rn(pr[p0 + pp], __half2float(*reinterpret_cast<const __half *>(vs + pp * 64))));
      __syncwarp();
      issue_v(c + kOaVDepth);
    }
    if (a.fuse_rope) {
      // the row's own V, rounded through f16 as the cache holds it
      const float vn = a.v_new[(int64_t)b * a.kv_stride + (int64_t)kvh * HD + d];
      o = __fadd_rn(o, __fmul_rn(pr[pos], __half2float(__float2half_rn(vn))));
    }
    if (valid) a.out[(int64_t)b * a.q_stride + (int64_t)kvh * G * HD + flat] = o;
  }
  cp_async_wait<0>();
  cluster.sync();  // nobody leaves while its shared memory may still be written or read
}

template <int G, int HD>
static int32_t launch_oa(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  const OaLayout L = oa_layout(G, HD, cap);
  static int configured = 0;
  if (L.total > configured) {
    CMLD_CUDA(cudaFuncSetAttribute(attn_ordered_kernel<G, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
    configured = L.total;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(kOaCluster, (unsigned)a.n_kv_heads, (unsigned)a.batch);
  cfg.blockDim = dim3(kOaThreads);
  cfg.dynamicSmemBytes = (size_t)L.total;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (a.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;
  attr[n_attr].val.clusterDim.x = kOaCluster;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, attn_ordered_kernel<G, HD>, a, cap));
  return CMLD_OK;
}

// Whether the cluster kernel takes this shape with contexts of up to `cap` positions.
bool attention_ordered_fits(int n_heads, int n_kv_heads, int head_dim, int64_t cap) {
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return false;
  const int G = n_heads / n_kv_heads;
  if (!(G == 1 || G == 2 || G == 3 || G == 4 || G == 8)) return false;
  if (!(head_dim == 64 || head_dim == 128)) return false;
  if ((G * head_dim / kOaCluster) % 8) return false;
  if (cap > 8192) return false;  // the exact sum takes at most 32 chunks of 256 terms
  return oa_layout(G, head_dim, cap).total <= 226 * 1024;
}

// Reference-order attention for rows whose contexts are at most `cap` positions long (a.max_pos bounds the cache rows).
int32_t launch_attention_ordered(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  if (!attention_ordered_fits(a.n_heads, a.n_kv_heads, a.head_dim, cap))
    return fail(CMLD_ERR_SHAPE, "attention (reference order, cluster form): shape %d/%d x %d with %lld positions not supported", a.n_heads,
                a.n_kv_heads, a.head_dim, (long long)cap);
  const int G = a.n_heads / a.n_kv_heads;
#define OA_CASE(g, hd) \
  if (G == g && a.head_dim == hd) return launch_oa<g, hd>(a, cap, s);
  OA_CASE(1, 64) OA_CASE(2, 64) OA_CASE(3, 64) OA_CASE(4, 64) OA_CASE(8, 64)
  OA_CASE(1, 128) OA_CASE(2, 128) OA_CASE(3, 128) OA_CASE(4, 128) OA_CASE(8, 128)
#undef OA_CASE
  return fail(CMLD_ERR_SHAPE, "attention (reference order): unsupported shape");
}

}  // namespace cmld
