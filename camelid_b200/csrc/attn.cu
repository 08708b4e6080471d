// Single-query grouped-query attention over the f16 KV cache (decode step).
//
// CPU form (attention_context_for_head_into_with_kernels, src/inference.rs:30287-30466 in the
// Camelid tree): score_p = dot(q, K_p) * scale; softmax over the cached positions; out =
// sum_p prob_p * V_p.  Here the positions of one (sequence, kv head) are cut into n_splits
// ranges handled by separate CTAs (flash-decoding): every CTA serves all n_heads/n_kv_heads
// query heads of its kv head so each K/V row is read once, keeps a running (max, sum, acc)
// per head.  The ranges are merged either inside a thread-block cluster through distributed shared
// memory (short contexts: eight ranges, one cluster per (sequence, kv head)) or through global memory
// by the CTA that finishes last (any context length).  The result agrees with the CPU's sequential
// sums up to f32 reassociation; the softmax exponentials are __expf (the reference-order kernel in
// exact.cu uses the bit-exact expf).
#include <cooperative_groups.h>

#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnMaxSplits = 64;  // ranges per (sequence, kv head)
constexpr int kAttnCluster = 8;     // CTAs of a cluster (one per range) in the cluster form
constexpr int kMaxGroup = 8;     // query heads per kv head
constexpr int kMaxPer = 8;       // head_dim / 32

// Eight consecutive f16 values (one 16-byte load) widened to f32.
__device__ __forceinline__ void unpack_halves8(const uint4 &raw, float (&out)[8]) {
  const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

constexpr int kMinSplitLen = 64;  // positions per range before another range is opened

// RoPE pair partner and sign: x'[d] = x[d]*c + sgn * x[partner]*s  (src/inference/rope.rs:495-530)
__device__ __forceinline__ float rope_elem(const float *x, int d, int rope_dim, int split_half, const float *ct, const float *st) {
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
  // first of the pair: x0*c - x1*s ; second: x0*s + x1*c
  return first ? __fsub_rn(__fmul_rn(x[d], c), __fmul_rn(x[partner], sn)) : __fadd_rn(__fmul_rn(x[partner], sn), __fmul_rn(x[d], c));
}

// CL = false: ranges through global memory, the CTA that finishes last merges them (any context length).
// CL = true: the kAttnCluster ranges of one (sequence, kv head) are the CTAs of one thread-block cluster and are
// merged through distributed shared memory: no partials in global memory, no fence, no ticket.
template <int G, int PER, bool CL>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t *tickets = a.tickets;
  constexpr int HD = PER * 32;
  const int kvh = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = a.positions[b];
  const int n_pos = pos + 1;
  const int slot = a.slots[b];
  // ranges of at least kMinSplitLen positions; CTAs beyond the last range have nothing to do.  In the cluster
  // form every CTA stays (an empty range contributes weight zero): all of them meet at the cluster barriers.
  const int len = CL ? (n_pos + kAttnCluster - 1) / kAttnCluster : max((n_pos + a.n_splits - 1) / a.n_splits, kMinSplitLen);
  const int n_active = CL ? kAttnCluster : (n_pos + len - 1) / len;
  if (pos < 0 || pos >= a.max_pos) return;  // the same for every CTA of a cluster
  if (!CL && split >= n_active) return;
  const int lo = split * len, hi = min(n_pos, lo + len);
  const bool owns_pos = CL ? (pos / len == split) : (split == n_active - 1);

  // A cache row is HD f16 = LPP 16-byte pieces: LPP lanes share one position, a warp covers PPW positions
  // at a time, and the CTA's NGRP lane groups stride through the range.  Each group keeps its own
  // running (max, sum, accumulator) per query head, so the main loop has no CTA-wide barrier at all;
  // the groups are merged once at the end.
  constexpr int LPP = HD / 8, PPW = 32 / LPP, NGRP = kAttnWarps * PPW;
  constexpr int U = 4;  // positions a group has in flight
  __shared__ float s_q[G][HD];
  __shared__ float s_acc[kAttnWarps][G][HD];
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G], s_wgt[kAttnWarps][G];
  __shared__ float s_w[G][kAttnMaxSplits];
  __shared__ float s_M[G];
  __shared__ bool s_last;

  __half *kbase = const_cast<__half *>(a.k_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  __half *vbase = const_cast<__half *>(a.v_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  if (a.fuse_rope) {
    const int half = a.rope_dim >> 1;
    const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) s_q[i / HD][i % HD] = rope_elem(q + (i / HD) * HD, i % HD, a.rope_dim, a.split_half, ct, st);
    if (owns_pos) {
      // this CTA's range holds the row's own position: append K (rotated) and V to the cache first
      const float *kn = a.k_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      const float *vn = a.v_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      for (int d = threadIdx.x; d < HD; d += kAttnThreads) {
        kbase[(int64_t)pos * HD + d] = __float2half_rn(rope_elem(kn, d, a.rope_dim, a.split_half, ct, st));
        vbase[(int64_t)pos * HD + d] = __float2half_rn(vn[d]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) s_q[i / HD][i % HD] = q[i];
  }
  __syncthreads();  // also orders the cache rows written above before this CTA reads them back
  const int lig = lane % LPP;
  float qr[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) qr[g][e] = s_q[g][lig * 8 + e];

  float m_run[G], l_run[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
  }

  // The trip count is the same for every lane of a warp (the shuffles below need the whole warp): a
  // warp walks bases lo + warp*PPW, + NGRP*U, ...; its groups take consecutive positions from the base
  // and a position beyond the range simply scores -inf.
  for (int base = lo + warp * PPW; base < hi; base += NGRP * U) {
    const int p0 = base + lane / LPP;
    uint4 kraw[U], vraw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = p0 + u * NGRP;
      if (p < hi) {
        kraw[u] = *reinterpret_cast<const uint4 *>(kbase + (int64_t)p * HD + lig * 8);
        vraw[u] = *reinterpret_cast<const uint4 *>(vbase + (int64_t)p * HD + lig * 8);
      } else {
        kraw[u] = vraw[u] = make_uint4(0, 0, 0, 0);
      }
    }
    float sc[U][G];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8];
      unpack_halves8(kraw[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = __fmaf_rn(qr[g][e], kf[e], d);
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        sc[u][g] = p0 + u * NGRP < hi ? d * a.scale : -INFINITY;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float bm = m_run[g];
#pragma unroll
      for (int u = 0; u < U; ++u) bm = fmaxf(bm, sc[u][g]);
      const float corr = bm == -INFINITY ? 1.0f : __expf(m_run[g] - bm);  // first batch: exp(-inf) = 0 on zeros
      l_run[g] *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= corr;
      m_run[g] = bm;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float vf[8];
      unpack_halves8(vraw[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = sc[u][g] == -INFINITY ? 0.0f : __expf(sc[u][g] - m_run[g]);
        l_run[g] += pr;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = __fmaf_rn(pr, vf[e], acc[g][e]);
      }
    }
  }

  // Merge the PPW groups of each warp by shuffles (same dims, different positions) ...
#pragma unroll
  for (int off = 16; off >= LPP; off >>= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m_run[g], off), lo2 = __shfl_xor_sync(0xffffffffu, l_run[g], off);
      const float M = fmaxf(m_run[g], mo);
      const float wa = m_run[g] == -INFINITY ? 0.0f : __expf(m_run[g] - M), wb = mo == -INFINITY ? 0.0f : __expf(mo - M);
      l_run[g] = l_run[g] * wa + lo2 * wb;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] = acc[g][e] * wa + __shfl_xor_sync(0xffffffffu, acc[g][e], off) * wb;
      m_run[g] = M;
    }
  }
  // ... then the warps through shared memory.
  if (lane < LPP) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int e = 0; e < 8; ++e) s_acc[warp][g][lane * 8 + e] = acc[g][e];
      if (lane == 0) {
        s_m[warp][g] = m_run[g];
        s_l[warp][g] = l_run[g];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float L = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float wt = s_m[w][g] == -INFINITY ? 0.0f : __expf(s_m[w][g] - M);
      s_wgt[w][g] = wt;
      L = __fmaf_rn(s_l[w][g], wt, L);
    }
    s_M[g] = M;
    s_l[0][g] = L;  // the range's sum, read below as s_l[0][g] (warp 0's own value is folded in already)
  }
  __syncthreads();
  if constexpr (CL) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    // this range's accumulator (the query copy is no longer needed: every lane holds its part in registers)
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
      const int g = i / HD, d = i % HD;
      float sacc = 0.0f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) sacc = __fmaf_rn(s_acc[w][g][d], s_wgt[w][g], sacc);
      s_q[g][d] = sacc;
    }
    cluster.sync();
    // every CTA merges its share of the outputs, reading the eight ranges' (max, sum, accumulator) from the
    // cluster's shared memory
    constexpr int OPC = G * HD / kAttnCluster;
    float *out = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
    for (int o = threadIdx.x; o < OPC; o += kAttnThreads) {
      const int i = split * OPC + o, g = i / HD;
      float Mr[kAttnCluster], Lr[kAttnCluster], Ar[kAttnCluster];
#pragma unroll
      for (int r = 0; r < kAttnCluster; ++r) {
        Mr[r] = cluster.map_shared_rank(&s_M[0], r)[g];
        Lr[r] = cluster.map_shared_rank(&s_l[0][0], r)[g];
        Ar[r] = cluster.map_shared_rank(&s_q[0][0], r)[i];
      }
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < kAttnCluster; ++r) M = fmaxf(M, Mr[r]);
      float L = 0.0f, acc_o = 0.0f;
#pragma unroll
      for (int r = 0; r < kAttnCluster; ++r) {
        const float w = Mr[r] == -INFINITY ? 0.0f : __expf(Mr[r] - M);
        L = __fmaf_rn(Lr[r], w, L);
        acc_o = __fmaf_rn(Ar[r], w, acc_o);
      }
      out[i] = __fdiv_rn(acc_o, L);
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
    return;
  }
  if (n_active == 1) {
    // a single range: normalise in place, no partials through global memory and no ticket
    float *out1 = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
      const int g = i / HD, d = i % HD;
      float sacc = 0.0f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) sacc = __fmaf_rn(s_acc[w][g][d], s_wgt[w][g], sacc);
      out1[i] = __fdiv_rn(sacc, s_l[0][g]);
    }
    return;
  }
  float *part = a.part + (((int64_t)b * a.n_heads + (int64_t)kvh * G) * a.n_splits) * (HD + 2);
  for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
    const int g = i / HD, d = i % HD;
    float sacc = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) sacc = __fmaf_rn(s_acc[w][g][d], s_wgt[w][g], sacc);
    part[((int64_t)g * a.n_splits + split) * (HD + 2) + d] = sacc;
  }
  if (threadIdx.x < G) {
    part[((int64_t)threadIdx.x * a.n_splits + split) * (HD + 2) + HD] = s_M[threadIdx.x];
    part[((int64_t)threadIdx.x * a.n_splits + split) * (HD + 2) + HD + 1] = s_l[0][threadIdx.x];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&tickets[b * a.n_kv_heads + kvh], 1u) == (unsigned)n_active - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // merge the ranges: out = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M).
  // First the per-(head, range) weights in parallel, then one thread per output.
  for (int i = threadIdx.x; i < G * n_active; i += kAttnThreads) {
    const int g = i / n_active, s2 = i % n_active;
    s_w[g][s2] = __ldcg(part + ((int64_t)g * a.n_splits + s2) * (HD + 2) + HD);  // m
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float M = -INFINITY;
    for (int s2 = 0; s2 < n_active; ++s2) M = fmaxf(M, s_w[g][s2]);
    s_M[g] = M;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * n_active; i += kAttnThreads) {
    const int g = i / n_active, s2 = i % n_active;
    const float ms = s_w[g][s2];
    s_w[g][s2] = ms == -INFINITY ? 0.0f : __expf(ms - s_M[g]);
  }
  __syncthreads();
  float *out = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
    const int g = i / HD, d = i % HD;
    const float *pg = part + (int64_t)g * a.n_splits * (HD + 2);
    float L = 0.0f, o = 0.0f;
#pragma unroll 8
    for (int s2 = 0; s2 < n_active; ++s2) {
      const float w = s_w[g][s2];
      L = __fmaf_rn(__ldcg(pg + (int64_t)s2 * (HD + 2) + HD + 1), w, L);
      o = __fmaf_rn(__ldcg(pg + (int64_t)s2 * (HD + 2) + d), w, o);
    }
    out[i] = __fdiv_rn(o, L);
  }
  if (threadIdx.x == 0) tickets[b * a.n_kv_heads + kvh] = 0;
}

template <int G, int PER>
static int32_t launch_gp(const AttnArgs &a, cudaStream_t s) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)a.n_kv_heads, (unsigned)(a.cluster ? kAttnCluster : a.n_splits), (unsigned)a.batch);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (a.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (a.cluster) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = kAttnCluster;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  static bool carveout_set = false;
  if (!carveout_set) {
    prefer_max_smem_carveout(attn_decode_kernel<G, PER, false>);
    prefer_max_smem_carveout(attn_decode_kernel<G, PER, true>);
    carveout_set = true;
  }
  if (a.cluster) CMLD_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_kernel<G, PER, true>, a));
  else CMLD_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_kernel<G, PER, false>, a));
  return CMLD_OK;
}

template <int G>
static int32_t launch_g(const AttnArgs &a, cudaStream_t s) {
  if (a.n_splits > kAttnMaxSplits) return fail(CMLD_ERR_SHAPE, "attention: more than %d ranges", kAttnMaxSplits);
  switch (a.head_dim) {
    case 32: return launch_gp<G, 1>(a, s);
    case 64: return launch_gp<G, 2>(a, s);
    case 128: return launch_gp<G, 4>(a, s);
    default: return fail(CMLD_ERR_SHAPE, "attention: head_dim %d not in {32,64,128}", a.head_dim);
  }
}

// `part` holds [batch][n_heads][n_splits][head_dim+2] floats; `tickets` batch*n_kv_heads
// counters that are zero before the launch (the merging CTA zeroes them again).
int32_t launch_attention(const AttnArgs &a, cudaStream_t s) {
  if (a.n_heads % a.n_kv_heads != 0) return fail(CMLD_ERR_SHAPE, "attention: n_heads %% n_kv_heads != 0");
  switch (a.n_heads / a.n_kv_heads) {
    case 1: return launch_g<1>(a, s);
    case 2: return launch_g<2>(a, s);
    case 3: return launch_g<3>(a, s);
    case 4: return launch_g<4>(a, s);
    case 8: return launch_g<8>(a, s);
    default: return fail(CMLD_ERR_SHAPE, "attention: %d query heads per kv head not supported", a.n_heads / a.n_kv_heads);
  }
}

}  // namespace cmld

// ====================================================================== allocation-free entry point
//
// Some hosts must not allocate device memory at the moment they need attention: a serving loop
// that has handed the whole device to a memory pool, a caller running under a "no allocator
// calls" rule on its latency path, or an embedder whose CUDA binding exposes launches and copies
// but no allocator.  cmld_attention_decode() makes a cudaMalloc/cudaFree pair per call for its
// split-range partials; this variant keeps those partials in a fixed array that is part of the
// library image, so it makes no allocator call at all.
//
// The price: the array exists once per device (every GPU that loads the library carries it until
// the process exits), problem sizes are capped, and every call uses the same bytes — two calls
// that overlap on the GPU (different streams or host threads) would corrupt each other.

namespace {

constexpr int kNoAllocMaxHeads = 64;
constexpr int kNoAllocMaxHeadDim = 128;
constexpr int kNoAllocSplits = 37;
constexpr size_t kNoAllocPartBytes = (size_t)kNoAllocMaxHeads * kNoAllocSplits * (kNoAllocMaxHeadDim + 2) * sizeof(float);
constexpr size_t kNoAllocTicketOff = kNoAllocPartBytes;                      // kNoAllocMaxHeads counters
constexpr size_t kNoAllocPosOff = kNoAllocTicketOff + kNoAllocMaxHeads * 4;  // position, slot
constexpr size_t kNoAllocBytes = kNoAllocPosOff + 16;                        // about 1.2 MiB

// Device storage.  In host code this name is only a handle for cudaGetSymbolAddress; it is never
// passed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
unsigned char *g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

}  // namespace

extern "C" int32_t cmld_attention_decode_noalloc(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                                 int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int64_t max_pos,
                                                 int64_t n_pos, float scale, float *out_dev) {
  using namespace cmld;
  if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (n_heads < 1 || n_kv_heads < 1 || n_heads > kNoAllocMaxHeads || head_dim > kNoAllocMaxHeadDim)
    return fail(CMLD_ERR_SHAPE, "attention_decode_noalloc takes at most %d query heads of head_dim <= %d (got %d x %d); "
                "use cmld_attention_decode for larger problems", kNoAllocMaxHeads, kNoAllocMaxHeadDim, n_heads, head_dim);
  if (n_pos < 1 || n_pos > max_pos) return fail(CMLD_ERR_INVALID, "n_pos %lld out of range", (long long)n_pos);
  int dev = 0;
  CMLD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(CMLD_ERR_INVALID, "device ordinal %d not supported", dev);
  if (!g_noalloc_ptr[dev]) {
    // One-time set-up on this device (it is the current one): turn the symbol into a device address.
    unsigned char *p = nullptr;
    CMLD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_scratch));
    if (!p) return fail(CMLD_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_ptr[dev] = p;
  }
  unsigned char *scratch = g_noalloc_ptr[dev];
  // same split count as cmld_attention_decode, so the two give identical bits
  const int n_splits = (int)std::max<int64_t>(1, std::min<int64_t>(kNoAllocSplits, max_pos / 32));
  // The array keeps whatever the last call left: the arrival counters must start at zero.
  CMLD_CUDA(cudaMemsetAsync(scratch + kNoAllocTicketOff, 0, kNoAllocMaxHeads * 4, nullptr));
  const int32_t ps[2] = {(int32_t)(n_pos - 1), 0};
  CMLD_CUDA(cudaMemcpyAsync(scratch + kNoAllocPosOff, ps, 8, cudaMemcpyHostToDevice, nullptr));
  AttnArgs a{};
  a.q = q_dev;
  a.k_cache = static_cast<const __half *>(k_cache_dev);
  a.v_cache = static_cast<const __half *>(v_cache_dev);
  a.positions = reinterpret_cast<const int32_t *>(scratch + kNoAllocPosOff);
  a.slots = a.positions + 1;
  a.n_heads = n_heads;
  a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim;
  a.batch = 1;
  a.n_splits = n_splits;
  a.max_pos = max_pos;
  a.scale = scale;
  a.part = reinterpret_cast<float *>(scratch);
  a.tickets = reinterpret_cast<uint32_t *>(scratch + kNoAllocTicketOff);
  a.out = out_dev;
  a.q_stride = (int64_t)n_heads * head_dim;
  a.cluster = n_pos <= 2048 ? 1 : 0;  // as cmld_attention_decode
  CMLD_TRY(launch_attention(a, nullptr));
  cudaError_t ce = cudaStreamSynchronize(nullptr);
  if (ce != cudaSuccess) return fail(CMLD_ERR_CUDA, "attention_decode_noalloc: %s", cudaGetErrorString(ce));
  return CMLD_OK;
}

