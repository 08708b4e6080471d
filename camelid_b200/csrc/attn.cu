// Single-query grouped-query attention over the f16 KV cache (decode step).
//
// CPU form (attention_context_for_head_into_with_kernels, src/inference.rs:30287-30466 in the
// Camelid tree): score_p = dot(q, K_p) * scale; softmax over the cached positions; out =
// sum_p prob_p * V_p.  Here the positions of one (sequence, kv head) are cut into n_splits
// ranges handled by separate CTAs (flash-decoding): every CTA serves all n_heads/n_kv_heads
// query heads of its kv head so each K/V row is read once, keeps a running (max, sum, acc)
// per head, and the CTA that finishes last merges the ranges.  The result agrees with the
// CPU's sequential sums up to f32 reassociation.
#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnChunk = 256;  // positions per softmax chunk
constexpr int kMaxGroup = 8;     // query heads per kv head
constexpr int kMaxPer = 8;       // head_dim / 32

// PER consecutive f16 values of a cache row, widened to f32 (one 2/4/8-byte load).
template <int PER>
__device__ __forceinline__ void load_halves(const __half *p, float (&out)[PER]) {
  if constexpr (PER == 4) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const __half2 h0 = *reinterpret_cast<const __half2 *>(&raw.x), h1 = *reinterpret_cast<const __half2 *>(&raw.y);
    out[0] = __low2float(h0);
    out[1] = __high2float(h0);
    out[2] = __low2float(h1);
    out[3] = __high2float(h1);
  } else if constexpr (PER == 2) {
    const __half2 h0 = *reinterpret_cast<const __half2 *>(p);
    out[0] = __low2float(h0);
    out[1] = __high2float(h0);
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e) out[e] = __half2float(p[e]);
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

template <int G, int PER>
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
  // ranges of at least kMinSplitLen positions; CTAs beyond the last range have nothing to do
  const int len = max((n_pos + a.n_splits - 1) / a.n_splits, kMinSplitLen);
  const int n_active = (n_pos + len - 1) / len;
  if (split >= n_active || pos < 0 || pos >= a.max_pos) return;
  const int lo = split * len, hi = min(n_pos, lo + len);

  __shared__ float s_q[G][HD];
  __shared__ float s_sc[G][kAttnChunk];
  __shared__ float s_red[kAttnWarps][G];
  __shared__ float s_acc[kAttnWarps][G][HD];
  __shared__ bool s_last;

  __half *kbase = const_cast<__half *>(a.k_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  __half *vbase = const_cast<__half *>(a.v_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  if (a.fuse_rope) {
    const int half = a.rope_dim >> 1;
    const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) s_q[i / HD][i % HD] = rope_elem(q + (i / HD) * HD, i % HD, a.rope_dim, a.split_half, ct, st);
    if (split == n_active - 1) {
      // this CTA's range ends at the row's own position: append K (rotated) and V to the cache first
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
  float qr[G][PER];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < PER; ++e) qr[g][e] = s_q[g][lane * PER + e];

  float m_run[G], l_run[G], acc[G][PER];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[g][e] = 0.0f;
  }

  for (int c0 = lo; c0 < hi; c0 += kAttnChunk) {
    const int cn = min(kAttnChunk, hi - c0);
    // scores of this chunk
    for (int p = warp; p < cn; p += kAttnWarps) {
      const __half *kr = kbase + (int64_t)(c0 + p) * HD + lane * PER;
      float kv[PER];
      load_halves<PER>(kr, kv);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < PER; ++e) d = __fmaf_rn(qr[g][e], kv[e], d);
        d = warp_sum(d);
        if (lane == 0) s_sc[g][p] = __fmul_rn(d, a.scale);
      }
    }
    __syncthreads();
    // chunk maximum per head
    float cm[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = -INFINITY;
      for (int p = threadIdx.x; p < cn; p += kAttnThreads) v = fmaxf(v, s_sc[g][p]);
      v = warp_max(v);
      if (lane == 0) s_red[warp][g] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = s_red[0][g];
#pragma unroll
      for (int w = 1; w < kAttnWarps; ++w) v = fmaxf(v, s_red[w][g]);
      cm[g] = fmaxf(m_run[g], v);
    }
    __syncthreads();
    // probabilities in place, running sums
    float ls[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.0f;
      for (int p = threadIdx.x; p < cn; p += kAttnThreads) {
        const float e = expf_exact(s_sc[g][p] - cm[g]);
        s_sc[g][p] = e;
        s += e;
      }
      s = warp_sum(s);
      if (lane == 0) s_red[warp][g] = s;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) s += s_red[w][g];
      ls[g] = s;
      const float corr = m_run[g] == -INFINITY ? 0.0f : expf_exact(m_run[g] - cm[g]);
      l_run[g] = l_run[g] * corr + ls[g];
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[g][e] *= corr;
      m_run[g] = cm[g];
    }
    // weighted values: warp w takes positions w, w+8, ...
    for (int p = warp; p < cn; p += kAttnWarps) {
      const __half *vr = vbase + (int64_t)(c0 + p) * HD + lane * PER;
      float vv[PER];
      load_halves<PER>(vr, vv);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = s_sc[g][p];
#pragma unroll
        for (int e = 0; e < PER; ++e) acc[g][e] = __fmaf_rn(pr, vv[e], acc[g][e]);
      }
    }
    __syncthreads();
  }

  // Each warp accumulated a subset of the positions against the shared (m_run, l_run);
  // add the warps' accumulators.
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < PER; ++e) s_acc[warp][g][lane * PER + e] = acc[g][e];
  __syncthreads();
  if (n_active == 1) {
    // a single range: normalise in place, no partials through global memory and no ticket
    float *out1 = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
    for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
      const int g = i / HD, d = i % HD;
      float sacc = 0.0f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) sacc += s_acc[w][g][d];
      // the merge below computes fma(acc, 1, 0) / fma(l, 1, 0): the same bits
      out1[i] = __fdiv_rn(sacc, l_run[g]);
    }
    return;
  }
  float *part = a.part + (((int64_t)b * a.n_heads + (int64_t)kvh * G) * a.n_splits) * (HD + 2);
  for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
    const int g = i / HD, d = i % HD;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) s += s_acc[w][g][d];
    part[((int64_t)g * a.n_splits + split) * (HD + 2) + d] = s;
  }
  if (threadIdx.x < G) {
    part[((int64_t)threadIdx.x * a.n_splits + split) * (HD + 2) + HD] = m_run[threadIdx.x];
    part[((int64_t)threadIdx.x * a.n_splits + split) * (HD + 2) + HD + 1] = l_run[threadIdx.x];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&tickets[b * a.n_kv_heads + kvh], 1u) == (unsigned)n_active - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // merge the ranges: out = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M).
  // First the per-(head, range) weights in parallel (s_sc is free now), then one thread per output.
  float *s_w = &s_sc[0][0];  // [G][n_active] weights, n_active <= 64 <= kAttnChunk
  for (int i = threadIdx.x; i < G * n_active; i += kAttnThreads) {
    const int g = i / n_active, s2 = i % n_active;
    s_w[g * kAttnChunk + s2] = __ldcg(part + ((int64_t)g * a.n_splits + s2) * (HD + 2) + HD);  // m
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float M = -INFINITY;
    for (int s2 = 0; s2 < n_active; ++s2) M = fmaxf(M, s_w[g * kAttnChunk + s2]);
    s_red[0][g] = M;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * n_active; i += kAttnThreads) {
    const int g = i / n_active, s2 = i % n_active;
    const float ms = s_w[g * kAttnChunk + s2];
    s_w[g * kAttnChunk + s2] = ms == -INFINITY ? 0.0f : expf_exact(ms - s_red[0][g]);
  }
  __syncthreads();
  float *out = a.out + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  for (int i = threadIdx.x; i < G * HD; i += kAttnThreads) {
    const int g = i / HD, d = i % HD;
    const float *pg = part + (int64_t)g * a.n_splits * (HD + 2);
    float L = 0.0f, o = 0.0f;
#pragma unroll 4
    for (int s2 = 0; s2 < n_active; ++s2) {
      const float w = s_w[g * kAttnChunk + s2];
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
  cfg.gridDim = dim3((unsigned)a.n_kv_heads, (unsigned)a.n_splits, (unsigned)a.batch);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  static bool carveout_set = false;
  if (!carveout_set) {
    prefer_max_smem_carveout(attn_decode_kernel<G, PER>);
    carveout_set = true;
  }
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_kernel<G, PER>, a));
  return CMLD_OK;
}

template <int G>
static int32_t launch_g(const AttnArgs &a, cudaStream_t s) {
  if (a.n_splits > kAttnChunk) return fail(CMLD_ERR_SHAPE, "attention: more than %d ranges", kAttnChunk);
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
  CMLD_TRY(launch_attention(a, nullptr));
  cudaError_t ce = cudaStreamSynchronize(nullptr);
  if (ce != cudaSuccess) return fail(CMLD_ERR_CUDA, "attention_decode_noalloc: %s", cudaGetErrorString(ce));
  return CMLD_OK;
}

