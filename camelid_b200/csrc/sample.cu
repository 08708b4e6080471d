// On-device token sampling over a resident logits row (the functions of src/cuda_resident/sampling.cuh in the
// Camelid tree): a temperature draw by the Gumbel-max trick — argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)),
// u_i a stateless splitmix64 hash of (seed, i) — and the same draw restricted to the tokens that pass a min-p
// filter.  One CTA walks the row; each thread keeps its best (score, index), then warps and the CTA combine them
// with the greedy tie rule (strictly greater wins, equal scores go to the lower index).
//
// The uniforms are integer arithmetic and equal the CPU's bit for bit.  logf / expf are the device's: a score can
// differ from a host evaluation in the last bits, so a draw can differ where two scores tie to within that.
#include "common.cuh"

namespace cmld {

namespace {

constexpr int kSampleThreads = 1024;

// 24 random bits to (0, 1): the midpoint (m + 0.5) / 2^24, with the one value that would round to 1.0 clamped to the
// largest float below it (sampling_uniform_from_u24).
__device__ __forceinline__ float uniform_from_u24(unsigned int m) { return fminf(((float)m + 0.5f) / 16777216.0f, 0.999999940395355224609375f); }

__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned int idx) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ULL * (unsigned long long)(idx + 1u);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z = z ^ (z >> 31);
  return uniform_from_u24((unsigned int)(z >> 40));
}

// 1 keep, 0 drop, -1 = too close to the cutoff (or not finite) to decide here: the caller samples that row on the
// CPU from the logits it already has (min_p_candidate).
__device__ __forceinline__ int min_p_keep(float logit, float max_logit, float min_p, int n) {
  if (n <= 0 || !isfinite(logit) || !isfinite(max_logit) || !isfinite(min_p) || min_p <= 0.0f || min_p >= 1.0f ||
      min_p < (4.0f * 1.1754943508222875e-38f) * (float)n)
    return -1;
  const float ratio = expf(logit - max_logit);
  const float margin = (64.0f * 1.1920928955078125e-7f) * min_p;
  if (!isfinite(ratio) || fabsf(ratio - min_p) <= margin) return -1;
  return ratio > min_p ? 1 : 0;
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ void take(Best &a, float ov, int oi) {
  if (ov > a.v || (ov == a.v && oi < a.i)) {
    a.v = ov;
    a.i = oi;
  }
}
// CTA-wide best; flag is OR-ed alongside.  Result valid in thread 0.
__device__ __forceinline__ Best cta_best(Best b, int &flag) {
  __shared__ float sv[kSampleThreads / 32];
  __shared__ int si[kSampleThreads / 32], sf[kSampleThreads / 32];
  for (int o = 16; o > 0; o >>= 1) {
    take(b, __shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o));
    flag |= __shfl_xor_sync(0xffffffffu, flag, o);
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) sv[w] = b.v, si[w] = b.i, sf[w] = flag;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int k = 1; k < kSampleThreads / 32; ++k) {
      take(b, sv[k], si[k]);
      flag |= sf[k];
    }
  __syncthreads();
  return b;
}

__global__ void __launch_bounds__(kSampleThreads) sample_gumbel_kernel(const float *__restrict__ logits, int n, float inv_temp,
                                                                      unsigned long long seed, uint32_t *out) {
  Best b{-3.4e38f, 0};
  // a thread walks increasing indices, so "strictly greater" keeps the lowest index among its equals
  for (int i = threadIdx.x; i < n; i += kSampleThreads) {
    const float g = -logf(-logf(hash_uniform(seed, (unsigned int)i)));
    const float v = logits[i] * inv_temp + g;
    if (v > b.v) b.v = v, b.i = i;
  }
  int flag = 0;
  b = cta_best(b, flag);
  if (threadIdx.x == 0) out[0] = (uint32_t)b.i;
}

// row maximum over the finite logits; flag set by a non-finite logit or an empty row
__device__ __forceinline__ float row_max(const float *logits, int n, int &bad) {
  __shared__ float sm[kSampleThreads / 32];
  __shared__ int sb[kSampleThreads / 32];
  __shared__ float s_max;
  __shared__ int s_bad;
  float m = -INFINITY;
  bad = n <= 0;
  for (int i = threadIdx.x; i < n; i += kSampleThreads) {
    const float x = logits[i];
    if (!isfinite(x)) bad = 1;
    else m = fmaxf(m, x);
  }
  for (int o = 16; o > 0; o >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m, sb[threadIdx.x >> 5] = bad;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < kSampleThreads / 32; ++k) m = fmaxf(m, sm[k]), bad |= sb[k];
    s_max = m, s_bad = bad;
  }
  __syncthreads();
  bad = s_bad;
  return s_max;
}

// Min-p filtering precedes temperature.  0xffffffff = sample this row on the CPU (sample_gumbel_filtered).
__global__ void __launch_bounds__(kSampleThreads) sample_filtered_kernel(const float *__restrict__ logits, int n, float temperature,
                                                                        float min_p, unsigned long long seed, uint32_t *out) {
  int bad;
  const float maximum = row_max(logits, n, bad);
  bad |= !isfinite(temperature) || temperature <= 0.0f;
  Best b{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < n; i += kSampleThreads) {
    const int keep = min_p_keep(logits[i], maximum, min_p, n);
    if (keep < 0) bad = 1;
    if (keep == 1) {
      const float g = -logf(-logf(hash_uniform(seed, (unsigned int)i)));
      // divide, then centre (sampling_centered_logit), then add the noise: a large common offset cannot erase the draw
      const float score = (logits[i] / temperature) - (maximum / temperature) + g;
      if (!isfinite(score)) bad = 1;
      take(b, score, i);
    }
  }
  b = cta_best(b, bad);
  if (threadIdx.x == 0) out[0] = (bad || b.i == 0x7fffffff) ? 0xffffffffu : (uint32_t)b.i;
}

__global__ void __launch_bounds__(kSampleThreads) min_p_mask_kernel(const float *__restrict__ logits, int n, float min_p, int32_t *mask) {
  int bad;
  const float maximum = row_max(logits, n, bad);
  for (int i = threadIdx.x; i < n; i += kSampleThreads) mask[i] = bad ? -1 : min_p_keep(logits[i], maximum, min_p, n);
}

__global__ void uniforms_kernel(unsigned long long seed, int n, float *out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = hash_uniform(seed, (unsigned int)i);
}

}  // namespace

int32_t launch_sample_gumbel(const float *logits, int32_t n, float inv_temp, uint64_t seed, uint32_t *out_dev, cudaStream_t s) {
  sample_gumbel_kernel<<<1, kSampleThreads, 0, s>>>(logits, n, inv_temp, (unsigned long long)seed, out_dev);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}
int32_t launch_sample_gumbel_filtered(const float *logits, int32_t n, float temperature, float min_p, uint64_t seed, uint32_t *out_dev,
                                      cudaStream_t s) {
  sample_filtered_kernel<<<1, kSampleThreads, 0, s>>>(logits, n, temperature, min_p, (unsigned long long)seed, out_dev);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}
int32_t launch_min_p_mask(const float *logits, int32_t n, float min_p, int32_t *mask_dev, cudaStream_t s) {
  min_p_mask_kernel<<<1, kSampleThreads, 0, s>>>(logits, n, min_p, mask_dev);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}
int32_t launch_sample_uniforms(uint64_t seed, int32_t n, float *out_dev, cudaStream_t s) {
  uniforms_kernel<<<(n + 255) / 256, 256, 0, s>>>((unsigned long long)seed, n, out_dev);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
