// GGUF block formats on the device: re-layout of wire bytes, bit-exact dequantisation,
// embedding-row gather, and the seeded synthetic-weight generator with its quantisers.
//
// This translation unit is compiled with -fmad=false: the reference forms
// (d*sc)*q - (dmin*m) and (d*sc)*q with separate roundings (Q4KBlock::dequantize and
// Q6KBlock::dequantize, src/tensor/mod.rs:5903-5924 and :6039-6066 in the Camelid tree), and
// the generator must reproduce the CPU checker's doubles exactly.
#include "common.cuh"

namespace cmld {

// ------------------------------------------------------------------ wire <-> device layout

// One thread per block.  to_wire = false: wire -> device layout; true: the inverse.
template <bool TO_WIRE>
__global__ void relayout_kernel(int qt_wire, uint8_t *__restrict__ wire, uint8_t *__restrict__ dev, int64_t rows,
                                int64_t cols, int64_t stride) {
  const int blk_vals = (qt_wire == CMLD_Q8_0 || qt_wire == CMLD_Q8_0_HOST36) ? 32 : 256;
  const int64_t bpr = cols / blk_vals;
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= rows * bpr) return;
  const int64_t r = idx / bpr, b = idx % bpr;
  uint8_t *drow = dev + r * stride;
  if (qt_wire == CMLD_Q8_0) {
    uint16_t *w = reinterpret_cast<uint16_t *>(wire + (r * bpr + b) * 34);
    uint16_t *dq = reinterpret_cast<uint16_t *>(drow + b * 32);
    uint16_t *dd = reinterpret_cast<uint16_t *>(drow + cols) + b;
    if (!TO_WIRE) {
      *dd = w[0];
      for (int i = 0; i < 16; ++i) dq[i] = w[1 + i];
    } else {
      w[0] = *dd;
      for (int i = 0; i < 16; ++i) w[1 + i] = dq[i];
    }
  } else if (qt_wire == CMLD_Q8_0_HOST36) {
    // {f32 scale; i8[32]}: the scale is an f16 value widened to f32, so narrowing is exact.
    uint32_t *w = reinterpret_cast<uint32_t *>(wire + (r * bpr + b) * 36);
    uint32_t *dq = reinterpret_cast<uint32_t *>(drow + b * 32);
    uint16_t *dd = reinterpret_cast<uint16_t *>(drow + cols) + b;
    if (!TO_WIRE) {
      *dd = f32_to_f16_bits(__uint_as_float(w[0]));
      for (int i = 0; i < 8; ++i) dq[i] = w[1 + i];
    } else {
      w[0] = __float_as_uint(f16_bits_to_f32(*dd));
      for (int i = 0; i < 8; ++i) w[1 + i] = dq[i];
    }
  } else if (qt_wire == CMLD_Q4_K) {
    uint4 *w = reinterpret_cast<uint4 *>(wire + (r * bpr + b) * 144);
    uint4 *d = reinterpret_cast<uint4 *>(drow + b * 144);
    if (!TO_WIRE) {
      for (int i = 0; i < 9; ++i) d[i] = w[i];
    } else {
      for (int i = 0; i < 9; ++i) w[i] = d[i];
    }
  } else {  // Q6_K: ql[128] qh[64] scales[16] d[2]
    uint16_t *w = reinterpret_cast<uint16_t *>(wire + (r * bpr + b) * 210);
    uint16_t *dblk = reinterpret_cast<uint16_t *>(drow + b * 208);
    uint16_t *dd = reinterpret_cast<uint16_t *>(drow + bpr * 208) + b;
    if (!TO_WIRE) {
      for (int i = 0; i < 104; ++i) dblk[i] = w[i];
      *dd = w[104];
    } else {
      for (int i = 0; i < 104; ++i) w[i] = dblk[i];
      w[104] = *dd;
    }
  }
}

int32_t launch_repack(int qt_in, const uint8_t *wire_dev, int64_t rows, int64_t cols, uint8_t *dst, cudaStream_t s) {
  const int qt_dev = qt_in == CMLD_Q8_0_HOST36 ? CMLD_Q8_0 : qt_in;
  const int blk = (qt_dev == CMLD_Q8_0) ? 32 : 256;
  const int64_t n = rows * (cols / blk);
  if (n == 0) return CMLD_OK;
  const int threads = 128;
  relayout_kernel<false><<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(
      qt_in, const_cast<uint8_t *>(wire_dev), dst, rows, cols, dev_row_stride(qt_dev, cols));
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

int32_t launch_unpack_to_wire(const Weight &w, uint8_t *wire_dev, cudaStream_t s) {
  const int blk = (w.qt == CMLD_Q8_0) ? 32 : 256;
  const int64_t n = w.rows * (w.cols / blk);
  if (n == 0) return CMLD_OK;
  const int threads = 128;
  relayout_kernel<true><<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(w.qt, wire_dev, w.data, w.rows,
                                                                                     w.cols, w.stride);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// ------------------------------------------------------------------ dequantisation

// Value of element `i` of a device-layout row.
__device__ __forceinline__ float dequant_element(const uint8_t *row, int qt, int64_t cols, int64_t i) {
  if (qt == CMLD_Q8_0) {
    const float d = f16_bits_to_f32(reinterpret_cast<const uint16_t *>(row + cols)[i >> 5]);
    return d * (float)reinterpret_cast<const int8_t *>(row)[i];
  }
  const int64_t nsb = cols >> 8, sb = i >> 8;
  const int e = (int)(i & 255);
  if (qt == CMLD_Q4_K) {
    const uint32_t *meta = reinterpret_cast<const uint32_t *>(row + sb * 144);
    const uint32_t dm = meta[0];
    const float d = f16_bits_to_f32((uint16_t)(dm & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(dm >> 16));
    const int p = e >> 6, hi = (e >> 5) & 1, l = e & 31;
    const uint8_t byte = row[sb * 144 + 16 + 32 * p + l];
    const int nib = hi ? (byte >> 4) : (byte & 15);
    int sc, m;
    q4k_scale_min(2 * p + hi, meta[1], meta[2], meta[3], sc, m);
    const float scale = d * (float)sc;
    const float mn = dmin * (float)m;
    return scale * (float)nib - mn;
  }
  // Q6_K
  const int h = e >> 7, stream = (e >> 5) & 3, l = e & 31;
  const uint8_t *ql = row + sb * 208 + 64 * h;
  const uint8_t qh = row[sb * 208 + 128 + 32 * h + l];
  const uint8_t lb = ql[(stream & 1) * 32 + l];
  const int lo = (stream & 2) ? (lb >> 4) : (lb & 15);
  const int q = (lo | (((qh >> (2 * stream)) & 3) << 4)) - 32;
  const int sc = reinterpret_cast<const int8_t *>(row + sb * 208 + 192)[8 * h + (l >> 4) + 2 * stream];
  const float d = f16_bits_to_f32(reinterpret_cast<const uint16_t *>(row + nsb * 208)[sb]);
  return d * (float)sc * (float)q;
}

__global__ void dequant_kernel(const uint8_t *__restrict__ data, int qt, int64_t cols, int64_t stride, int64_t row0,
                               int64_t nrows, float *__restrict__ out) {
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= nrows * cols) return;
  const int64_t r = idx / cols, c = idx % cols;
  out[idx] = dequant_element(data + (row0 + r) * stride, qt, cols, c);
}

int32_t launch_dequant(const Weight &w, int64_t row0, int64_t nrows, float *out, cudaStream_t s) {
  const int64_t n = nrows * w.cols;
  if (n == 0) return CMLD_OK;
  if (w.qt == CMLD_F32) {
    CMLD_CUDA(cudaMemcpyAsync(out, w.data + row0 * w.stride, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    return CMLD_OK;
  }
  dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(w.data, w.qt, w.cols, w.stride, row0, nrows, out);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// Embedding lookup (CpuTensor::embedding_lookup, src/tensor/mod.rs:2899-3216): dequantise
// row tokens[b] of the table into out[b][cols].
__global__ void embed_gather_kernel(const uint8_t *__restrict__ data, int qt, int64_t rows, int64_t cols,
                                    int64_t stride, const int32_t *__restrict__ tokens, float *__restrict__ out) {
  const int b = blockIdx.y;
  int64_t tok = tokens[b];
  if (tok < 0 || tok >= rows) tok = 0;  // ids are validated on the host; keep device reads in range regardless
  const uint8_t *row = data + tok * stride;
  for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < cols; c += (int64_t)gridDim.x * blockDim.x)
    out[(int64_t)b * cols + c] = qt == CMLD_F32 ? reinterpret_cast<const float *>(row)[c]
                                                : dequant_element(row, qt, cols, c);
}

int32_t launch_embed_gather(const Weight &w, const int32_t *tokens_dev, int32_t batch, float *out, cudaStream_t s) {
  static bool carveout_set = false;
  if (!carveout_set) {
    prefer_max_smem_carveout(embed_gather_kernel);
    carveout_set = true;
  }
  dim3 grid((unsigned)((w.cols + 255) / 256), (unsigned)batch);
  embed_gather_kernel<<<grid, 256, 0, s>>>(w.data, w.qt, w.rows, w.cols, w.stride, tokens_dev, out);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// ------------------------------------------------------------------ seeded synthetic weights
//
// value(seed, stream, index): splitmix64-hashed counters -> Box-Muller in double with
// polynomial log / cos built from + - * / only, so this reproduces the CPU checker's
// generator bit-for-bit (no contraction in this file).

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ uint64_t synth_hash(uint64_t seed, uint64_t stream, uint64_t index, uint64_t salt) {
  uint64_t h = splitmix64(seed ^ 0x632be59bd9b4e019ull);
  h = splitmix64(h ^ (stream * 0x9e3779b97f4a7c15ull + salt));
  return splitmix64(h ^ index);
}

__device__ double synth_log(double u) {
  uint64_t b = (uint64_t)__double_as_longlong(u);
  int e = (int)((b >> 52) & 0x7ff) - 1023;
  b = (b & 0x000fffffffffffffull) | 0x3ff0000000000000ull;
  double m = __longlong_as_double((long long)b);
  if (m > 1.4142135623730951) {
    m = m * 0.5;
    e += 1;
  }
  const double s = (m - 1.0) / (m + 1.0);
  const double s2 = s * s;
  double p = 1.0 / 19.0;
  p = p * s2 + 1.0 / 17.0;
  p = p * s2 + 1.0 / 15.0;
  p = p * s2 + 1.0 / 13.0;
  p = p * s2 + 1.0 / 11.0;
  p = p * s2 + 1.0 / 9.0;
  p = p * s2 + 1.0 / 7.0;
  p = p * s2 + 1.0 / 5.0;
  p = p * s2 + 1.0 / 3.0;
  p = p * s2 + 1.0;
  return 2.0 * s * p + (double)e * 0.6931471805599453;
}

__device__ double synth_cos2pi(double t) {
  double sign = 1.0;
  if (t >= 0.5) t = 1.0 - t;
  if (t > 0.25) {
    t = 0.5 - t;
    sign = -1.0;
  }
  bool use_sin = false;
  if (t > 0.125) {
    t = 0.25 - t;
    use_sin = true;
  }
  const double x = t * 6.283185307179586;
  const double x2 = x * x;
  double r;
  if (use_sin) {
    double p = -1.0 / 39916800.0;
    p = p * x2 + 1.0 / 362880.0;
    p = p * x2 - 1.0 / 5040.0;
    p = p * x2 + 1.0 / 120.0;
    p = p * x2 - 1.0 / 6.0;
    p = p * x2 + 1.0;
    r = x * p;
  } else {
    double p = 1.0 / 479001600.0;
    p = p * x2 - 1.0 / 3628800.0;
    p = p * x2 + 1.0 / 40320.0;
    p = p * x2 - 1.0 / 720.0;
    p = p * x2 + 1.0 / 24.0;
    p = p * x2 - 1.0 / 2.0;
    p = p * x2 + 1.0;
    r = p;
  }
  return sign * r;
}

__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t stream, uint64_t index, float sigma) {
  const uint64_t h1 = synth_hash(seed, stream, index, 1);
  const uint64_t h2 = synth_hash(seed, stream, index, 2);
  const double u1 = ((double)(h1 >> 11) + 1.0) * (1.0 / 9007199254740992.0);
  const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
  const double r = sqrt(-2.0 * synth_log(u1));
  const double z = r * synth_cos2pi(u2);
  return (float)z * sigma;
}

__device__ __forceinline__ float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// quantize_block_q8_0 (src/quantize.rs:98-119), written straight into the device layout.
__device__ void quantize_store_q8_0(const float *src, uint8_t *row, int64_t cols, int64_t b) {
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) amax = fabsf(src[i]) > amax ? fabsf(src[i]) : amax;
  const float d = amax / 127.0f;
  const float id = d != 0.0f ? 1.0f / d : 0.0f;
  reinterpret_cast<uint16_t *>(row + cols)[b] = f32_to_f16_bits(d);
  int8_t *q = reinterpret_cast<int8_t *>(row + b * 32);
  for (int i = 0; i < 32; ++i) q[i] = (int8_t)clampf(roundf(src[i] * id), -128.0f, 127.0f);
}

// quantize_block_q4_k (src/quantize.rs:152-244).
__device__ void quantize_store_q4_k(const float *src, uint8_t *row, int64_t sb) {
  float mins[8], maxs[8];
  for (int g = 0; g < 8; ++g) {
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < 32; ++i) {
      const float v = src[32 * g + i];
      if (v < mn) mn = v;
      if (v > mx) mx = v;
    }
    mins[g] = mn;
    maxs[g] = mx;
  }
  float super_min = 0.0f, super_max = 0.0f;
  for (int g = 0; g < 8; ++g) {
    const float emin = fminf(mins[g], 0.0f);
    const float gs = fmaxf(maxs[g] - emin, 0.0f) / 15.0f;
    if (gs > super_max) super_max = gs;
    const float mm = fmaxf(-mins[g], 0.0f);
    if (mm > super_min) super_min = mm;
  }
  const float d = super_max / 63.0f, dmin = super_min / 63.0f;
  const float id = d != 0.0f ? 1.0f / d : 0.0f;
  const float idmin = dmin != 0.0f ? 1.0f / dmin : 0.0f;
  uint8_t sc[8], m[8];
  for (int g = 0; g < 8; ++g) {
    const float emin = fminf(mins[g], 0.0f);
    const float gs = fmaxf(maxs[g] - emin, 0.0f) / 15.0f;
    sc[g] = (uint8_t)clampf(roundf(gs * id), 0.0f, 63.0f);
    m[g] = (uint8_t)clampf(roundf(fmaxf(-mins[g], 0.0f) * idmin), 0.0f, 63.0f);
  }
  uint8_t *meta = row + sb * 144;
  reinterpret_cast<uint16_t *>(meta)[0] = f32_to_f16_bits(d);
  reinterpret_cast<uint16_t *>(meta)[1] = f32_to_f16_bits(dmin);
  uint8_t ps[12];
  for (int g = 0; g < 12; ++g) ps[g] = 0;
  for (int g = 0; g < 4; ++g) {
    ps[g] = sc[g] & 0x3f;
    ps[g + 4] = m[g] & 0x3f;
  }
  for (int g = 4; g < 8; ++g) {
    ps[g - 4] |= (uint8_t)((sc[g] >> 4) << 6);
    ps[g] |= (uint8_t)((m[g] >> 4) << 6);
    ps[g + 4] = (uint8_t)((sc[g] & 0x0f) | ((m[g] & 0x0f) << 4));
  }
  for (int g = 0; g < 12; ++g) meta[4 + g] = ps[g];
  uint8_t *qs = row + sb * 144 + 16;
  for (int p = 0; p < 4; ++p) {
    const float d0 = d * (float)sc[2 * p], d1 = d * (float)sc[2 * p + 1];
    const float m0 = -(dmin * (float)m[2 * p]), m1 = -(dmin * (float)m[2 * p + 1]);
    const float i0 = d0 != 0.0f ? 1.0f / d0 : 0.0f, i1 = d1 != 0.0f ? 1.0f / d1 : 0.0f;
    for (int i = 0; i < 32; ++i) {
      const uint8_t lo = (uint8_t)clampf(roundf((src[64 * p + i] - m0) * i0), 0.0f, 15.0f);
      const uint8_t hi = (uint8_t)clampf(roundf((src[64 * p + 32 + i] - m1) * i1), 0.0f, 15.0f);
      qs[32 * p + i] = (uint8_t)((lo & 0x0f) | (hi << 4));
    }
  }
}

// This project's Q6_K quantiser (the reference has none): per 16-value group gs = amax/31,
// d = max(gs)/127 as f16, sc = round(gs/d), q = round(x/(d*sc)) in [-32,31].
__device__ void quantize_store_q6_k(const float *src, uint8_t *row, int64_t nsb, int64_t sb) {
  float gs[16];
  float smax = 0.0f;
  for (int j = 0; j < 16; ++j) {
    float amax = 0.0f;
    for (int i = 0; i < 16; ++i) amax = fabsf(src[16 * j + i]) > amax ? fabsf(src[16 * j + i]) : amax;
    gs[j] = amax / 31.0f;
    if (gs[j] > smax) smax = gs[j];
  }
  const float d = smax / 127.0f;
  const float id = d != 0.0f ? 1.0f / d : 0.0f;
  uint8_t *ql = row + sb * 208, *qh = row + sb * 208 + 128;
  int8_t *scp = reinterpret_cast<int8_t *>(row + sb * 208 + 192);
  reinterpret_cast<uint16_t *>(row + nsb * 208)[sb] = f32_to_f16_bits(d);
  float sub_id[16];
  for (int j = 0; j < 16; ++j) {
    const int8_t s = (int8_t)clampf(roundf(gs[j] * id), 0.0f, 127.0f);
    scp[j] = s;
    const float sub_d = d * (float)s;
    sub_id[j] = sub_d != 0.0f ? 1.0f / sub_d : 0.0f;
  }
  for (int h = 0; h < 2; ++h)
    for (int l = 0; l < 32; ++l) {
      uint8_t q[4];
      for (int st = 0; st < 4; ++st) {
        const int idx = 128 * h + 32 * st + l;
        q[st] = (uint8_t)((int)clampf(roundf(src[idx] * sub_id[idx >> 4]), -32.0f, 31.0f) + 32);
      }
      ql[64 * h + l] = (uint8_t)((q[0] & 0x0f) | ((q[2] & 0x0f) << 4));
      ql[64 * h + l + 32] = (uint8_t)((q[1] & 0x0f) | ((q[3] & 0x0f) << 4));
      qh[32 * h + l] = (uint8_t)((q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6));
    }
}

// One thread per block of 32 (Q8_0 / F32) or 256 (K-quants) values.
__global__ void synth_kernel(uint8_t *__restrict__ data, int qt, int64_t rows, int64_t cols, int64_t stride,
                             uint64_t seed, uint64_t stream, int64_t row0, float sigma) {
  const int blk = (qt == CMLD_Q8_0 || qt == CMLD_F32) ? 32 : 256;
  const int64_t bpr = cols / blk;
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= rows * bpr) return;
  const int64_t r = idx / bpr, b = idx % bpr;
  uint8_t *row = data + r * stride;
  const uint64_t base = (uint64_t)((row0 + r) * cols + b * blk);
  if (qt == CMLD_F32) {
    float *o = reinterpret_cast<float *>(row) + b * 32;
    for (int i = 0; i < 32; ++i) o[i] = synth_normal(seed, stream, base + i, sigma);
    return;
  }
  if (qt == CMLD_Q8_0) {
    float v[32];
    for (int i = 0; i < 32; ++i) v[i] = synth_normal(seed, stream, base + i, sigma);
    quantize_store_q8_0(v, row, cols, b);
    return;
  }
  float v[256];
  for (int i = 0; i < 256; ++i) v[i] = synth_normal(seed, stream, base + i, sigma);
  if (qt == CMLD_Q4_K) quantize_store_q4_k(v, row, b);
  else quantize_store_q6_k(v, row, bpr, b);
}

int32_t launch_synth(const Weight &w, uint64_t seed, uint64_t stream_id, int64_t row0, float sigma, cudaStream_t s) {
  const int blk = (w.qt == CMLD_Q8_0 || w.qt == CMLD_F32) ? 32 : 256;
  const int64_t n = w.rows * (w.cols / blk);
  if (n == 0) return CMLD_OK;
  const int threads = 64;
  synth_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(w.data, w.qt, w.rows, w.cols, w.stride, seed,
                                                                           stream_id, row0, sigma);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

}  // namespace cmld
