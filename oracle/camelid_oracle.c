/*
 * camelid_oracle.c — CPU restatement of Camelid's decode-step arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it is
 * linked/loaded by the test-suite, by the smoke check and by the benchmark's CPU
 * baseline leg, never by the product path.
 *
 * Camelid is a Rust crate and no Rust toolchain is available where this is built, so
 * the reference cannot be compiled; every function below restates, in plain C, the
 * arithmetic of the reference function it cites (paths are relative to the Camelid
 * source tree).  All float maths is IEEE f32 with no contraction (build with
 * -ffp-contract=off); fmaf() appears only where the reference writes mul_add; sums are
 * sequential in the stated index order; expf/sinf/cosf/powf/sqrtf are glibc's, which is
 * what Rust's std calls on Linux.
 *
 * Pinning: the dequantisers are checked bit-for-bit against the reference's golden
 * vectors (tests/fixtures/dequant/{Q8_0,Q4_K,Q6_K}.json), and the quantisers, dots,
 * RoPE, attention, top-k and MoE against the closed-form cases of the reference's unit
 * tests (see tests/test_oracle_*.py).  A whole-model K-quant forward has no golden
 * vector in the reference: end-to-end logits are "parity unpinned" by in-repo
 * fixtures and rest on the component pins.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { QT_Q8_0 = 8, QT_Q4_K = 12, QT_Q6_K = 14, QT_F32 = 0 }; /* GGUF type ids: src/gguf/reader.rs:94-128 */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------ f16 */

/* src/tensor/mod.rs:5416-5455 (f32_to_f16_bits): RNE, subnormals, overflow->inf. */
ORACLE_API uint16_t orc_f32_to_f16_bits(float value) {
  uint32_t bits = f32_bits(value);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  int32_t exp = (int32_t)((bits >> 23) & 0xffu);
  uint32_t frac = bits & 0x007fffffu;
  if (exp == 0xff) {
    uint16_t nan = frac != 0 ? (uint16_t)(0x0200u | ((frac >> 13) & 0x03ffu)) : 0;
    return (uint16_t)(sign | 0x7c00u | nan);
  }
  int32_t half_exp = exp - 127 + 15;
  if (half_exp >= 0x1f) return (uint16_t)(sign | 0x7c00u);
  if (half_exp <= 0) {
    if (half_exp < -10) return sign;
    uint32_t mant = frac | 0x00800000u;
    uint32_t shift = (uint32_t)(14 - half_exp);
    uint16_t half = (uint16_t)(mant >> shift);
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half & 1) == 1)) half += 1;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)half_exp << 10) | (frac >> 13);
  uint32_t rem = frac & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1) == 1)) half += 1;
  return (uint16_t)(sign | (uint16_t)half);
}

/* src/tensor/mod.rs:5463-5544 (f16_bits_to_f32 / fast_f16_to_f32): exact widening. */
ORACLE_API float orc_f16_bits_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
  uint32_t exp = (uint32_t)(h & 0x7c00u) >> 10;
  uint32_t frac = (uint32_t)(h & 0x03ffu);
  if (exp == 0) {
    if (frac == 0) return bits_f32(sign);
    /* subnormal: value = frac * 2^-24, exact in f32 */
    float v = (float)frac * 5.9604644775390625e-8f;
    return sign ? -v : v;
  }
  if (exp == 0x1f) return bits_f32(sign | 0x7f800000u | (frac << 13));
  return bits_f32(sign | ((exp + 112u) << 23) | (frac << 13));
}

/* src/inference/kv_f16.rs:33-67: the KV store's f32->f16; as above but any NaN
 * becomes sign|0x7E00. */
ORACLE_API uint16_t orc_kv_f32_to_f16_bits(float value) {
  if (value != value) return (uint16_t)(((f32_bits(value) >> 16) & 0x8000u) | 0x7e00u);
  return orc_f32_to_f16_bits(value);
}

static inline float f16_round(float v) { return orc_f16_bits_to_f32(orc_f32_to_f16_bits(v)); }
static inline float kv_f16_round(float v) { return orc_f16_bits_to_f32(orc_kv_f32_to_f16_bits(v)); }

ORACLE_API void orc_kv_round_row(const float *x, float *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = kv_f16_round(x[i]);
}

/* ------------------------------------------------------------------ block sizes */

ORACLE_API int64_t orc_row_bytes(int qt, int64_t cols) {
  switch (qt) {
    case QT_Q8_0: return cols / 32 * 34;
    case QT_Q4_K: return cols / 256 * 144;
    case QT_Q6_K: return cols / 256 * 210;
    case QT_F32: return cols * 4;
    default: return -1;
  }
}

/* ------------------------------------------------------------------ dequant */

/* src/tensor/mod.rs:5365-5409 (decode_q8_0_blocks): w = f16->f32(d) * q. */
static void dequant_q8_0_block(const uint8_t *b, float *out) {
  float d = orc_f16_bits_to_f32((uint16_t)(b[0] | (b[1] << 8)));
  for (int j = 0; j < 32; ++j) out[j] = d * (float)(int8_t)b[2 + j];
}

/* src/tensor/mod.rs:5997-6006 (q4_k_scale_min). */
static inline void q4k_scale_min(int idx, const uint8_t *s, uint8_t *sc, uint8_t *m) {
  if (idx < 4) {
    *sc = s[idx] & 63;
    *m = s[idx + 4] & 63;
  } else {
    *sc = (uint8_t)((s[idx + 4] & 0x0f) | ((s[idx - 4] >> 6) << 4));
    *m = (uint8_t)((s[idx + 4] >> 4) | ((s[idx] >> 6) << 4));
  }
}

/* src/tensor/mod.rs:5903-5924 (Q4KBlock::dequantize): (d*sc)*nib - (dmin*m). */
static void dequant_q4_k_block(const uint8_t *b, float *out) {
  float d = orc_f16_bits_to_f32((uint16_t)(b[0] | (b[1] << 8)));
  float dmin = orc_f16_bits_to_f32((uint16_t)(b[2] | (b[3] << 8)));
  const uint8_t *scales = b + 4;
  const uint8_t *qs = b + 16;
  for (int p = 0; p < 4; ++p) {
    uint8_t sc0, m0, sc1, m1;
    q4k_scale_min(2 * p, scales, &sc0, &m0);
    q4k_scale_min(2 * p + 1, scales, &sc1, &m1);
    float ls = d * (float)sc0, hs = d * (float)sc1;
    float lm = dmin * (float)m0, hm = dmin * (float)m1;
    for (int l = 0; l < 32; ++l) {
      uint8_t byte = qs[32 * p + l];
      out[64 * p + l] = ls * (float)(byte & 0x0f) - lm;
      out[64 * p + 32 + l] = hs * (float)(byte >> 4) - hm;
    }
  }
}

/* Signed 6-bit codes of one Q6_K superblock, src/tensor/mod.rs:6039-6066. */
static void q6k_codes(const uint8_t *b, int8_t *a) {
  const uint8_t *ql = b, *qh = b + 128;
  for (int h = 0; h < 2; ++h) {
    for (int l = 0; l < 32; ++l) {
      uint8_t q = qh[32 * h + l];
      a[128 * h + l] = (int8_t)((int)((ql[64 * h + l] & 0x0f) | ((q & 3) << 4)) - 32);
      a[128 * h + l + 32] = (int8_t)((int)((ql[64 * h + l + 32] & 0x0f) | (((q >> 2) & 3) << 4)) - 32);
      a[128 * h + l + 64] = (int8_t)((int)((ql[64 * h + l] >> 4) | (((q >> 4) & 3) << 4)) - 32);
      a[128 * h + l + 96] = (int8_t)((int)((ql[64 * h + l + 32] >> 4) | (((q >> 6) & 3) << 4)) - 32);
    }
  }
}

/* src/tensor/mod.rs:6039-6066 (Q6KBlock::dequantize): (d*sc)*q, left to right. */
static void dequant_q6_k_block(const uint8_t *b, float *out) {
  float d = orc_f16_bits_to_f32((uint16_t)(b[208] | (b[209] << 8)));
  const int8_t *sc = (const int8_t *)(b + 192);
  int8_t a[256];
  q6k_codes(b, a);
  for (int h = 0; h < 2; ++h)
    for (int l = 0; l < 32; ++l) {
      int is = l / 16;
      for (int s = 0; s < 4; ++s) {
        int idx = 128 * h + l + 32 * s;
        out[idx] = d * (float)sc[8 * h + is + 2 * s] * (float)a[idx];
      }
    }
}

ORACLE_API int orc_dequant(int qt, const uint8_t *wire, int64_t n_elements, float *out) {
  switch (qt) {
    case QT_Q8_0:
      for (int64_t b = 0; b < n_elements / 32; ++b) dequant_q8_0_block(wire + b * 34, out + b * 32);
      return 0;
    case QT_Q4_K:
      for (int64_t b = 0; b < n_elements / 256; ++b) dequant_q4_k_block(wire + b * 144, out + b * 256);
      return 0;
    case QT_Q6_K:
      for (int64_t b = 0; b < n_elements / 256; ++b) dequant_q6_k_block(wire + b * 210, out + b * 256);
      return 0;
    case QT_F32:
      memcpy(out, wire, (size_t)n_elements * 4);
      return 0;
    default:
      return -1;
  }
}

/* ------------------------------------------------------------------ weight quantisers */

/* Rust f32::round(): half away from zero == C roundf(). */

/* src/quantize.rs:98-119 (quantize_block_q8_0). */
static void quantize_block_q8_0(const float *src, uint8_t *dst) {
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) {
    float a = fabsf(src[i]);
    if (a > amax) amax = a;
  }
  float d = amax / 127.0f;
  float id = d != 0.0f ? 1.0f / d : 0.0f;
  uint16_t h = orc_f32_to_f16_bits(d);
  dst[0] = (uint8_t)(h & 0xff);
  dst[1] = (uint8_t)(h >> 8);
  for (int i = 0; i < 32; ++i) {
    float x0 = roundf(src[i] * id);
    if (x0 < -128.0f) x0 = -128.0f;
    if (x0 > 127.0f) x0 = 127.0f;
    dst[2 + i] = (uint8_t)(int8_t)x0;
  }
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
/* Rust f32::min/max: the non-NaN operand wins; equal to fminf/fmaxf. */

/* src/quantize.rs:152-244 (quantize_block_q4_k). */
static void quantize_block_q4_k(const float *src, uint8_t *dst) {
  float mins[8], maxs[8];
  for (int g = 0; g < 8; ++g) {
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < 32; ++i) {
      float v = src[32 * g + i];
      if (v < mn) mn = v;
      if (v > mx) mx = v;
    }
    mins[g] = mn;
    maxs[g] = mx;
  }
  float super_min = 0.0f, super_max = 0.0f;
  for (int g = 0; g < 8; ++g) {
    float emin = fminf(mins[g], 0.0f);
    float gs = fmaxf(maxs[g] - emin, 0.0f) / 15.0f;
    if (gs > super_max) super_max = gs;
    float mm = fmaxf(-mins[g], 0.0f);
    if (mm > super_min) super_min = mm;
  }
  float d = super_max / 63.0f, dmin = super_min / 63.0f;
  float id = d != 0.0f ? 1.0f / d : 0.0f;
  float idmin = dmin != 0.0f ? 1.0f / dmin : 0.0f;
  uint16_t dh = orc_f32_to_f16_bits(d), mh = orc_f32_to_f16_bits(dmin);
  dst[0] = (uint8_t)(dh & 0xff); dst[1] = (uint8_t)(dh >> 8);
  dst[2] = (uint8_t)(mh & 0xff); dst[3] = (uint8_t)(mh >> 8);
  uint8_t sc[8], m[8];
  for (int g = 0; g < 8; ++g) {
    float emin = fminf(mins[g], 0.0f);
    float gs = fmaxf(maxs[g] - emin, 0.0f) / 15.0f;
    sc[g] = (uint8_t)clampf(roundf(gs * id), 0.0f, 63.0f);
    m[g] = (uint8_t)clampf(roundf(fmaxf(-mins[g], 0.0f) * idmin), 0.0f, 63.0f);
  }
  uint8_t ps[12];
  memset(ps, 0, 12);
  for (int g = 0; g < 4; ++g) {
    ps[g] = sc[g] & 0x3f;
    ps[g + 4] = m[g] & 0x3f;
  }
  for (int g = 4; g < 8; ++g) {
    ps[g - 4] |= (uint8_t)((sc[g] >> 4) << 6);
    ps[g] |= (uint8_t)((m[g] >> 4) << 6);
    ps[g + 4] = (uint8_t)((sc[g] & 0x0f) | ((m[g] & 0x0f) << 4));
  }
  memcpy(dst + 4, ps, 12);
  uint8_t qv[8][32];
  for (int g = 0; g < 8; ++g) {
    float sub_d = d * (float)sc[g];
    float sub_min = -(dmin * (float)m[g]);
    float sub_id = sub_d != 0.0f ? 1.0f / sub_d : 0.0f;
    for (int i = 0; i < 32; ++i)
      qv[g][i] = (uint8_t)clampf(roundf((src[32 * g + i] - sub_min) * sub_id), 0.0f, 15.0f);
  }
  for (int p = 0; p < 4; ++p)
    for (int i = 0; i < 32; ++i)
      dst[16 + 32 * p + i] = (uint8_t)((qv[2 * p][i] & 0x0f) | (qv[2 * p + 1][i] << 4));
}

/*
 * Q6_K weight quantiser.  The reference ships none (its quantiser emits Q8_0, Q4_0 and
 * Q4_K only, src/quantize.rs:20-25), so this is this project's own definition, written
 * in the style of the reference's Q4_K one: per 16-value group gs = amax/31; d =
 * max(gs)/127 stored as f16; sc = round(gs/d) in [0,127]; q = round(x / (d*sc)) clamped
 * to [-32,31], stored +32 in the Q6_K wire layout that src/tensor/mod.rs:6009-6067
 * decodes.  The CUDA generator repeats it bit-for-bit.
 */
static void quantize_block_q6_k(const float *src, uint8_t *dst) {
  float gs[16];
  float smax = 0.0f;
  for (int j = 0; j < 16; ++j) {
    float amax = 0.0f;
    for (int i = 0; i < 16; ++i) {
      float a = fabsf(src[16 * j + i]);
      if (a > amax) amax = a;
    }
    gs[j] = amax / 31.0f;
    if (gs[j] > smax) smax = gs[j];
  }
  float d = smax / 127.0f;
  float id = d != 0.0f ? 1.0f / d : 0.0f;
  uint16_t dh = orc_f32_to_f16_bits(d);
  int8_t sc[16];
  uint8_t q[256];
  for (int j = 0; j < 16; ++j) {
    sc[j] = (int8_t)clampf(roundf(gs[j] * id), 0.0f, 127.0f);
    float sub_d = d * (float)sc[j];
    float sub_id = sub_d != 0.0f ? 1.0f / sub_d : 0.0f;
    for (int i = 0; i < 16; ++i)
      q[16 * j + i] = (uint8_t)((int)clampf(roundf(src[16 * j + i] * sub_id), -32.0f, 31.0f) + 32);
  }
  memset(dst, 0, 210);
  for (int h = 0; h < 2; ++h)
    for (int l = 0; l < 32; ++l) {
      uint8_t q1 = q[128 * h + l], q2 = q[128 * h + l + 32], q3 = q[128 * h + l + 64], q4 = q[128 * h + l + 96];
      dst[64 * h + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
      dst[64 * h + l + 32] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
      dst[128 + 32 * h + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
  memcpy(dst + 192, sc, 16);
  dst[208] = (uint8_t)(dh & 0xff);
  dst[209] = (uint8_t)(dh >> 8);
}

ORACLE_API int orc_quantize(int qt, const float *src, int64_t n_elements, uint8_t *dst) {
  switch (qt) {
    case QT_Q8_0: {
      int64_t nb = n_elements / 32;
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < nb; ++b) quantize_block_q8_0(src + b * 32, dst + b * 34);
      return 0;
    }
    case QT_Q4_K: {
      int64_t nb = n_elements / 256;
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < nb; ++b) quantize_block_q4_k(src + b * 256, dst + b * 144);
      return 0;
    }
    case QT_Q6_K: {
      int64_t nb = n_elements / 256;
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < nb; ++b) quantize_block_q6_k(src + b * 256, dst + b * 210);
      return 0;
    }
    default:
      return -1;
  }
}

/* ------------------------------------------------------------------ seeded synthetic data */

/*
 * Counter-based generator for the synthetic models: value(seed, stream, index) is a pure
 * function, so any shard is reproducible anywhere.  Hash = splitmix64 finaliser (the
 * mixing the reference's sampler uses, src/inference.rs:9313-9333); the normal deviate is
 * Box-Muller evaluated in double with this file's own log/cos polynomials (only + - * /
 * and sqrt, all correctly rounded), so the CUDA generator, compiled without contraction,
 * reproduces every value bit-for-bit.
 */
static inline uint64_t splitmix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

static inline uint64_t synth_hash(uint64_t seed, uint64_t stream, uint64_t index, uint64_t salt) {
  uint64_t h = splitmix64(seed ^ 0x632be59bd9b4e019ull);
  h = splitmix64(h ^ (stream * 0x9e3779b97f4a7c15ull + salt));
  return splitmix64(h ^ index);
}

/* ln(u) for u in (0,1]: u = m*2^e, m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh(s), s=(m-1)/(m+1). */
static double synth_log(double u) {
  uint64_t b;
  memcpy(&b, &u, 8);
  int e = (int)((b >> 52) & 0x7ff) - 1023;
  b = (b & 0x000fffffffffffffull) | 0x3ff0000000000000ull;
  double m;
  memcpy(&m, &b, 8);
  if (m > 1.4142135623730951) {
    m = m * 0.5;
    e += 1;
  }
  double s = (m - 1.0) / (m + 1.0);
  double s2 = s * s;
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

/* cos(2*pi*t) for t in [0,1): fold to [0,1/8] and use Taylor polynomials. */
static double synth_cos2pi(double t) {
  double sign = 1.0;
  if (t >= 0.5) t = 1.0 - t;      /* cos(2pi t) = cos(2pi(1-t)) */
  if (t > 0.25) {                 /* cos(2pi t) = -cos(2pi(1/2 - t)) */
    t = 0.5 - t;
    sign = -1.0;
  }
  int use_sin = 0;
  if (t > 0.125) {                /* cos(2pi t) = sin(2pi(1/4 - t)) */
    t = 0.25 - t;
    use_sin = 1;
  }
  double x = t * 6.283185307179586;
  double x2 = x * x;
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

static inline float synth_normal(uint64_t seed, uint64_t stream, uint64_t index, float sigma) {
  uint64_t h1 = synth_hash(seed, stream, index, 1);
  uint64_t h2 = synth_hash(seed, stream, index, 2);
  double u1 = ((double)(h1 >> 11) + 1.0) * (1.0 / 9007199254740992.0); /* (0,1] */
  double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);         /* [0,1) */
  double r = sqrt(-2.0 * synth_log(u1));
  double z = r * synth_cos2pi(u2);
  return (float)z * sigma;
}

ORACLE_API void orc_synth_normal(uint64_t seed, uint64_t stream, int64_t start, int64_t n, float sigma, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = synth_normal(seed, stream, (uint64_t)(start + i), sigma);
}

/* Uniform token ids in [0, vocab). */
ORACLE_API void orc_synth_tokens(uint64_t seed, uint64_t stream, int64_t n, int32_t vocab, int32_t *out) {
  for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)(synth_hash(seed, stream, (uint64_t)i, 3) % (uint64_t)vocab);
}

/* Generate rows [row0,row0+rows) of a [*, cols] tensor of N(0,sigma) and quantise to wire. */
ORACLE_API int orc_synth_tensor(int qt, uint64_t seed, uint64_t stream, int64_t row0, int64_t rows, int64_t cols,
                                float sigma, uint8_t *dst) {
  int64_t rb = orc_row_bytes(qt, cols);
  if (rb < 0) return -1;
  int rc = 0;
#pragma omp parallel
  {
    float *tmp = (float *)malloc((size_t)cols * 4);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      for (int64_t c = 0; c < cols; ++c) tmp[c] = synth_normal(seed, stream, (uint64_t)((row0 + r) * cols + c), sigma);
      if (qt == QT_F32) {
        memcpy(dst + r * rb, tmp, (size_t)cols * 4);
      } else {
        int64_t nb = cols / (qt == QT_Q8_0 ? 32 : 256);
        for (int64_t b = 0; b < nb; ++b) {
          if (qt == QT_Q8_0) quantize_block_q8_0(tmp + b * 32, dst + r * rb + b * 34);
          else if (qt == QT_Q4_K) quantize_block_q4_k(tmp + b * 256, dst + r * rb + b * 144);
          else quantize_block_q6_k(tmp + b * 256, dst + r * rb + b * 210);
        }
      }
    }
    free(tmp);
  }
  return rc;
}

/* ------------------------------------------------------------------ activation quantisers */

/* src/inference.rs:22510-22528 (quantize_q8_0_block, non-mac). scales[] receives the
 * f16-rounded scale as f32; the inverse uses the UNROUNDED scale. */
ORACLE_API void orc_quantize_act_q8_0(const float *x, int64_t n, int8_t *qs, float *scales) {
  for (int64_t b = 0; b < n / 32; ++b) {
    const float *blk = x + b * 32;
    float max_abs = 0.0f;
    for (int i = 0; i < 32; ++i) max_abs = fmaxf(max_abs, fabsf(blk[i]));
    float unrounded = max_abs / 127.0f;
    scales[b] = f16_round(unrounded);
    float inv = unrounded == 0.0f ? 0.0f : 1.0f / unrounded;
    for (int i = 0; i < 32; ++i) qs[b * 32 + i] = (int8_t)clampf(roundf(blk[i] * inv), -128.0f, 127.0f);
  }
}

/* src/inference.rs:23112-23116 (nearest_int_reference). */
static inline int32_t nearest_int_reference(float fval) {
  float val = fval + 12582912.0f;
  return (int32_t)(f32_bits(val) & 0x007fffffu) - 0x00400000;
}

/* src/inference.rs:23121-23152 (quantize_q8_k_blocks). */
ORACLE_API void orc_quantize_act_q8_k(const float *x, int64_t n, int8_t *qs, float *d) {
  for (int64_t b = 0; b < n / 256; ++b) {
    const float *blk = x + b * 256;
    float amax = 0.0f, mx = 0.0f;
    for (int i = 0; i < 256; ++i) {
      float a = fabsf(blk[i]);
      if (a > amax) {
        amax = a;
        mx = blk[i];
      }
    }
    if (amax == 0.0f) {
      d[b] = 0.0f;
      memset(qs + b * 256, 0, 256);
      continue;
    }
    float iscale = -127.0f / mx;
    for (int i = 0; i < 256; ++i) {
      int32_t q = nearest_int_reference(iscale * blk[i]);
      if (q > 127) q = 127;
      qs[b * 256 + i] = (int8_t)q;
    }
    d[b] = 1.0f / iscale;
  }
}

/* ------------------------------------------------------------------ row dots */

/* Q8_0 weight (wire, f16 scale) x Q8_0 activation: src/inference.rs:26191-26199 with the
 * wire twin :22729-22745.  term = ((float)isum * w_scale) * x_scale, summed in block order. */
static float q8_0_row_dot(const uint8_t *w, const int8_t *xq, const float *xs, int64_t nb) {
  float sum = 0.0f;
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t *blk = w + b * 34;
    float ws = orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    int32_t isum = 0;
    for (int j = 0; j < 32; ++j) isum += (int32_t)(int8_t)blk[2 + j] * (int32_t)xq[b * 32 + j];
    sum += (float)isum * ws * xs[b];
  }
  return sum;
}

/* Q4_K x Q8_K, production order: src/diffusion_gemma/refmath.rs:504-562 (q4_k_dot_scalar). */
static float q4_k_row_dot(const uint8_t *w, const int8_t *xq, const float *xd, int64_t nsb) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < nsb; ++i) {
    const uint8_t *blk = w + i * 144;
    const int8_t *y = xq + i * 256;
    float d = xd[i] * orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    float dmin = xd[i] * orc_f16_bits_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
    const uint8_t *qs = blk + 16;
    int64_t prod = 0;
    for (int g = 0; g < 8; ++g) {
      uint8_t sc, m;
      q4k_scale_min(g, blk + 4, &sc, &m);
      int32_t bs = 0;
      for (int t = 0; t < 32; ++t) bs += y[32 * g + t];
      prod += (int64_t)bs * (int64_t)m;
    }
    sumf = fmaf(-dmin, (float)prod, sumf);
    int64_t s1 = 0, s2 = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, sc1, m_;
      q4k_scale_min(2 * j, blk + 4, &sc0, &m_);
      q4k_scale_min(2 * j + 1, blk + 4, &sc1, &m_);
      int64_t lo = 0, hi = 0;
      for (int t = 0; t < 32; ++t) {
        lo += (int64_t)(qs[32 * j + t] & 0x0f) * (int64_t)y[64 * j + t];
        hi += (int64_t)(qs[32 * j + t] >> 4) * (int64_t)y[64 * j + 32 + t];
      }
      s1 += lo * sc0;
      s2 += hi * sc1;
    }
    sumf = fmaf(d, (float)(s1 + s2), sumf);
  }
  return sumf;
}

/* Q6_K x Q8_K: src/inference.rs:25535-25581 (q6_k_wire_row_dot). */
static float q6_k_row_dot(const uint8_t *w, const int8_t *xq, const float *xd, int64_t nsb) {
  float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t i = 0; i < nsb; ++i) {
    const uint8_t *blk = w + i * 210;
    const int8_t *y = xq + i * 256;
    float d = orc_f16_bits_to_f32((uint16_t)(blk[208] | (blk[209] << 8))) * xd[i];
    int8_t a[256];
    q6k_codes(blk, a);
    int32_t aux[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 16; ++j) {
      int32_t scale = (int32_t)(int8_t)blk[192 + j];
      for (int l = 0; l < 8; ++l) aux[l] += scale * (int32_t)y[16 * j + l] * (int32_t)a[16 * j + l];
      for (int l = 0; l < 8; ++l) aux[l] += scale * (int32_t)y[16 * j + 8 + l] * (int32_t)a[16 * j + 8 + l];
    }
    for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux[l];
  }
  float r = 0.0f;
  for (int l = 0; l < 8; ++l) r += sums[l];
  return r;
}

/* src/tensor/mod.rs:3464-3480 (dot_product, non-mac): one accumulator, index order. */
static float dot_f32(const float *a, const float *b, int64_t n) {
  float s = 0.0f;
  for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

/* Scratch for one quantised activation row. */
typedef struct {
  int8_t *q;
  float *s;
} act_q;

/*
 * y[r] = W[r] . x for a quantised row-major [rows][cols] matrix in GGUF wire form and an
 * f32 activation row.  The activation is quantised once (Q8_0 for Q8_0 weights, Q8_K for
 * K-quants; src/inference.rs:22058-22204, 23704-23765, 25443-25491) and rows are spread
 * over threads the way the reference spreads them over its rayon pool.
 */
ORACLE_API int orc_matvec(int qt, const uint8_t *w, int64_t rows, int64_t cols, const float *x, float *y) {
  int8_t *xq = (int8_t *)malloc((size_t)cols);
  float *xs = (float *)malloc((size_t)(cols / 32 + 1) * 4);
  int rc = 0;
  if (qt == QT_Q8_0) {
    orc_quantize_act_q8_0(x, cols, xq, xs);
    int64_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q8_0_row_dot(w + r * nb * 34, xq, xs, nb);
  } else if (qt == QT_Q4_K) {
    orc_quantize_act_q8_k(x, cols, xq, xs);
    int64_t nsb = cols / 256;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q4_k_row_dot(w + r * nsb * 144, xq, xs, nsb);
  } else if (qt == QT_Q6_K) {
    orc_quantize_act_q8_k(x, cols, xq, xs);
    int64_t nsb = cols / 256;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q6_k_row_dot(w + r * nsb * 210, xq, xs, nsb);
  } else if (qt == QT_F32) {
    /* f32 weights x f32 activation, sequential dot: src/inference.rs:29382-29409. */
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = dot_f32(x, (const float *)w + r * cols, cols);
  } else {
    rc = -1;
  }
  free(xq);
  free(xs);
  return rc;
}

/* Same, with the activation already quantised by the caller (kernel-level parity). */
ORACLE_API int orc_matvec_quantised(int qt, const uint8_t *w, int64_t rows, int64_t cols, const int8_t *xq,
                                    const float *xs, float *y) {
  if (qt == QT_Q8_0) {
    int64_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q8_0_row_dot(w + r * nb * 34, xq, xs, nb);
  } else if (qt == QT_Q4_K) {
    int64_t nsb = cols / 256;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q4_k_row_dot(w + r * nsb * 144, xq, xs, nsb);
  } else if (qt == QT_Q6_K) {
    int64_t nsb = cols / 256;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) y[r] = q6_k_row_dot(w + r * nsb * 210, xq, xs, nsb);
  } else {
    return -1;
  }
  return 0;
}

/*
 * Mixtral expert matvec: the reference loads non-Q8_0 merged expert tensors as f32
 * (src/inference.rs:832-846) and multiplies with the plain sequential f32 dot
 * (expert_matrix_view else-branch, :14109-14123): dequantise the row, then dot_f32.
 */
ORACLE_API int orc_matvec_dequant_f32(int qt, const uint8_t *w, int64_t rows, int64_t cols, const float *x, float *y) {
  int64_t rb = orc_row_bytes(qt, cols);
  if (rb < 0) return -1;
#pragma omp parallel
  {
    float *tmp = (float *)malloc((size_t)cols * 4);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      orc_dequant(qt, w + r * rb, cols, tmp);
      y[r] = dot_f32(x, tmp, cols);
    }
    free(tmp);
  }
  return 0;
}

/* ------------------------------------------------------------------ per-token ops */

/* src/tensor/mod.rs:2740-2764 (rms_norm_into, non-mac). */
ORACLE_API void orc_rms_norm(const float *x, const float *w, int64_t n, float eps, float *out) {
  float ss = 0.0f;
  for (int64_t i = 0; i < n; ++i) ss += x[i] * x[i];
  float mean_square = ss / (float)n;
  float scale = 1.0f / sqrtf(mean_square + eps);
  for (int64_t i = 0; i < n; ++i) out[i] = x[i] * scale * w[i];
}

/* RoPE table for one position: src/inference/rope.rs:495-560 (scaling None, no rope_freqs)
 * and :600-655 (the table the GPU lane receives). */
ORACLE_API void orc_rope_table(int64_t position, int32_t rope_dim, float base, float *cosv, float *sinv) {
  for (int32_t i = 0; i < rope_dim / 2; ++i) {
    float theta = powf(base, -((float)i * 2.0f) / (float)rope_dim);
    float ang = (float)position * theta;
    sinv[i] = sinf(ang);
    cosv[i] = cosf(ang);
  }
}

/* src/inference/rope.rs:495-530 (apply_rope_to_row, Forward). */
ORACLE_API void orc_rope_apply(float *data, int32_t heads, int32_t head_dim, int32_t rope_dim, const float *cosv,
                               const float *sinv, int32_t split_half) {
  int32_t half = rope_dim / 2;
  for (int32_t p = 0; p < half; ++p) {
    float c = cosv[p], s = sinv[p];
    for (int32_t h = 0; h < heads; ++h) {
      int32_t d0 = split_half ? h * head_dim + p : h * head_dim + 2 * p;
      int32_t d1 = split_half ? d0 + half : d0 + 1;
      float x0 = data[d0], x1 = data[d1];
      data[d0] = (x0 * c) - (x1 * s);
      data[d1] = (x0 * s) + (x1 * c);
    }
  }
}

/*
 * One query head over an f16-exact KV history: src/inference.rs:30297-30466 (F32 lane,
 * non-blocked dot).  k/v point at this kv-head's rows, consecutive positions `stride`
 * floats apart.
 */
ORACLE_API int orc_attention_head(const float *q, const float *k, const float *v, int64_t stride, int64_t n_pos,
                                  int32_t head_dim, float scale, float *out, float *scores) {
  for (int64_t p = 0; p < n_pos; ++p) scores[p] = dot_f32(q, k + p * stride, head_dim) * scale;
  float mx = -INFINITY;
  for (int64_t p = 0; p < n_pos; ++p) mx = fmaxf(mx, scores[p]);
  float sum = 0.0f;
  for (int64_t p = 0; p < n_pos; ++p) {
    scores[p] = expf(scores[p] - mx);
    sum += scores[p];
  }
  if (sum == 0.0f || !isfinite(sum)) return -1;
  float inv = 1.0f / sum;
  for (int32_t d = 0; d < head_dim; ++d) out[d] = 0.0f;
  for (int64_t p = 0; p < n_pos; ++p) {
    float prob = scores[p] * inv;
    const float *vr = v + p * stride;
    for (int32_t d = 0; d < head_dim; ++d) out[d] += prob * vr[d];
  }
  return 0;
}

/* The expf algorithm the CUDA library restates (camelid_b200/csrc/expf_exact.cuh), written the same
 * way in C so that a CPU test can compare it with this machine's libm expf over many inputs. */
ORACLE_API float orc_expf_twin(float x) {
  static const uint64_t T[32] = {
      0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
      0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
      0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
      0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
      0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
      0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
      0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
      0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};
  if (x != x) return x;
  if (x > 0x1.62e42ep6f) return INFINITY;
  if (x < -0x1.9fe368p6f) return 0.0f;
  double xd = (double)x;
  double z = (0x1.71547652b82fep+0 * 32.0) * xd;
  double kd = z + 0x1.8p+52;
  uint64_t ki;
  memcpy(&ki, &kd, 8);
  kd = kd - 0x1.8p+52;
  double r = z - kd;
  uint64_t t = T[ki & 31] + (ki << 47);
  double s;
  memcpy(&s, &t, 8);
  double zz = (0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0) * r + 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
  double r2 = r * r;
  double y = (0x1.62e42ff0c52d6p-1 / 32.0) * r + 1.0;
  y = zz * r2 + y;
  y = y * s;
  return (float)y;
}

/* Count of inputs in [lo, hi] (n evenly spaced floats) where the twin and libm expf differ. */
ORACLE_API int64_t orc_expf_twin_mismatches(float lo, float hi, int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) {
    float x = lo + (hi - lo) * (float)((double)i / (double)(n - 1));
    float a = orc_expf_twin(x), b = expf(x);
    if (f32_bits(a) != f32_bits(b)) ++bad;
  }
  return bad;
}

/* src/inference.rs:13231-13236 (SwiGLU line). */
ORACLE_API void orc_silu_mul(const float *g, const float *u, int64_t n, float *out) {
  for (int64_t i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}

/* src/inference.rs:8904-8917 (greedy_sample): strict >, first index wins. */
ORACLE_API int32_t orc_argmax(const float *x, int64_t n) {
  int64_t best = 0;
  float bv = x[0];
  for (int64_t i = 1; i < n; ++i)
    if (x[i] > bv) {
      bv = x[i];
      best = i;
    }
  return (int32_t)best;
}

/* total_cmp order on f32 (Rust f32::total_cmp). */
static inline int32_t total_key(float f) {
  int32_t b = (int32_t)f32_bits(f);
  return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

/* src/inference.rs:13940-13991 (softmax_top_k): sort (value desc, idx asc), keep k,
 * softmax over the kept, re-sort (weight desc, idx asc). */
ORACLE_API int orc_softmax_top_k(const float *logits, int32_t n, int32_t k, int32_t *idx_out, float *w_out) {
  if (n <= 0 || k <= 0) return 0;
  int32_t *order = (int32_t *)malloc((size_t)n * 4);
  for (int32_t i = 0; i < n; ++i) order[i] = i;
  /* stable insertion sort: value descending (total order), index ascending */
  for (int32_t i = 1; i < n; ++i) {
    int32_t cur = order[i];
    int32_t j = i - 1;
    while (j >= 0 && (total_key(logits[order[j]]) < total_key(logits[cur]))) {
      order[j + 1] = order[j];
      --j;
    }
    order[j + 1] = cur;
  }
  int32_t kk = k < n ? k : n;
  float mx = -INFINITY;
  for (int32_t i = 0; i < kk; ++i) mx = fmaxf(mx, logits[order[i]]);
  float sum = 0.0f;
  for (int32_t i = 0; i < kk; ++i) {
    float v = logits[order[i]];
    w_out[i] = isfinite(v) ? expf(v - mx) : 0.0f;
    idx_out[i] = order[i];
    sum += w_out[i];
  }
  if (sum > 0.0f) {
    for (int32_t i = 0; i < kk; ++i) w_out[i] /= sum;
  } else {
    for (int32_t i = 0; i < kk; ++i) w_out[i] = 1.0f / (float)kk;
  }
  for (int32_t i = 1; i < kk; ++i) {
    int32_t ci = idx_out[i];
    float cw = w_out[i];
    int32_t j = i - 1;
    while (j >= 0 && (total_key(w_out[j]) < total_key(cw) || (total_key(w_out[j]) == total_key(cw) && idx_out[j] > ci))) {
      idx_out[j + 1] = idx_out[j];
      w_out[j + 1] = w_out[j];
      --j;
    }
    idx_out[j + 1] = ci;
    w_out[j + 1] = cw;
  }
  free(order);
  return kk;
}

/* ------------------------------------------------------------------ Q8_0 KV cache (src/tensor/kv_quant.rs, scalar path) */

/* quantize_block_q8_0 (:123-143): d = amax/127, id = 1/d, q = clamp(round_half_away(x*id), -127, 127); the stored scale
 * is f16(d).  codes[32] receive the int8 codes as floats; returns the f16-rounded scale as f32. */
ORACLE_API float orc_kv_q8_0_quantize_block(const float *src, float *codes) {
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) {
    float a = fabsf(src[i]);
    if (a > amax) amax = a;
  }
  float d = amax / 127.0f;
  float id = d != 0.0f ? 1.0f / d : 0.0f;
  for (int i = 0; i < 32; ++i) {
    float v = roundf(src[i] * id);
    if (v < -127.0f) v = -127.0f;
    if (v > 127.0f) v = 127.0f;
    codes[i] = (float)(int8_t)v;
  }
  return orc_f16_bits_to_f32(orc_f32_to_f16_bits(d));
}

/* One head over a Q8_0 cache: score = (sum over blocks of (sum_i q_i * code_i) * d) * scale (vec_dot_row_q8_0, :180-201,
 * scalar form), the softmax of attention_context_for_head (src/inference.rs:30287-30466), then per position
 * out_i = fma(prob * d, code_i, out_i) (axpy_row_q8_0, :203-221).  kq/vq: codes as floats, rows `stride` apart;
 * kd/vd: block scales, rows `sstride` apart. */
ORACLE_API int orc_attention_head_q8(const float *q, const float *kq, const float *kd, const float *vq, const float *vd,
                                     int64_t stride, int64_t sstride, int64_t n_pos, int32_t head_dim, float scale, float *out,
                                     float *scores) {
  int32_t nb = head_dim / 32;
  for (int64_t p = 0; p < n_pos; ++p) {
    float total = 0.0f;
    for (int32_t b = 0; b < nb; ++b) {
      float sum = 0.0f;
      for (int32_t i = 0; i < 32; ++i) sum += q[b * 32 + i] * kq[p * stride + b * 32 + i];
      total += sum * kd[p * sstride + b];
    }
    scores[p] = total * scale;
  }
  float mx = -INFINITY;
  for (int64_t p = 0; p < n_pos; ++p) mx = fmaxf(mx, scores[p]);
  float sum = 0.0f;
  for (int64_t p = 0; p < n_pos; ++p) {
    scores[p] = expf(scores[p] - mx);
    sum += scores[p];
  }
  if (sum == 0.0f || !isfinite(sum)) return -1;
  float inv = 1.0f / sum;
  for (int32_t d = 0; d < head_dim; ++d) out[d] = 0.0f;
  for (int64_t p = 0; p < n_pos; ++p) {
    float prob = scores[p] * inv;
    for (int32_t b = 0; b < nb; ++b) {
      float pd = prob * vd[p * sstride + b];
      for (int32_t i = 0; i < 32; ++i) out[b * 32 + i] = fmaf(pd, vq[p * stride + b * 32 + i], out[b * 32 + i]);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ sampling (src/cuda_resident/sampling.cuh) */

/* sampling_uniform_from_u24 + splitmix_uniform: 24 hashed bits of (seed, index) as a float in (0, 1). */
ORACLE_API float orc_sample_uniform(uint64_t seed, uint32_t idx) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ULL * (uint64_t)(idx + 1u);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z = z ^ (z >> 31);
  uint32_t m = (uint32_t)(z >> 40);
  float u = ((float)m + 0.5f) / 16777216.0f;
  return u < 0.999999940395355224609375f ? u : 0.999999940395355224609375f;
}

/* How many of the 2^24 mantissas the clamp of sampling_uniform_from_u24 changes (the reference's host test expects
 * exactly one: "uniform 16777216 changed 1", src/inference/cuda_min_p_host_tests.rs:228). */
ORACLE_API int32_t orc_sample_uniform_clamped_count(void) {
  int32_t changed = 0;
  for (uint32_t m = 0; m < (1u << 24); ++m) {
    float u = ((float)m + 0.5f) / 16777216.0f;
    if (u >= 1.0f || u != (u < 0.999999940395355224609375f ? u : 0.999999940395355224609375f)) ++changed;
  }
  return changed;
}

/* min_p_candidate: 1 keep, 0 drop, -1 undecided. */
ORACLE_API int32_t orc_min_p_candidate(float logit, float max_logit, float min_p, int32_t n) {
  if (n <= 0 || !isfinite(logit) || !isfinite(max_logit) || !isfinite(min_p) || min_p <= 0.0f || min_p >= 1.0f ||
      min_p < (4.0f * 1.1754943508222875e-38f) * (float)n)
    return -1;
  float ratio = expf(logit - max_logit);
  float margin = (64.0f * 1.1920928955078125e-7f) * min_p;
  if (!isfinite(ratio) || fabsf(ratio - min_p) <= margin) return -1;
  return ratio > min_p ? 1 : 0;
}

/* sample_gumbel: argmax_i(logit_i * inv_temp - log(-log(u_i))), lower index on ties.  scores (optional) receives every
 * token's score, for tolerance checks of a device draw. */
ORACLE_API int32_t orc_sample_gumbel(const float *logits, int32_t n, float inv_temp, uint64_t seed, float *scores) {
  float best = -3.4e38f;
  int32_t besti = 0;
  for (int32_t i = 0; i < n; ++i) {
    float g = -logf(-logf(orc_sample_uniform(seed, (uint32_t)i)));
    float v = logits[i] * inv_temp + g;
    if (scores) scores[i] = v;
    if (v > best) { best = v; besti = i; }
  }
  return besti;
}

/* sample_gumbel_filtered: min-p filter, then the draw over the kept tokens; -1 = hand the row to the CPU sampler. */
ORACLE_API int32_t orc_sample_gumbel_filtered(const float *logits, int32_t n, float temperature, float min_p, uint64_t seed,
                                              float *scores) {
  float maximum = -INFINITY;
  int bad = n <= 0;
  for (int32_t i = 0; i < n; ++i) {
    if (!isfinite(logits[i])) bad = 1;
    else if (logits[i] > maximum) maximum = logits[i];
  }
  if (!isfinite(temperature) || temperature <= 0.0f) bad = 1;
  float best = -INFINITY;
  int32_t besti = 0x7fffffff;
  for (int32_t i = 0; i < n; ++i) {
    if (scores) scores[i] = -INFINITY;
    int32_t keep = orc_min_p_candidate(logits[i], maximum, min_p, n);
    if (keep < 0) bad = 1;
    if (keep == 1) {
      float g = -logf(-logf(orc_sample_uniform(seed, (uint32_t)i)));
      float score = (logits[i] / temperature) - (maximum / temperature) + g;
      if (!isfinite(score)) bad = 1;
      if (scores) scores[i] = score;
      if (score > best || (score == best && i < besti)) { best = score; besti = i; }
    }
  }
  return (bad || besti == 0x7fffffff) ? -1 : besti;
}

/* ------------------------------------------------------------------ model forward */

typedef struct {
  int32_t qt;
  const uint8_t *data; /* GGUF wire bytes, row-major [rows][cols] */
  int64_t rows, cols;
} orc_tensor;

typedef struct {
  orc_tensor q, k, v, o, gate, up, down;
  const float *attn_norm, *ffn_norm;
  /* Mixtral: router f32 [n_expert][hidden]; expert slabs are [n_expert] consecutive
   * [rows][cols] matrices (src/inference.rs:14032-14035, 14110-14111). */
  const float *router;
  orc_tensor gate_exps, up_exps, down_exps;
} orc_layer;

typedef struct {
  int32_t n_layers, n_heads, n_kv_heads, head_dim, hidden, ffn_dim, rope_dim, max_pos, vocab;
  float eps, rope_base;
  int32_t split_half, n_experts, n_experts_used;
  orc_layer *layers;
  orc_tensor token_embd, output;
  const float *final_norm;
  float *kcache, *vcache; /* [layer][kv_head][max_pos][head_dim], f16-exact f32 */
  int32_t kv_q8;          /* KV cache held as Q8_0 blocks (src/tensor/kv_quant.rs): kcache/vcache then hold the int8 codes as
                             floats and kscale/vscale the f16-rounded block scales */
  float *kscale, *vscale; /* [layer][kv_head][max_pos][head_dim/32] */
  float *rope_freq;       /* optional per-pair frequencies (rope_pair_frequency, src/inference/rope.rs:532); NULL = base^(-2i/d) */
} orc_model;

ORACLE_API orc_model *orc_model_create(int32_t n_layers, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                       int32_t hidden, int32_t ffn_dim, int32_t rope_dim, int32_t max_pos,
                                       int32_t vocab, float eps, float rope_base, int32_t split_half,
                                       int32_t n_experts, int32_t n_experts_used) {
  orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
  m->n_layers = n_layers; m->n_heads = n_heads; m->n_kv_heads = n_kv_heads; m->head_dim = head_dim;
  m->hidden = hidden; m->ffn_dim = ffn_dim; m->rope_dim = rope_dim; m->max_pos = max_pos; m->vocab = vocab;
  m->eps = eps; m->rope_base = rope_base; m->split_half = split_half;
  m->n_experts = n_experts; m->n_experts_used = n_experts_used;
  m->layers = (orc_layer *)calloc((size_t)n_layers, sizeof(orc_layer));
  size_t kv = (size_t)n_layers * n_kv_heads * max_pos * head_dim;
  m->kcache = (float *)calloc(kv, 4);
  m->vcache = (float *)calloc(kv, 4);
  return m;
}

ORACLE_API void orc_model_destroy(orc_model *m) {
  if (!m) return;
  free(m->layers); free(m->kcache); free(m->vcache); free(m->kscale); free(m->vscale); free(m->rope_freq); free(m);
}

static orc_tensor mk_tensor(int32_t qt, const uint8_t *data, int64_t rows, int64_t cols) {
  orc_tensor t; t.qt = qt; t.data = data; t.rows = rows; t.cols = cols; return t;
}

/* Switches the model's KV cache to Q8_0 blocks (before the first forward). */
ORACLE_API int orc_model_set_kv_q8(orc_model *m, int32_t on) {
  if (m->head_dim % 32) return -1;
  m->kv_q8 = on ? 1 : 0;
  if (on && !m->kscale) {
    size_t n = (size_t)m->n_layers * m->n_kv_heads * m->max_pos * (m->head_dim / 32);
    m->kscale = (float *)calloc(n, 4);
    m->vscale = (float *)calloc(n, 4);
  }
  return 0;
}

/* Per-pair RoPE frequencies for models with rope_freqs.weight or scaled RoPE (copied). */
ORACLE_API int orc_model_set_rope_frequencies(orc_model *m, const float *freq, int32_t n) {
  if (n != m->rope_dim / 2) return -1;
  free(m->rope_freq);
  m->rope_freq = (float *)malloc((size_t)n * 4);
  memcpy(m->rope_freq, freq, (size_t)n * 4);
  return 0;
}

/* The llama3 wavelength-dependent scaling of one frequency (llama3_scaled_rope_frequency, src/inference/rope.rs:733-757). */
ORACLE_API float orc_rope_llama3_frequency(float frequency, float factor, float original_context, float low_freq_factor,
                                           float high_freq_factor) {
  float wavelength = (2.0f * 3.14159265358979323846f) / frequency;
  float low_w = original_context / low_freq_factor, high_w = original_context / high_freq_factor;
  if (wavelength < high_w) return frequency;
  if (wavelength > low_w) return frequency / factor;
  float smooth = (original_context / wavelength - low_freq_factor) / (high_freq_factor - low_freq_factor);
  return ((1.0f - smooth) * frequency / factor) + (smooth * frequency);
}

/* Pointers are borrowed: the caller keeps the buffers alive. slot: 0..6 = q,k,v,o,gate,up,down. */
ORACLE_API int orc_model_set_proj(orc_model *m, int32_t layer, int32_t slot, int32_t qt, const uint8_t *data) {
  if (layer < 0 || layer >= m->n_layers) return -1;
  orc_layer *L = &m->layers[layer];
  int64_t qw = (int64_t)m->n_heads * m->head_dim, kvw = (int64_t)m->n_kv_heads * m->head_dim;
  switch (slot) {
    case 0: L->q = mk_tensor(qt, data, qw, m->hidden); break;
    case 1: L->k = mk_tensor(qt, data, kvw, m->hidden); break;
    case 2: L->v = mk_tensor(qt, data, kvw, m->hidden); break;
    case 3: L->o = mk_tensor(qt, data, m->hidden, qw); break;
    case 4: L->gate = mk_tensor(qt, data, m->ffn_dim, m->hidden); break;
    case 5: L->up = mk_tensor(qt, data, m->ffn_dim, m->hidden); break;
    case 6: L->down = mk_tensor(qt, data, m->hidden, m->ffn_dim); break;
    default: return -1;
  }
  return 0;
}

ORACLE_API int orc_model_set_norms(orc_model *m, int32_t layer, const float *attn_norm, const float *ffn_norm) {
  if (layer < 0 || layer >= m->n_layers) return -1;
  m->layers[layer].attn_norm = attn_norm;
  m->layers[layer].ffn_norm = ffn_norm;
  return 0;
}

ORACLE_API int orc_model_set_moe(orc_model *m, int32_t layer, const float *router, int32_t qt_gate,
                                 const uint8_t *gate, int32_t qt_up, const uint8_t *up, int32_t qt_down,
                                 const uint8_t *down) {
  if (layer < 0 || layer >= m->n_layers) return -1;
  orc_layer *L = &m->layers[layer];
  L->router = router;
  L->gate_exps = mk_tensor(qt_gate, gate, m->ffn_dim, m->hidden);
  L->up_exps = mk_tensor(qt_up, up, m->ffn_dim, m->hidden);
  L->down_exps = mk_tensor(qt_down, down, m->hidden, m->ffn_dim);
  return 0;
}

ORACLE_API void orc_model_set_output(orc_model *m, const float *final_norm, int32_t qt, const uint8_t *data) {
  m->final_norm = final_norm;
  m->output = mk_tensor(qt, data, m->vocab, m->hidden);
}

ORACLE_API void orc_model_set_token_embd(orc_model *m, int32_t qt, const uint8_t *data) {
  m->token_embd = mk_tensor(qt, data, m->vocab, m->hidden);
}

/* K and V rows of one layer as [kv_head][n_pos][head_dim] (the layout of the reference's
 * read_kv_layer, src/cuda_resident.rs:17448). */
ORACLE_API int orc_model_read_kv(const orc_model *m, int32_t layer, int64_t n_pos, float *ck, float *cv) {
  if (layer < 0 || layer >= m->n_layers || n_pos < 0 || n_pos > m->max_pos) return -1;
  int32_t hd = m->head_dim;
  const float *kc = m->kcache + (size_t)layer * m->n_kv_heads * m->max_pos * hd;
  const float *vc = m->vcache + (size_t)layer * m->n_kv_heads * m->max_pos * hd;
  for (int32_t kh = 0; kh < m->n_kv_heads; ++kh) {
    memcpy(ck + (size_t)kh * n_pos * hd, kc + (size_t)kh * m->max_pos * hd, (size_t)n_pos * hd * 4);
    memcpy(cv + (size_t)kh * n_pos * hd, vc + (size_t)kh * m->max_pos * hd, (size_t)n_pos * hd * 4);
  }
  return 0;
}

/* The inverse of orc_model_read_kv: positions 0..n_pos-1 of one layer's cache take the given rows,
 * rounded to f16 like rows the forward pass stores (the reference's seed_layer, src/cuda_resident.rs:17355:
 * a test hook that plants a KV prefix before decoding). */
ORACLE_API int orc_model_write_kv(orc_model *m, int32_t layer, int64_t n_pos, const float *ck, const float *cv) {
  if (layer < 0 || layer >= m->n_layers || n_pos < 0 || n_pos > m->max_pos) return -1;
  int32_t hd = m->head_dim;
  float *kc = m->kcache + (size_t)layer * m->n_kv_heads * m->max_pos * hd;
  float *vc = m->vcache + (size_t)layer * m->n_kv_heads * m->max_pos * hd;
  for (int32_t kh = 0; kh < m->n_kv_heads; ++kh)
    for (int64_t i = 0; i < n_pos * hd; ++i) {
      kc[(size_t)kh * m->max_pos * hd + i] = kv_f16_round(ck[(size_t)kh * n_pos * hd + i]);
      vc[(size_t)kh * m->max_pos * hd + i] = kv_f16_round(cv[(size_t)kh * n_pos * hd + i]);
    }
  return 0;
}

/* src/tensor/mod.rs:2899-3216 (embedding_lookup): dequantise one row. */
ORACLE_API int orc_embedding(const orc_model *m, int32_t token, float *out) {
  if (token < 0 || token >= m->vocab || !m->token_embd.data) return -1;
  int64_t rb = orc_row_bytes(m->token_embd.qt, m->hidden);
  return orc_dequant(m->token_embd.qt, m->token_embd.data + (int64_t)token * rb, m->hidden, out);
}

static int tensor_matvec(const orc_tensor *t, const float *x, float *y) {
  return orc_matvec(t->qt, t->data, t->rows, t->cols, x, y);
}

/* src/inference.rs:14142-14280 (mixtral_moe_ffn), one row. */
static int moe_ffn(const orc_model *m, const orc_layer *L, const float *x, float *out) {
  int32_t ne = m->n_experts, k = m->n_experts_used;
  int64_t hidden = m->hidden, ff = m->ffn_dim;
  float *logits = (float *)malloc((size_t)ne * 4);
  orc_matvec(QT_F32, (const uint8_t *)L->router, ne, hidden, x, logits);
  int32_t *sel = (int32_t *)malloc((size_t)k * 4);
  float *wts = (float *)malloc((size_t)k * 4);
  int32_t kk = orc_softmax_top_k(logits, ne, k, sel, wts);
  float *g = (float *)malloc((size_t)ff * 4), *u = (float *)malloc((size_t)ff * 4), *act = (float *)malloc((size_t)ff * 4);
  float *eo = (float *)malloc((size_t)hidden * 4);
  for (int64_t c = 0; c < hidden; ++c) out[c] = 0.0f;
  int64_t gb = orc_row_bytes(L->gate_exps.qt, hidden) * ff, ub = orc_row_bytes(L->up_exps.qt, hidden) * ff;
  int64_t db = orc_row_bytes(L->down_exps.qt, ff) * hidden;
  for (int32_t s = 0; s < kk; ++s) {
    int32_t e = sel[s];
    orc_matvec_dequant_f32(L->gate_exps.qt, L->gate_exps.data + e * gb, ff, hidden, x, g);
    orc_matvec_dequant_f32(L->up_exps.qt, L->up_exps.data + e * ub, ff, hidden, x, u);
    orc_silu_mul(g, u, ff, act);
    orc_matvec_dequant_f32(L->down_exps.qt, L->down_exps.data + e * db, hidden, ff, act, eo);
    for (int64_t c = 0; c < hidden; ++c) out[c] += eo[c] * wts[s];
  }
  free(logits); free(sel); free(wts); free(g); free(u); free(act); free(eo);
  return 0;
}

/*
 * One decode step (src/inference.rs:9419-10199 forward_layer_timed, 6411-6669).
 * x_in: the token's embedding row [hidden]; position: zero-based.  Writes the KV rows at
 * `position`.  logits may be NULL.  taps, if non-NULL, receives the residual stream after
 * every layer: [n_layers][hidden].  hidden_out, if non-NULL, the final (pre-norm) hidden.
 */
ORACLE_API int orc_forward(orc_model *m, const float *x_in, int64_t position, float *logits, float *hidden_out,
                           float *taps) {
  if (position < 0 || position >= m->max_pos) return -1;
  int64_t hidden = m->hidden, qw = (int64_t)m->n_heads * m->head_dim, kvw = (int64_t)m->n_kv_heads * m->head_dim;
  int64_t ff = m->ffn_dim;
  int32_t hd = m->head_dim;
  float *h = (float *)malloc((size_t)hidden * 4), *normed = (float *)malloc((size_t)hidden * 4);
  float *q = (float *)malloc((size_t)qw * 4), *k = (float *)malloc((size_t)kvw * 4), *v = (float *)malloc((size_t)kvw * 4);
  float *ctx = (float *)malloc((size_t)qw * 4), *delta = (float *)malloc((size_t)hidden * 4);
  float *g = (float *)malloc((size_t)ff * 4), *u = (float *)malloc((size_t)ff * 4), *act = (float *)malloc((size_t)ff * 4);
  float *cosv = (float *)malloc((size_t)m->rope_dim * 2), *sinv = (float *)malloc((size_t)m->rope_dim * 2);
  float *scores = (float *)malloc((size_t)(position + 1) * 4);
  memcpy(h, x_in, (size_t)hidden * 4);
  if (m->rope_freq) {
    /* angle = position * frequency, then sin/cos (apply_rope_to_row, src/inference/rope.rs:500-502) */
    for (int32_t i = 0; i < m->rope_dim / 2; ++i) {
      float ang = (float)position * m->rope_freq[i];
      sinv[i] = sinf(ang);
      cosv[i] = cosf(ang);
    }
  } else {
    orc_rope_table(position, m->rope_dim, m->rope_base, cosv, sinv);
  }
  float scale = 1.0f / sqrtf((float)hd); /* src/inference/diagnostic_config.rs:300-317 */
  int group = m->n_heads / m->n_kv_heads;
  int rc = 0;
  for (int32_t li = 0; li < m->n_layers && rc == 0; ++li) {
    orc_layer *L = &m->layers[li];
    orc_rms_norm(h, L->attn_norm, hidden, m->eps, normed);
    tensor_matvec(&L->q, normed, q);
    tensor_matvec(&L->k, normed, k);
    tensor_matvec(&L->v, normed, v);
    orc_rope_apply(q, m->n_heads, hd, m->rope_dim, cosv, sinv, m->split_half);
    orc_rope_apply(k, m->n_kv_heads, hd, m->rope_dim, cosv, sinv, m->split_half);
    float *kc = m->kcache + (size_t)li * m->n_kv_heads * m->max_pos * hd;
    float *vc = m->vcache + (size_t)li * m->n_kv_heads * m->max_pos * hd;
    int32_t nb = hd / 32;
    float *ks = m->kv_q8 ? m->kscale + (size_t)li * m->n_kv_heads * m->max_pos * nb : NULL;
    float *vs = m->kv_q8 ? m->vscale + (size_t)li * m->n_kv_heads * m->max_pos * nb : NULL;
    if (m->kv_q8) {
      for (int32_t kh = 0; kh < m->n_kv_heads; ++kh)
        for (int32_t b = 0; b < nb; ++b) {
          size_t row = (size_t)kh * m->max_pos + position;
          ks[row * nb + b] = orc_kv_q8_0_quantize_block(k + kh * hd + b * 32, kc + row * hd + b * 32);
          vs[row * nb + b] = orc_kv_q8_0_quantize_block(v + kh * hd + b * 32, vc + row * hd + b * 32);
        }
      for (int32_t hh = 0; hh < m->n_heads && rc == 0; ++hh) {
        size_t h0 = (size_t)(hh / group) * m->max_pos;
        rc = orc_attention_head_q8(q + hh * hd, kc + h0 * hd, ks + h0 * nb, vc + h0 * hd, vs + h0 * nb, hd, nb, position + 1, hd,
                                   scale, ctx + hh * hd, scores);
      }
    } else {
    for (int32_t kh = 0; kh < m->n_kv_heads; ++kh)
      for (int32_t d = 0; d < hd; ++d) {
        kc[((size_t)kh * m->max_pos + position) * hd + d] = kv_f16_round(k[kh * hd + d]);
        vc[((size_t)kh * m->max_pos + position) * hd + d] = kv_f16_round(v[kh * hd + d]);
      }
    }
    if (m->kv_q8) {
      /* done above */
    } else if (position == 0) {
      /* single cached position: the context is a copy of V (src/inference.rs:29858-29951) */
      for (int32_t hh = 0; hh < m->n_heads; ++hh)
        memcpy(ctx + hh * hd, vc + ((size_t)(hh / group) * m->max_pos) * hd, (size_t)hd * 4);
    } else {
      for (int32_t hh = 0; hh < m->n_heads && rc == 0; ++hh) {
        int32_t kh = hh / group;
        rc = orc_attention_head(q + hh * hd, kc + (size_t)kh * m->max_pos * hd, vc + (size_t)kh * m->max_pos * hd,
                                hd, position + 1, hd, scale, ctx + hh * hd, scores);
      }
    }
    tensor_matvec(&L->o, ctx, delta);
    for (int64_t i = 0; i < hidden; ++i) h[i] = h[i] + delta[i];
    orc_rms_norm(h, L->ffn_norm, hidden, m->eps, normed);
    if (L->router) {
      moe_ffn(m, L, normed, delta);
    } else {
      tensor_matvec(&L->gate, normed, g);
      tensor_matvec(&L->up, normed, u);
      orc_silu_mul(g, u, ff, act);
      tensor_matvec(&L->down, act, delta);
    }
    for (int64_t i = 0; i < hidden; ++i) h[i] = h[i] + delta[i];
    if (taps) memcpy(taps + (size_t)li * hidden, h, (size_t)hidden * 4);
  }
  if (hidden_out) memcpy(hidden_out, h, (size_t)hidden * 4);
  if (logits && rc == 0) {
    orc_rms_norm(h, m->final_norm, hidden, m->eps, normed);
    tensor_matvec(&m->output, normed, logits);
  }
  free(h); free(normed); free(q); free(k); free(v); free(ctx); free(delta); free(g); free(u); free(act);
  free(cosv); free(sinv); free(scores);
  return rc;
}

/* Greedy generation from token ids: prompt positions then n_gen tokens; returns ids. */
static float top2_gap(const float *x, int64_t n) {
  float a = -INFINITY, b = -INFINITY;
  for (int64_t i = 0; i < n; ++i) {
    if (x[i] > a) { b = a; a = x[i]; }
    else if (x[i] > b) b = x[i];
  }
  return a - b;
}

/* gaps, if non-NULL, receives for every generated token the difference between the largest
 * and second-largest logit it was chosen from (how close the greedy choice was to a tie). */
ORACLE_API int orc_generate_gaps(orc_model *m, const int32_t *prompt, int32_t n_prompt, int32_t n_gen, int64_t start_pos,
                                 int32_t *out_tokens, float *last_logits, float *gaps);

ORACLE_API int orc_generate(orc_model *m, const int32_t *prompt, int32_t n_prompt, int32_t n_gen, int64_t start_pos,
                            int32_t *out_tokens, float *last_logits) {
  return orc_generate_gaps(m, prompt, n_prompt, n_gen, start_pos, out_tokens, last_logits, NULL);
}

ORACLE_API int orc_generate_gaps(orc_model *m, const int32_t *prompt, int32_t n_prompt, int32_t n_gen, int64_t start_pos,
                                 int32_t *out_tokens, float *last_logits, float *gaps) {
  float *emb = (float *)malloc((size_t)m->hidden * 4);
  float *logits = (float *)malloc((size_t)m->vocab * 4);
  int64_t pos = start_pos;
  int rc = 0;
  int32_t tok = 0;
  for (int32_t i = 0; i < n_prompt && rc == 0; ++i) {
    rc = orc_embedding(m, prompt[i], emb);
    if (rc) break;
    rc = orc_forward(m, emb, pos++, i + 1 == n_prompt ? logits : NULL, NULL, NULL);
  }
  for (int32_t i = 0; i < n_gen && rc == 0; ++i) {
    tok = orc_argmax(logits, m->vocab);
    out_tokens[i] = tok;
    if (gaps) gaps[i] = top2_gap(logits, m->vocab);
    if (i + 1 == n_gen) break;
    rc = orc_embedding(m, tok, emb);
    if (rc) break;
    rc = orc_forward(m, emb, pos++, logits, NULL, NULL);
  }
  if (last_logits) memcpy(last_logits, logits, (size_t)m->vocab * 4);
  free(emb); free(logits);
  return rc;
}

ORACLE_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORACLE_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
