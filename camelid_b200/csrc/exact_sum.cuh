// Sequential f32 sum of non-negative terms, computed in parallel with the sequential sum's bits.
//
// Camelid's CPU path adds the squares of RMSNorm (rms_norm_into, src/tensor/mod.rs:2740-2764) and
// the softmax weights of attention (src/inference.rs:30297-30466) one after another into a single
// f32 accumulator.  A tree sum differs from that in the last bits, and because the result feeds an
// int8 quantiser the difference can flip a code.  A 4096-long dependent chain of additions costs
// ~8 us on the GPU; this file gets the same bits in about one.
//
// Idea.  All terms are >= 0, so the running sum s never decreases.  While s stays inside one binade
// [2^e, 2^(e+1)) it is an integer multiple S of u = 2^(e-23), and round-to-nearest addition of a
// term t is  S <- S + round(t/u)  — an integer addition, except for exact ties (t/u = k + 1/2),
// which go to the even neighbour and therefore depend on the parity of S only.  So a run of terms
// that keeps s inside one binade acts on S as a pair of increments (d0, d1): S + d0 if S is even,
// S + d1 if S is odd, and such pairs compose associatively.
//
// Procedure.  Items are groups of 8 consecutive terms.  A double-precision prefix sum predicts each
// item's binade.  Items whose predicted binade does not change across them are "fast": a lane
// computes their (d0, d1) under that binade.  The other items (the few where the sum crosses into a
// new binade, and the very first) are "slow".  Runs of fast items with the same binade inside a
// 256-term chunk are composed with a warp scan.  Finally one thread walks the events (run ends and
// slow items) in order with the exact s: a run is applied in O(1) after checking that s really is in
// the predicted binade and stays there; a slow item, or a run whose check fails, is replayed term by
// term with real f32 additions.  Every path yields the sequential sum's bits; the prediction only
// decides how much is replayed.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define XS_HD __host__ __device__ __forceinline__
#else
#define XS_HD inline
#include <cmath>
#endif

namespace cmld {
namespace xsum {

constexpr int kItem = 8;            // terms per item (one lane)
constexpr int kChunk = 256;         // terms per chunk (one warp pass)
constexpr uint32_t kSlow = 0xffu;   // exponent field of a slow item

// An item or a composed run: low 24 bits of w0 / w1 = d0 / d1; high byte of w0 = the f32 biased
// exponent of the binade (kSlow: replay); high byte of w1 = the lane where the run starts.
struct Item {
  uint32_t w0, w1;
};

XS_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
XS_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
XS_HD float add_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  volatile float r = a + b;
  return r;
#endif
}
XS_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  volatile float r = a * b;
  return r;
#endif
}
XS_HD int dbl_exponent(double a) {  // unbiased exponent of a positive normal double
#if defined(__CUDA_ARCH__)
  return ((__double2hiint(a) >> 20) & 0x7ff) - 1023;
#else
  uint64_t u;
  memcpy(&u, &a, 8);
  return (int)((u >> 52) & 0x7ff) - 1023;
#endif
}

// (d0, d1) of `first` followed by `second`.
XS_HD void compose(uint32_t f0, uint32_t f1, uint32_t g0, uint32_t g1, uint32_t &h0, uint32_t &h1) {
  h0 = f0 + ((f0 & 1u) ? g1 : g0);
  h1 = f1 + (((f1 + 1u) & 1u) ? g1 : g0);
}

// One item: 8 terms t[] that follow an (approximate, double) prefix sum `a_start`.  Returns the
// biased f32 exponent of the predicted binade, or kSlow, and the item's increments.
XS_HD uint32_t item_local(const float (&t)[kItem], double a_start, uint32_t &d0, uint32_t &d1) {
  d0 = d1 = 0;
  double a_end = a_start;
  for (int i = 0; i < kItem; ++i) a_end += (double)t[i];
  if (!(a_start > 0.0) || !(a_end < 3.0e38)) return kSlow;
  const int eb = dbl_exponent(a_start);
  if (eb != dbl_exponent(a_end) || eb < -100 || eb > 126) return kSlow;
  const float scale = bits_f32((uint32_t)(23 - eb + 127) << 23);  // 2^(23-eb): term -> units of the binade's ulp
  for (int i = 0; i < kItem; ++i) {
    const float q = mul_rn(t[i], scale);  // exact (power of two) unless it underflows towards 0, where it rounds to 0 units anyway
    if (!(q < 8388608.0f)) return kSlow;  // a term as large as the binade itself (or NaN): cannot stay inside it
#if defined(__CUDA_ARCH__)
    const float kf = floorf(q);
#else
    const float kf = std::floor(q);
#endif
    const float fr = q - kf;  // exact
    const uint32_t k = (uint32_t)kf;
    if (fr == 0.5f) {
      // tie: the sum moves to the even neighbour, which depends on the parity of S + k
      d0 += k + ((d0 + k) & 1u);
      d1 += k + ((1u + d1 + k) & 1u);
    } else {
      const uint32_t r = k + (fr > 0.5f ? 1u : 0u);
      d0 += r;
      d1 += r;
    }
    if ((d0 | d1) >> 24) return kSlow;
  }
  return (uint32_t)(eb + 127);
}

// The walk over one chunk's events.  `sq` holds the chunk's terms (for replays), `items` its 32
// items (already composed along runs), `events` the lanes that end a run or are slow.
XS_HD float walk_chunk(float s, const float *sq, const Item *items, uint32_t events) {
  while (events) {
#if defined(__CUDA_ARCH__)
    const int lane = __ffs((int)events) - 1;
#else
    const int lane = __builtin_ctz(events);
#endif
    events &= events - 1;
    const Item it = items[lane];
    const uint32_t e = it.w0 >> 24;
    int first = lane;  // first lane to replay if the fast path does not apply
    if (e != kSlow) {
      const uint32_t sb = f32_bits(s);
      if ((sb >> 23) == e) {
        const uint32_t m = sb & 0x7fffffu;
        const uint32_t d = ((m & 1u) ? it.w1 : it.w0) & 0xffffffu;
        if (m + d < 0x800000u) {  // still inside the binade: the integer step is the f32 result
          s = bits_f32(sb + d);
          continue;
        }
      }
      first = (int)(it.w1 >> 24);
    }
    for (int i = first * kItem; i < (lane + 1) * kItem; ++i) s = add_rn(s, sq[i]);
  }
  return s;
}

#if defined(__CUDACC__)

// Device side.  A warp prepares one chunk: lane l holds terms [8l, 8l+8) of the chunk in t[], and
// a_start is the approximate prefix sum at the lane's first term.  Writes the chunk's items
// (composed along runs) and returns the event mask (same value in every lane).
__device__ __forceinline__ uint32_t prepare_chunk(const float (&t)[kItem], double a_start, int lane, Item *items) {
  uint32_t d0, d1;
  const uint32_t e = item_local(t, a_start, d0, d1);
  const uint32_t e_prev = __shfl_up_sync(0xffffffffu, e, 1);
  const bool boundary = lane == 0 || e == kSlow || e_prev == kSlow || e != e_prev;  // a run starts here
  const uint32_t bmask = __ballot_sync(0xffffffffu, boundary);
  const int rs = 31 - __clz((int)(bmask & (0xffffffffu >> (31 - lane))));  // start of this lane's run
  // inclusive scan along runs: after the step with offset o a lane holds the composition of up to 2o items ending at it
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t p0 = __shfl_up_sync(0xffffffffu, d0, o), p1 = __shfl_up_sync(0xffffffffu, d1, o);
    if (lane - o >= rs) {
      uint32_t h0, h1;
      compose(p0, p1, d0, d1, h0, h1);
      d0 = h0;
      d1 = h1;
    }
  }
  // a composed run may exceed the binade; the walk sees that as m + d >= 2^23 only if d is kept in range
  const bool too_big = e != kSlow && ((d0 | d1) >> 24) != 0;
  Item it;
  it.w0 = (too_big ? 0xffffffu : d0) | (e << 24);
  it.w1 = (too_big ? 0xffffffu : d1) | ((uint32_t)rs << 24);
  items[lane] = it;
  const bool run_end = lane == 31 || ((bmask >> (lane + 1)) & 1u);
  return __ballot_sync(0xffffffffu, e == kSlow || run_end);
}

// CTA-wide: the sequential f32 sum of sq[0..n) (n a multiple of 256, all terms >= 0), by NWARPS
// warps that all call this with their warp / lane ids; the result is returned to every thread.
// `bar` is the id of a named barrier over exactly NWARPS*32 threads that no other code uses meanwhile.
//   ws_chunk: n/256 doubles, ws_events: n/256 words, ws_items: n/8 items, ws_out: 1 float.
template <int NWARPS>
__device__ __forceinline__ float cta_sum(const float *sq, int n, int warp, int lane, int bar, double *ws_chunk,
                                         uint32_t *ws_events, Item *ws_items, float *ws_out) {
  const int n_chunks = n >> 8;  // at most 32
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));  // sq complete
  // approximate prefix sums in double: per chunk first
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
    const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
    double loc = (double)a.x + (double)a.y + (double)a.z + (double)a.w + (double)b.x + (double)b.y + (double)b.z + (double)b.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loc += __shfl_xor_sync(0xffffffffu, loc, o);
    if (lane == 0) ws_chunk[ch] = loc;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    double base = lane < ch ? ws_chunk[lane] : 0.0;  // n <= 8192: at most 32 chunks
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
    const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
    const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
    const float t[kItem] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    double loc = 0.0;
#pragma unroll
    for (int i = 0; i < kItem; ++i) loc += (double)t[i];
    double incl = loc;  // inclusive scan over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double p = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += p;
    }
    const uint32_t ev = prepare_chunk(t, base + (incl - loc), lane, ws_items + ch * 32);
    if (lane == 0) ws_events[ch] = ev;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  if (warp == 0 && lane == 0) {
    float s = 0.0f;
    for (int ch = 0; ch < n_chunks; ++ch) s = walk_chunk(s, sq + ch * kChunk, ws_items + ch * 32, ws_events[ch]);
    *ws_out = s;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  return *ws_out;
}

// Shared-memory bytes cta_sum needs besides sq itself, for n terms.
__host__ __device__ inline int workspace_bytes(int n) { return (n >> 8) * 8 + (n >> 8) * 4 + (n >> 3) * 8 + 16; }

#endif  // __CUDACC__

}  // namespace xsum
}  // namespace cmld
