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
// Procedure.  Items are groups of 8 consecutive terms.  A parallel (tree) prefix sum predicts each
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

// (d0, d1) of `first` followed by `second`.
XS_HD void compose(uint32_t f0, uint32_t f1, uint32_t g0, uint32_t g1, uint32_t &h0, uint32_t &h1) {
  h0 = f0 + ((f0 & 1u) ? g1 : g0);
  h1 = f1 + (((f1 + 1u) & 1u) ? g1 : g0);
}

// One item: 8 terms t[] that follow an approximate prefix sum `a_start` (a tree sum: it only has to predict
// the binade) and end at `a_end`.  Returns the biased f32 exponent of the predicted binade, or kSlow, and
// the item's increments.
XS_HD uint32_t item_local(const float (&t)[kItem], float a_start, float a_end, uint32_t &d0, uint32_t &d1) {
  d0 = d1 = 0;
  if (!(a_start > 0.0f) || !(a_end < 3.0e38f)) return kSlow;
  const int eb = (int)(f32_bits(a_start) >> 23) - 127;
  if (eb != (int)(f32_bits(a_end) >> 23) - 127 || eb < -100 || eb > 126) return kSlow;
  const float scale = bits_f32((uint32_t)(23 - eb + 127) << 23);  // 2^(23-eb): term -> units of the binade's ulp
  for (int i = 0; i < kItem; ++i) {
    const float q = mul_rn(t[i], scale);  // exact (power of two) unless it underflows towards 0, where it rounds to 0 units anyway
    if (!(q < 8388608.0f)) return kSlow;  // a term as large as the binade itself (or NaN): cannot stay inside it
#if defined(__CUDA_ARCH__)
    const uint32_t k = (uint32_t)__float2int_rd(q);
#else
    const uint32_t k = (uint32_t)std::floor(q);
#endif
    const float fr = q - (float)k;  // exact
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
// The exact sum s is the only loop-carried value: the next event's item is fetched before the current
// one is applied, and a slow item's eight terms are loaded before they are added.
XS_HD float walk_chunk(float s, const float *sq, const Item *items, uint32_t events) {
  if (!events) return s;
#if defined(__CUDA_ARCH__)
  int lane = __ffs((int)events) - 1;
#else
  int lane = __builtin_ctz(events);
#endif
  Item it = items[lane];
  while (true) {
    events &= events - 1;
    int lane_n = 0;
    Item it_n = it;
    if (events) {
#if defined(__CUDA_ARCH__)
      lane_n = __ffs((int)events) - 1;
#else
      lane_n = __builtin_ctz(events);
#endif
      it_n = items[lane_n];
    }
    const uint32_t e = it.w0 >> 24;
    if (e != kSlow) {
      // s is in binade e iff t = bits(s) - (e << 23) < 2^23 (as unsigned); then t is its mantissa field
      const uint32_t sb = f32_bits(s);
      const uint32_t t = sb - (e << 23);
      const uint32_t d = ((t & 1u) ? it.w1 : it.w0) & 0xffffffu;
      if (t + d < 0x800000u && t < 0x800000u) {  // in the binade and still inside it afterwards: the integer step is the f32 result
        s = bits_f32(sb + d);
      } else {
        const int first = (int)(it.w1 >> 24);
        for (int i = first * kItem; i < (lane + 1) * kItem; ++i) s = add_rn(s, sq[i]);
      }
    } else {
      const float *q = sq + lane * kItem;
      const float t0 = q[0], t1 = q[1], t2 = q[2], t3 = q[3], t4 = q[4], t5 = q[5], t6 = q[6], t7 = q[7];
      s = add_rn(s, t0);
      s = add_rn(s, t1);
      s = add_rn(s, t2);
      s = add_rn(s, t3);
      s = add_rn(s, t4);
      s = add_rn(s, t5);
      s = add_rn(s, t6);
      s = add_rn(s, t7);
    }
    if (!events) break;
    lane = lane_n;
    it = it_n;
  }
  return s;
}

#if defined(__CUDACC__)

// Device side.  A warp prepares one chunk: lane l holds terms [8l, 8l+8) of the chunk in t[], and
// a_start is the approximate prefix sum at the lane's first term.  Writes the chunk's items
// (composed along runs) and returns the event mask (same value in every lane).
__device__ __forceinline__ uint32_t prepare_chunk(const float (&t)[kItem], float a_start, float a_end, int lane, Item *items) {
  uint32_t d0, d1;
  const uint32_t e = item_local(t, a_start, a_end, d0, d1);
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

// One event of the flat list the walker goes through: a composed run (or a slow item) and where its terms are.
struct Event {
  uint32_t w0, w1;   // as Item
  uint32_t first;    // index in sq of the first term to replay if the run's step cannot be taken
  uint32_t end;      // index in sq one past the event's last term
};

// The walk over the whole list; s is the only loop-carried value: the next event's record, and the eight
// terms a slow event adds, are fetched one event ahead.
__device__ __forceinline__ float walk_events(const float *sq, const Event *ev, int n_events) {
  float s = 0.0f;
  if (n_events <= 0) return s;
  uint4 cur = *reinterpret_cast<const uint4 *>(ev);
  float4 ca = *reinterpret_cast<const float4 *>(sq + cur.w - kItem), cb = *reinterpret_cast<const float4 *>(sq + cur.w - kItem + 4);
  for (int k = 0; k < n_events; ++k) {
    const uint4 nxt = *reinterpret_cast<const uint4 *>(ev + (k + 1 < n_events ? k + 1 : k));
    const float4 na = *reinterpret_cast<const float4 *>(sq + nxt.w - kItem), nb = *reinterpret_cast<const float4 *>(sq + nxt.w - kItem + 4);
    const uint32_t e = cur.x >> 24;
    const uint32_t sb = __float_as_uint(s);
    const uint32_t t = sb - (e << 23);  // s is in binade e iff t < 2^23 (unsigned); then t is its mantissa field
    const uint32_t d = ((t & 1u) ? cur.y : cur.x) & 0xffffffu;
    if (e != kSlow && t < 0x800000u && t + d < 0x800000u) {
      s = __uint_as_float(sb + d);  // still inside the binade: the integer step is the f32 result
    } else {
      // a slow item (its own eight terms), or a run whose step cannot be taken: replay from cur.z
      for (uint32_t i = cur.z; i + kItem < cur.w; ++i) s = __fadd_rn(s, sq[i]);
      s = __fadd_rn(s, ca.x);
      s = __fadd_rn(s, ca.y);
      s = __fadd_rn(s, ca.z);
      s = __fadd_rn(s, ca.w);
      s = __fadd_rn(s, cb.x);
      s = __fadd_rn(s, cb.y);
      s = __fadd_rn(s, cb.z);
      s = __fadd_rn(s, cb.w);
    }
    cur = nxt;
    ca = na;
    cb = nb;
  }
  return s;
}

// CTA-wide: the sequential f32 sum of sq[0..n) (n a multiple of 256, at most 8192, all terms >= 0), by
// NWARPS warps that all call this with their warp / lane ids; the result is returned to every thread.
// `bar` is the id of a named barrier over exactly NWARPS*32 threads that no other code uses meanwhile.
// `ws` is workspace_bytes(n) bytes of shared memory, 16-byte aligned.
template <int NWARPS>
__device__ __forceinline__ float cta_sum(const float *sq, int n, int warp, int lane, int bar, uint8_t *ws) {
  const int n_chunks = n >> 8;  // at most 32
  float *ws_chunk = reinterpret_cast<float *>(ws);                      // [32] chunk sums (approximate)
  uint32_t *ws_mask = reinterpret_cast<uint32_t *>(ws + 256);           // [32] event lanes per chunk
  float *ws_out = reinterpret_cast<float *>(ws + 384);
  Item *ws_items = reinterpret_cast<Item *>(ws + 400);                  // [n / 8]
  Event *ws_events = reinterpret_cast<Event *>(ws + 400 + (n >> 3) * 8);  // [n / 8]
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));  // sq complete
  // approximate prefix sums (tree sums: they only predict binades): per chunk first
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
    const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
    float loc = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loc += __shfl_xor_sync(0xffffffffu, loc, o);
    if (lane == 0) ws_chunk[ch] = loc;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    float base = lane < ch ? ws_chunk[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
    const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
    const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
    const float t[kItem] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const float loc = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
    float incl = loc;  // inclusive scan over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float p = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += p;
    }
    const uint32_t ev = prepare_chunk(t, base + (incl - loc), base + incl, lane, ws_items + ch * 32);
    if (lane == 0) ws_mask[ch] = ev;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  // the events of all chunks as one list, in order
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    int before = lane < ch ? __popc(ws_mask[lane]) : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    const uint32_t mine = ws_mask[ch];
    if ((mine >> lane) & 1u) {
      const Item it = ws_items[ch * 32 + lane];
      Event e;
      e.w0 = it.w0;
      e.w1 = it.w1;
      e.first = (uint32_t)(ch * kChunk + (int)(it.w1 >> 24) * kItem);
      e.end = (uint32_t)(ch * kChunk + (lane + 1) * kItem);
      if ((it.w0 >> 24) == kSlow) e.first = e.end - kItem;
      ws_events[before + __popc(mine & ((1u << lane) - 1u))] = e;
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  if (warp == 0 && lane == 0) {
    int total = 0;
    for (int ch = 0; ch < n_chunks; ++ch) total += __popc(ws_mask[ch]);
    *ws_out = walk_events(sq, ws_events, total);
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  return *ws_out;
}

// Shared-memory bytes cta_sum needs besides sq itself, for n terms.
__host__ __device__ inline int workspace_bytes(int n) { return 400 + (n >> 3) * 8 + (n >> 3) * 16; }

#endif  // __CUDACC__

}  // namespace xsum
}  // namespace cmld
