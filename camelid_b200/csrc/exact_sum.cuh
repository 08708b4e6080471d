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
// which go to the even neighbour and therefore depend on the parity of S.  So a run of terms without
// ties that keeps s inside one binade adds one integer d to S, and such runs compose by addition.
//
// Procedure.  Items are groups of 8 consecutive terms.  A parallel (tree) prefix sum predicts each
// item's binade.  Items whose predicted binade does not change across them and that hold no tie are
// "fast": a lane computes their d under that binade.  The other items (the few where the sum crosses
// into a new binade, the rare ones with a tie, and the very first) are "slow".  Runs of fast items
// with the same binade inside a 256-term chunk are summed with a warp scan.  Finally one thread walks
// the events (run ends and slow items) in order with the exact s: a run is applied as one integer
// addition, a slow item is replayed term by term with real f32 additions.  Every record of the walk
// has the same shape — a run's integer step, then the eight terms of the slow item behind it (zeros
// if there is none) — so the walk runs without a branch; it only records on the side whether every
// run really started and ended inside its predicted binade, and is repeated with the check in front
// of every step (replaying a failed run term by term) in the rare case that one did not.  Every
// path yields the sequential sum's bits; the prediction only decides how much is replayed.
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

// An item or a summed run: low 24 bits of w0 = d; high byte of w0 = the f32 biased exponent of the
// binade (kSlow: replay); w1 = the lane where the run starts.
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

// One item: 8 terms t[] that follow an approximate prefix sum `a_start` (a tree sum: it only has to predict
// the binade) and end at `a_end`.  Returns the biased f32 exponent of the predicted binade, or kSlow, and
// the item's increment d in units of the binade's ulp.
XS_HD uint32_t item_local(const float (&t)[kItem], float a_start, float a_end, uint32_t &d) {
  d = 0;
  if (!(a_start > 0.0f) || !(a_end < 3.0e38f)) return kSlow;
  const int eb = (int)(f32_bits(a_start) >> 23) - 127;
  if (eb != (int)(f32_bits(a_end) >> 23) - 127 || eb < -100 || eb > 126) return kSlow;
  const float scale = bits_f32((uint32_t)(23 - eb + 127) << 23);  // 2^(23-eb): term -> units of the binade's ulp
  // q + 2^23 rounds q to an integer (ties to even); its bits minus those of 2^23 are that integer (also when the sum
  // is 2^24).  A term as large as the binade itself (q >= 2^23) makes that difference >= 2^23, so the item's d shows
  // it; NaN and infinity never get here (a_end is not finite then).
  float worst = 0.0f;  // largest |q - round(q)|: 0.5 means a tie, whose result depends on the parity of S
  uint32_t acc = 0;
  for (int i = 0; i < kItem; ++i) {
    const float q = mul_rn(t[i], scale);  // exact (power of two) unless it underflows towards 0, where it rounds to 0 units anyway
    const float m = add_rn(q, 8388608.0f);
    const float diff = add_rn(q, -add_rn(m, -8388608.0f));  // both subtractions are exact
#if defined(__CUDA_ARCH__)
    worst = fmaxf(worst, fabsf(diff));
#else
    worst = std::fmax(worst, std::fabs(diff));
#endif
    acc += f32_bits(m);
  }
  d = acc - (uint32_t)kItem * 0x4b000000u;
  if (worst == 0.5f || (d >> 23)) return kSlow;
  return (uint32_t)(eb + 127);
}

// The walk over one chunk's events, every step checked.  `sq` holds the chunk's terms (for replays), `items`
// its 32 items (already summed along runs), `events` the lanes that end a run or are slow.
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
    int first = lane;  // a slow item replays its own eight terms
    if (e != kSlow) {
      // s is in binade e iff t = bits(s) - (e << 23) < 2^23 (as unsigned); then t is its mantissa field
      const uint32_t sb = f32_bits(s);
      const uint32_t t = sb - (e << 23), d = it.w0 & 0xffffffu;
      if (t < 0x800000u && t + d < 0x800000u) {  // in the binade and still inside it afterwards: the integer step is the f32 result
        s = bits_f32(sb + d);
        continue;
      }
      first = (int)it.w1;  // the run's first item
    }
    for (int i = first * kItem; i < (lane + 1) * kItem; ++i) s = add_rn(s, sq[i]);
  }
  return s;
}

#if defined(__CUDACC__)

// Device side.  A warp prepares one chunk: lane l holds terms [8l, 8l+8) of the chunk in t[], and
// a_start is the approximate prefix sum at the lane's first term.  Writes the chunk's items
// (summed along runs) and returns the event mask (same value in every lane).
__device__ __forceinline__ uint32_t prepare_chunk(const float (&t)[kItem], float a_start, float a_end, int lane, Item *items, uint32_t &slow_mask) {
  uint32_t d;
  const uint32_t e = item_local(t, a_start, a_end, d);
  const uint32_t e_prev = __shfl_up_sync(0xffffffffu, e, 1);
  const bool boundary = lane == 0 || e == kSlow || e_prev == kSlow || e != e_prev;  // a run starts here
  const uint32_t bmask = __ballot_sync(0xffffffffu, boundary);
  const int rs = 31 - __clz((int)(bmask & (0xffffffffu >> (31 - lane))));  // start of this lane's run
  // inclusive sum along runs (at most 32 x 2^24: no overflow)
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t p = __shfl_up_sync(0xffffffffu, d, o);
    if (lane - o >= rs) d += p;
  }
  // a run longer than the binade: the walk sees t + d >= 2^23 as long as d is kept in range
  const bool too_big = e != kSlow && (d >> 24) != 0;
  Item it;
  it.w0 = (too_big ? 0xffffffu : d) | (e << 24);
  it.w1 = (uint32_t)rs;
  items[lane] = it;
  const bool run_end = lane == 31 || ((bmask >> (lane + 1)) & 1u);
  slow_mask = __ballot_sync(0xffffffffu, e == kSlow);
  return __ballot_sync(0xffffffffu, e == kSlow || run_end);
}

// One event of the flat list the walker goes through.  Every event is "one integer step, then eight f32 additions":
// a run has its increment and, if the item behind it is slow, that item's eight terms (else eight zeros); a slow item
// that follows another slow item (or nothing) has a zero increment and its own terms — so the walk is one straight
// line of code without a branch (a lone thread pays tens of cycles for every taken branch).
struct Event {
  uint32_t d;        // the run's increment (0 without a run)
  uint32_t ebits;    // the run's binade as f32 exponent bits (e << 23)
  uint32_t span;     // the run: items [bits 0-10, bits 11-21) of sq (replayed if the step cannot be taken); bit 31: there is a run
  uint32_t taddr;    // shared-memory address of the eight terms to add after the step (none: eight zeros)
};
constexpr uint32_t kRunFlag = 0x80000000u;
constexpr int kWalkUnroll = 6;  // the walk's trip: records rotate through three registers sets, terms through two

// The walk, every step checked: a run whose step cannot be taken is replayed term by term.
static __device__ __noinline__ float walk_events_checked(const float *sq, const Event *ev, int n_events, uint32_t zero_addr) {
  const uint32_t sq_addr = (uint32_t)__cvta_generic_to_shared(sq);
  float s = 0.0f;
  for (int k = 0; k < n_events; ++k) {
    const Event cur = ev[k];
    if (cur.span & kRunFlag) {
      const uint32_t sb = __float_as_uint(s), t = sb - cur.ebits;
      if (t < 0x800000u && t + cur.d < 0x800000u) {
        s = __uint_as_float(sb + cur.d);
      } else {
        const uint32_t first = (cur.span & 0x7ffu) * kItem, end = ((cur.span >> 11) & 0x7ffu) * kItem;
        for (uint32_t i = first; i < end; ++i) s = __fadd_rn(s, sq[i]);
      }
    }
    if (cur.taddr != zero_addr) {
      const float *t = sq + ((cur.taddr - sq_addr) >> 2);
      for (int i = 0; i < kItem; ++i) s = __fadd_rn(s, t[i]);
    }
  }
  return s;
}

// The walk over the whole list (n_events a multiple of kWalkUnroll, two more readable records behind it).  s is
// the only loop-carried value and no branch depends on anything: whether every run started and ended inside its
// binade is collected on the side, in the issue slots the dependent additions leave free.  Records are fetched two
// events ahead and an event's terms one event ahead, into registers that rotate with the unrolled trip, so the
// loads are never waited for and nothing is moved.  Falls back to the checked walk if a run did not fit.
__device__ __forceinline__ float walk_events(const float *sq, const Event *ev, int n_events, uint32_t zero_addr) {
  uint32_t sb = 0, bad = 0;
  uint32_t ea = (uint32_t)__cvta_generic_to_shared(ev);
  uint4 H0, H1, H2;
  float4 A0, B0, A1, B1;
#define XS_LDH(H, ADDR) asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(H.x), "=r"(H.y), "=r"(H.z), "=r"(H.w) : "r"(ADDR))
#define XS_LDT(A, B, H)                                                                                                   \
  do {                                                                                                                    \
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(A.x), "=f"(A.y), "=f"(A.z), "=f"(A.w) : "r"(H.w));       \
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(B.x), "=f"(B.y), "=f"(B.z), "=f"(B.w) : "r"(H.w + 16u)); \
  } while (0)
#define XS_STEP(K, HC, HN, HNN, AC, BC, AN, BN)                                        \
  do {                                                                                 \
    XS_LDH(HNN, ea + 16u * ((K) + 2));                                                 \
    XS_LDT(AN, BN, HN);                                                                \
    const uint32_t t_ = sb - HC.y;                                                     \
    sb += HC.x;                                                                        \
    float s_ = __uint_as_float(sb);                                                    \
    s_ = __fadd_rn(s_, AC.x);                                                          \
    bad |= (t_ | (t_ + HC.x)) & (uint32_t)((int32_t)HC.z >> 31); /* t >= 2^23: s is not in the binade; t + d >= 2^23: it would leave it */ \
    s_ = __fadd_rn(s_, AC.y);                                                          \
    s_ = __fadd_rn(s_, AC.z);                                                          \
    s_ = __fadd_rn(s_, AC.w);                                                          \
    s_ = __fadd_rn(s_, BC.x);                                                          \
    s_ = __fadd_rn(s_, BC.y);                                                          \
    s_ = __fadd_rn(s_, BC.z);                                                          \
    s_ = __fadd_rn(s_, BC.w);                                                          \
    sb = __float_as_uint(s_);                                                          \
  } while (0)
  XS_LDH(H0, ea);
  XS_LDH(H1, ea + 16u);
  XS_LDT(A0, B0, H0);
  for (int k = 0; k < n_events; k += kWalkUnroll) {
    XS_STEP(0, H0, H1, H2, A0, B0, A1, B1);
    XS_STEP(1, H1, H2, H0, A1, B1, A0, B0);
    XS_STEP(2, H2, H0, H1, A0, B0, A1, B1);
    XS_STEP(3, H0, H1, H2, A1, B1, A0, B0);
    XS_STEP(4, H1, H2, H0, A0, B0, A1, B1);
    XS_STEP(5, H2, H0, H1, A1, B1, A0, B0);
    ea += 16u * kWalkUnroll;
  }
#undef XS_LDH
#undef XS_LDT
#undef XS_STEP
  if (bad >> 23) return walk_events_checked(sq, ev, n_events, zero_addr);
  return __uint_as_float(sb);
}

// CTA-wide: the sequential f32 sum of sq[0..n) (n a multiple of 256, at most 8192, all terms >= 0), by
// NWARPS warps that all call this with their warp / lane ids; the result is returned to every thread.
// `bar` is the id of a named barrier over exactly NWARPS*32 threads that no other code uses meanwhile.
// `ws` is workspace_bytes(n) bytes of shared memory, 16-byte aligned.
template <int NWARPS>
__device__ __forceinline__ float cta_sum(const float *sq, int n, int warp, int lane, int bar, uint8_t *ws) {
  constexpr int kTrips = (32 + NWARPS - 1) / NWARPS;  // chunks a warp may own (chunk = warp + trip * NWARPS)
  const int n_chunks = n >> 8;  // at most 32
  float *ws_chunk = reinterpret_cast<float *>(ws);                      // [32] chunk sums (approximate)
  uint32_t *ws_slow = reinterpret_cast<uint32_t *>(ws + 128);           // [32] slow items per chunk
  uint32_t *ws_mask = reinterpret_cast<uint32_t *>(ws + 256);           // [32] event lanes per chunk
  float *ws_out = reinterpret_cast<float *>(ws + 384);
  int *ws_total = reinterpret_cast<int *>(ws + 388);                    // number of events, padded to the walk's trip
  float *ws_zero = reinterpret_cast<float *>(ws + 400);                 // [8] zeros: the terms of a padding event
  Item *ws_items = reinterpret_cast<Item *>(ws + 448);                  // [n / 8]
  Event *ws_events = reinterpret_cast<Event *>(ws + 448 + (n >> 3) * 8);  // [n / 8 + 8]
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));  // sq complete
  // approximate prefix sums (tree sums: they only predict binades): inside every chunk first; the terms stay in registers
  // (the first chunk's terms stay in registers across the barrier; a warp's further chunks — rows wider than
  // NWARPS * 256 — are read again: fewer live registers in the kernels that inline this)
  float tt[kItem], incl_[kTrips], loc_[kTrips];
  if (warp == 0 && lane < 8) ws_zero[lane] = 0.0f;
#pragma unroll
  for (int trip = 0; trip < kTrips; ++trip) {
    const int ch = warp + trip * NWARPS;
    if (ch < n_chunks) {
      const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
      const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
      if (trip == 0) {
        tt[0] = a.x, tt[1] = a.y, tt[2] = a.z, tt[3] = a.w;
        tt[4] = b.x, tt[5] = b.y, tt[6] = b.z, tt[7] = b.w;
      }
      const float loc = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
      float incl = loc;  // inclusive scan over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float p = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += p;
      }
      incl_[trip] = incl;
      loc_[trip] = loc;
      if (lane == 31) ws_chunk[ch] = incl;
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
#pragma unroll
  for (int trip = 0; trip < kTrips; ++trip) {
    const int ch = warp + trip * NWARPS;
    if (ch < n_chunks) {
      float base = lane < ch ? ws_chunk[lane] : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
      uint32_t slow_mask, ev;
      if (trip == 0) {
        ev = prepare_chunk(tt, base + (incl_[trip] - loc_[trip]), base + incl_[trip], lane, ws_items + ch * 32, slow_mask);
      } else {
        const float4 a = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem);
        const float4 b = *reinterpret_cast<const float4 *>(sq + ch * kChunk + lane * kItem + 4);
        const float t2[kItem] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        ev = prepare_chunk(t2, base + (incl_[trip] - loc_[trip]), base + incl_[trip], lane, ws_items + ch * 32, slow_mask);
      }
      if (lane == 0) {
        ws_mask[ch] = ev;
        ws_slow[ch] = slow_mask;
      }
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  // The events of all chunks as one list, in order.  A slow item whose previous item is fast rides on that run's
  // record (the run's step, then the item's eight terms); every other event lane owns a record.
  const uint32_t sq_addr = (uint32_t)__cvta_generic_to_shared(sq);
  const uint32_t zero_addr = (uint32_t)__cvta_generic_to_shared(ws_zero);
  // lanes c of a chunk's slow items that ride: slow, previous item (lane c - 1, or the previous chunk's last) fast
  auto riders = [&](int c) {
    const uint32_t sl = ws_slow[c];
    const uint32_t prev_slow = (sl << 1) | (c > 0 ? (ws_slow[c - 1] >> 31) : 1u);
    return sl & ~prev_slow;
  };
  for (int ch = warp; ch < n_chunks; ch += NWARPS) {
    int before = lane < ch ? __popc(ws_mask[lane] & ~riders(lane)) : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    const uint32_t mine = ws_mask[ch], slow_c = ws_slow[ch], ride = riders(ch), own = mine & ~ride;
    if ((mine >> lane) & 1u) {
      const Item it = ws_items[ch * 32 + lane];
      const uint32_t end_item = (uint32_t)(ch * 32 + lane + 1);
      const uint32_t my_terms = sq_addr + (end_item - 1) * (kItem * 4u);
      const int below = __popc(own & ((1u << lane) - 1u));
      if ((ride >> lane) & 1u) {
        ws_events[before + below - 1].taddr = my_terms;  // the record of the run that ends just before this item
      } else if ((slow_c >> lane) & 1u) {
        Event e;
        e.d = 0u;
        e.ebits = 0u;
        e.span = 0u;
        e.taddr = my_terms;
        ws_events[before + below] = e;
      } else {
        const bool next_slow = lane < 31 ? ((slow_c >> (lane + 1)) & 1u) != 0 : (ch + 1 < n_chunks && (ws_slow[ch + 1] & 1u));
        Event *e = ws_events + before + below;
        e->d = it.w0 & 0xffffffu;
        e->ebits = (it.w0 >> 24) << 23;
        e->span = (uint32_t)(ch * 32 + (int)it.w1) | (end_item << 11) | kRunFlag;
        if (!next_slow) e->taddr = zero_addr;  // else the slow item behind this run writes its terms' address here
      }
    }
    if (ch == n_chunks - 1) {
      // padding (no step, eight zeros) up to the walk's trip and two records beyond it
      const int total = before + __popc(own);
      if (lane < kWalkUnroll + 1) {
        Event e;
        e.d = 0u;
        e.ebits = 0u;
        e.span = 0u;
        e.taddr = zero_addr;
        ws_events[total + lane] = e;
      }
      if (lane == 0) *ws_total = (total + kWalkUnroll - 1) / kWalkUnroll * kWalkUnroll;
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  if (warp == 0 && lane == 0) *ws_out = walk_events(sq, ws_events, *ws_total, zero_addr);
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NWARPS * 32));
  return *ws_out;
}

// For tests: the checked walk over the event list the last cta_sum call left in `ws`, with the binade of every second
// run made wrong first, so that those runs are replayed term by term — the result must have the same bits.  One thread.
__device__ inline float rewalk_with_forced_replays(const float *sq, int n, uint8_t *ws) {
  Event *ev = reinterpret_cast<Event *>(ws + 448 + (n >> 3) * 8);
  const int total = *reinterpret_cast<const int *>(ws + 388);
  int runs = 0;
  for (int k = 0; k < total; ++k)
    if ((ev[k].span & kRunFlag) && (runs++ & 1)) ev[k].ebits ^= 0x00800000u;
  return walk_events_checked(sq, ev, total, (uint32_t)__cvta_generic_to_shared(ws + 400));
}

// Shared-memory bytes cta_sum needs besides sq itself, for n terms.
__host__ __device__ inline int workspace_bytes(int n) { return 448 + (n >> 3) * 8 + ((n >> 3) + 8) * 16; }

#endif  // __CUDACC__

}  // namespace xsum
}  // namespace cmld
