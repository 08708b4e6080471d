// Host build of exact_sum.cuh: the per-item arithmetic and the checked event walk are the code the kernels
// run; the warp scan that sums runs is replaced by a loop.  Compares with the plain sequential f32 sum
// over thousands of seeded arrays (outliers, exact ties, zeros, powers of two, tiny and huge terms).
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <random>
#include "../camelid_b200/csrc/exact_sum.cuh"  // compiled for the host: the same item / compose / walk code the kernels run
using namespace cmld::xsum;

static long g_replayed = 0, g_events = 0, g_terms = 0;

static float emu(const std::vector<float> &sq) {
  const int n = (int)sq.size(), nch = n / 256;
  std::vector<float> chunk(nch);
  for (int c = 0; c < nch; ++c) { float s = 0; for (int i = 0; i < 256; ++i) s += sq[c * 256 + i]; chunk[c] = s; }
  float s = 0.0f;
  float base = 0;
  for (int c = 0; c < nch; ++c) {
    Item items[32];
    uint32_t e[32], d[32];
    float a = base;
    for (int l = 0; l < 32; ++l) {
      float t[8];
      for (int i = 0; i < 8; ++i) t[i] = sq[c * 256 + l * 8 + i];
      float a_end = a;
      for (int i = 0; i < 8; ++i) a_end += t[i];
      e[l] = item_local(t, a, a_end, d[l]);
      a = a_end;
    }
    uint32_t events = 0;
    int rs = 0;
    uint32_t acc = 0;
    for (int l = 0; l < 32; ++l) {
      bool boundary = l == 0 || e[l] == kSlow || e[l - 1] == kSlow || e[l] != e[l - 1];
      if (boundary) { rs = l; acc = d[l]; }
      else acc += d[l];
      bool too_big = e[l] != kSlow && (acc >> 24);
      items[l].w0 = (too_big ? 0xffffffu : acc) | (e[l] << 24);
      items[l].w1 = (uint32_t)rs;
      bool next_boundary = l == 31 || e[l + 1] == kSlow || e[l] == kSlow || e[l + 1] != e[l];
      if (e[l] == kSlow || next_boundary) events |= 1u << l;
    }
    // count replays
    {
      float s2 = s; uint32_t ev = events;
      while (ev) { int lane = __builtin_ctz(ev); ev &= ev - 1; ++g_events;
        Item it = items[lane]; uint32_t ee = it.w0 >> 24; int first = lane; bool fast = false;
        if (ee != kSlow) { uint32_t sb = f32_bits(s2); if ((sb >> 23) == ee) { uint32_t m = sb & 0x7fffff; uint32_t dd = it.w0 & 0xffffff; if (m + dd < 0x800000u) { s2 = bits_f32(sb + dd); fast = true; } } if (!fast) first = it.w1; }
        if (!fast) { for (int i = first * 8; i < (lane + 1) * 8; ++i) { s2 = add_rn(s2, sq[c * 256 + i]); ++g_replayed; } }
      }
    }
    s = walk_chunk(s, sq.data() + c * 256, items, events);
    base += chunk[c];
  }
  g_terms += n;
  return s;
}

static float seq(const std::vector<float> &sq) { float s = 0; for (float t : sq) s = add_rn(s, t); return s; }

int main() {
  std::mt19937_64 rng(12345);
  std::normal_distribution<float> nd(0.f, 1.f);
  long bad = 0, total = 0;
  for (int trial = 0; trial < 6000; ++trial) {
    int n = 256 * (1 + (int)(rng() % 32));
    std::vector<float> sq(n);
    int mode = trial % 12;
    float sigma = std::pow(10.0f, (float)((int)(rng() % 13) - 6));
    for (int i = 0; i < n; ++i) {
      float x = nd(rng) * sigma;
      if (mode == 1 && rng() % 100 == 0) x *= 100.f;          // outliers
      if (mode == 2) x = (float)((int)(rng() % 64)) / 8.0f;     // few mantissa bits: many ties
      if (mode == 3 && rng() % 3) x = 0.f;                      // zeros
      if (mode == 4) x = std::ldexp((float)(rng() % 4 + 1), (int)(rng() % 20) - 10);  // powers of two
      if (mode == 5 && i < 100) x = 0.f;                        // leading zeros
      if (mode == 6) x = (i == 700) ? 1e4f : x;                 // one giant
      if (mode == 7) x = 1.0f;                                  // constant
      if (mode == 8) x = 0.5f + (float)(rng() % 2);             // ties everywhere
      if (mode == 9) x = nd(rng) * 1e-18f;                      // tiny squares (subnormal range)
      if (mode == 10) x = nd(rng) * 1e15f;                      // large
      if (mode == 11) x = std::sqrt((float)(rng() % 1024 + 1) * 0.5f); // sqrt values
      sq[i] = mul_rn(x, x);
    }
    float a = emu(sq), b = seq(sq);
    ++total;
    if (f32_bits(a) != f32_bits(b)) { if (bad < 10) printf("MISMATCH trial %d mode %d n %d: %.9g vs %.9g\n", trial, mode, n, a, b); ++bad; }
  }
  printf("%ld/%ld mismatches; events per 4096 terms %.1f; replayed terms fraction %.4f\n", bad, total, (double)g_events * 4096 / g_terms, (double)g_replayed / g_terms);
  // the typical case: 4096 squares of N(0,1)
  g_replayed = g_events = g_terms = 0;
  for (int trial = 0; trial < 2000; ++trial) {
    std::vector<float> sq(4096);
    for (auto &v : sq) { float x = nd(rng); v = mul_rn(x, x); }
    float a = emu(sq), b = seq(sq);
    if (f32_bits(a) != f32_bits(b)) { printf("MISMATCH typical\n"); ++bad; }
  }
  printf("typical N(0,1), n=4096: events %.1f, replayed terms %.1f per sum\n", (double)g_events / 2000, (double)g_replayed / 2000);
  return bad != 0;
}
