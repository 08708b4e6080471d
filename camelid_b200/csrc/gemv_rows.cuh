// Row kernels of the fused dequantise-and-matvec, shared by the direct-load kernel (weights
// read from global memory) and the staged kernel (weights and activations already in shared
// memory).  A warp works on R rows at once; a lane owns 16-byte units of each row's code
// stream and accumulates f32 partial sums that the caller combines with a shuffle tree.
//
// Integer parts follow Camelid's CPU dots exactly (Q8_0: q8_0_dot_rows, src/inference.rs:26166;
// Q4_K: q4_k_dot_scalar, src/diffusion_gemma/refmath.rs:504; Q6_K: q6_k_wire_row_dot,
// src/inference.rs:25535); only the order of the f32 additions differs.
#pragma once

#include "common.cuh"

namespace cmld {

template <bool SMEM>
__device__ __forceinline__ uint4 ld_w16(const uint8_t *p) {
  if constexpr (SMEM) return *reinterpret_cast<const uint4 *>(p);
  else return ld_stream16(p);
}
template <bool SMEM, typename T>
__device__ __forceinline__ T ld_a(const T *p) {
  if constexpr (SMEM) return *p;
  else return __ldg(p);
}

__device__ __forceinline__ int dot16(const uint4 &a, const int4 &b) {
  int s = __dp4a((int)a.x, b.x, 0);
  s = __dp4a((int)a.y, b.y, s);
  s = __dp4a((int)a.z, b.z, s);
  return __dp4a((int)a.w, b.w, s);
}

// act: quantised activation rows (Q8_0 codes/scales), act_stride bytes apart.
template <int B, int R, int U, bool SMEM>
__device__ __forceinline__ void rows_q8_0(const uint8_t *const (&row)[R], int64_t cols, const uint8_t *act, int64_t act_stride,
                                          int lane, float (&acc)[R][B]) {
  const int units = (int)(cols >> 4);
  const int64_t sc_off = act_scale_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * U) {
    uint4 wv[R][U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
#pragma unroll
      for (int r = 0; r < R; ++r) wv[r][i] = u < units ? ld_w16<SMEM>(row[r] + (int64_t)u * 16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      const int blk = u >> 1;
      float ws[R];
#pragma unroll
      for (int r = 0; r < R; ++r) ws[r] = f16_bits_to_f32(ld_a<SMEM>(reinterpret_cast<const uint16_t *>(row[r] + cols) + blk));
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xv = ld_a<SMEM>(reinterpret_cast<const int4 *>(a) + u);
        const float xs = ld_a<SMEM>(reinterpret_cast<const float *>(a + sc_off) + blk);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int isum = dot16(wv[r][i], xv);
          acc[r][b] = __fadd_rn(acc[r][b], __fmul_rn(__fmul_rn((float)isum, ws[r]), xs));
        }
      }
    }
  }
}

template <int B, int R, int U, bool SMEM>
__device__ __forceinline__ void rows_q4_k(const uint8_t *const (&row)[R], int64_t cols, const uint8_t *act, int64_t act_stride,
                                          int lane, float (&acc)[R][B]) {
  const int nsb = (int)(cols >> 8);
  const int units = nsb * 8;
  const int64_t sc_off = act_scale_off(cols), bs_off = act_bsum_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * U) {
    uint4 wv[R][U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
#pragma unroll
      for (int r = 0; r < R; ++r) wv[r][i] = u < units ? ld_w16<SMEM>(row[r] + (int64_t)(u >> 3) * 144 + 16 + (u & 7) * 16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      // The lane's 16 bytes hold values 64j+16h.. (low nibbles) and 64j+32+16h.. (high nibbles)
      // of superblock sb; for the mins term the lane owns 32-value group t.
      const int sb = u >> 3, t = u & 7, j = t >> 1, h = t & 1;
      float dw[R], dmw[R];
      int scl[R], sch[R], mt[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint4 meta = ld_a<SMEM>(reinterpret_cast<const uint4 *>(row[r] + (int64_t)sb * 144));
        dw[r] = f16_bits_to_f32((uint16_t)(meta.x & 0xffff));
        dmw[r] = f16_bits_to_f32((uint16_t)(meta.x >> 16));
        int unused;
        q4k_scale_min(2 * j, meta.y, meta.z, meta.w, scl[r], unused);
        q4k_scale_min(2 * j + 1, meta.y, meta.z, meta.w, sch[r], unused);
        q4k_scale_min(t, meta.y, meta.z, meta.w, unused, mt[r]);
      }
      uint4 lo[R], hi[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint4 w = wv[r][i];
        lo[r] = make_uint4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu);
        hi[r] = make_uint4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, (w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu);
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xlo = ld_a<SMEM>(reinterpret_cast<const int4 *>(a + sb * 256 + 64 * j + 16 * h));
        const int4 xhi = ld_a<SMEM>(reinterpret_cast<const int4 *>(a + sb * 256 + 64 * j + 32 + 16 * h));
        const float xd = ld_a<SMEM>(reinterpret_cast<const float *>(a + sc_off) + sb);
        const int bs2 = ld_a<SMEM>(reinterpret_cast<const int *>(a + bs_off) + sb * 8 + t);  // two i16 sums of group t
        const int bsum = (int)(short)(bs2 & 0xffff) + (bs2 >> 16);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int s = dot16(lo[r], xlo) * scl[r] + dot16(hi[r], xhi) * sch[r];
          const int p = bsum * mt[r];
          const float d = __fmul_rn(xd, dw[r]), dmin = __fmul_rn(xd, dmw[r]);
          acc[r][b] = __fmaf_rn(d, (float)s, __fmaf_rn(-dmin, (float)p, acc[r][b]));
        }
      }
    }
  }
}

template <int B, int R, int U, bool SMEM>
__device__ __forceinline__ void rows_q6_k(const uint8_t *const (&row)[R], int64_t cols, const uint8_t *act, int64_t act_stride,
                                          int lane, float (&acc)[R][B]) {
  const int nsb = (int)(cols >> 8);
  const int units = nsb * 8;
  const int64_t sc_off = act_scale_off(cols), bs_off = act_bsum_off(cols);
  for (int u0 = 0; u0 < units; u0 += 32 * U) {
    uint4 wl[R][U], wh[R][U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      const int sb = u >> 3, t = u & 7;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (u < units) {
          wl[r][i] = ld_w16<SMEM>(row[r] + (int64_t)sb * 208 + t * 16);
          // qh bytes for l = 16c.. of half h: shared by the two lanes s' = 0,1
          wh[r][i] = ld_a<SMEM>(reinterpret_cast<const uint4 *>(row[r] + (int64_t)sb * 208 + 128 + 32 * (t >> 2) + 16 * (t & 1)));
        } else {
          wl[r][i] = wh[r][i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u >= units) continue;
      // unit t of superblock sb: half h, ql sub-run s' (streams s' and s'+2), l = 16c..16c+15
      const int sb = u >> 3, t = u & 7, h = t >> 2, sp = (t >> 1) & 1, c = t & 1;
      const int jlo = 8 * h + 2 * sp + c;  // 16-value group of the low-nibble stream; the high stream is jlo + 4
      float dw[R];
      int slo[R], shi[R];
      uint4 qlo[R], qhi[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        dw[r] = f16_bits_to_f32(ld_a<SMEM>(reinterpret_cast<const uint16_t *>(row[r] + (int64_t)nsb * 208) + sb));
        const int8_t *sc = reinterpret_cast<const int8_t *>(row[r] + (int64_t)sb * 208 + 192);
        slo[r] = ld_a<SMEM>(sc + jlo);
        shi[r] = ld_a<SMEM>(sc + jlo + 4);
        const uint4 l4 = wl[r][i], h4 = wh[r][i];
        const int sh_lo = 2 * sp, sh_hi = 2 * sp + 4;
        qlo[r] = make_uint4((l4.x & 0x0f0f0f0fu) | (((h4.x >> sh_lo) & 0x03030303u) << 4),
                            (l4.y & 0x0f0f0f0fu) | (((h4.y >> sh_lo) & 0x03030303u) << 4),
                            (l4.z & 0x0f0f0f0fu) | (((h4.z >> sh_lo) & 0x03030303u) << 4),
                            (l4.w & 0x0f0f0f0fu) | (((h4.w >> sh_lo) & 0x03030303u) << 4));
        qhi[r] = make_uint4(((l4.x >> 4) & 0x0f0f0f0fu) | (((h4.x >> sh_hi) & 0x03030303u) << 4),
                            ((l4.y >> 4) & 0x0f0f0f0fu) | (((h4.y >> sh_hi) & 0x03030303u) << 4),
                            ((l4.z >> 4) & 0x0f0f0f0fu) | (((h4.z >> sh_hi) & 0x03030303u) << 4),
                            ((l4.w >> 4) & 0x0f0f0f0fu) | (((h4.w >> sh_hi) & 0x03030303u) << 4));
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *a = act + b * act_stride;
        const int4 xlo = ld_a<SMEM>(reinterpret_cast<const int4 *>(a + sb * 256 + jlo * 16));
        const int4 xhi = ld_a<SMEM>(reinterpret_cast<const int4 *>(a + sb * 256 + (jlo + 4) * 16));
        const float xd = ld_a<SMEM>(reinterpret_cast<const float *>(a + sc_off) + sb);
        const short *bs = reinterpret_cast<const short *>(a + bs_off) + sb * 16;
        const int blo = ld_a<SMEM>(bs + jlo), bhi = ld_a<SMEM>(bs + jlo + 4);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          // codes are stored +32: sum (q-32)*x = dot(q,x) - 32*sum(x)
          const int s = slo[r] * (dot16(qlo[r], xlo) - 32 * blo) + shi[r] * (dot16(qhi[r], xhi) - 32 * bhi);
          acc[r][b] = __fadd_rn(acc[r][b], __fmul_rn(__fmul_rn(dw[r], xd), (float)s));
        }
      }
    }
  }
}

}  // namespace cmld
