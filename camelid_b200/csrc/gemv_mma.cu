// Batched quantised matvec for 9..32 activation rows: the weights are streamed ONCE for all rows and the
// int8 x int8 block dot products run on the tensor cores (mma.sync m16n8k32 / m16n8k16, s8 x s8 -> s32).
//
// Same arithmetic as the row kernels (q4_k_q8_k_dot_rows / q6_k_q8_k_dot_rows / q8_0_dot_rows,
// src/inference.rs:23154-23520 and :26166 in the Camelid tree): integer dot per scale group, integer
// scale multiply, one f32 step per superblock (per block for Q8_0).  Only the order in which the
// superblocks' f32 terms of one row are added differs (here: in column order within a 1024-column
// chunk, chunks added in order), so results agree with the <= 8-row kernel up to f32 reassociation.
//
// Layout of the work: the columns are cut into chunks of 1024 (4 superblocks); a CTA owns ONE chunk for
// its whole life and keeps the quantised activations of that chunk for all rows in shared memory
// (32 x 1024 codes + scales), so the operand that every weight needs is loaded once per CTA.  Each warp
// works alone on units of 16 weight rows (one MMA row tile) of the CTA's chunk, for all <= 4 column
// tiles of 8 activation rows: no reduction across warps, no CTA barrier after the start.  A warp copies
// the next unit's chunk bytes into its second buffer with 16-byte asynchronous copies (cp.async) while
// it computes on the first — a row's chunk is only 576..1088 bytes, and one bulk (TMA) request per such
// piece was measured to cap the kernel at about 50 ns per request per SM; rows are padded in shared
// memory to a bank-conflict-free pitch.  With more than one chunk the per-chunk partial sums go to a
// scratch array and a small kernel adds them in chunk order (plus the residual).
#include "common.cuh"

namespace cmld {

constexpr int kMmaMaxWarps = 12;  // warps per CTA: as many as have room for their two buffers
constexpr int kMmaMaxThreads = kMmaMaxWarps * 32;
constexpr int kMmaChunkSb = 4;  // superblocks (of 256 columns) per chunk
constexpr int kMmaChunkCols = kMmaChunkSb * 256;
constexpr int kMmaCodeStride = kMmaChunkCols + 16;  // bytes between activation rows in shared memory (conflict-free)

namespace {

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// D(16x8, s32) = A(16x32, s8, row-major) * B(32x8, s8, column-major).  Lane (g = lane/4, t = lane%4) holds
// A: a0 = row g, k 4t..4t+3; a1 = row g+8, same k; a2 = row g, k 16+4t..; a3 = row g+8, k 16+4t..
// B: b0 = k 4t..4t+3 of column g; b1 = k 16+4t.. of column g
// D: d0,d1 = row g, columns 2t, 2t+1; d2,d3 = row g+8, columns 2t, 2t+1
__device__ __forceinline__ void mma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
// D(16x8) = A(16x16) * B(16x8): a0 = row g, k 4t..4t+3; a1 = row g+8; b0 = k 4t..4t+3 of column g.
__device__ __forceinline__ void mma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

struct MmaJob {
  const uint8_t *w;
  int32_t qt, rows, first_tile, n_tiles, row_off;
  int64_t stride;
  float *y;
  const float *residual;
  int64_t y_stride;
};

struct MmaArgs {
  MmaJob job[3];
  int32_t n_jobs, total_tiles, cols, batch, n_chunks, ctas_per_chunk, stage_bytes, n_warps, rows_cat, q8_0;
  const uint8_t *act;  // quantised activation rows, global layout, the format the jobs' types need
  float *partial;      // [chunk][batch][rows_cat] when n_chunks > 1
  int32_t *status;
  int32_t off_codes, off_scale, off_bsum, off_ring;
  // expert mode (counts != null): blockIdx.y = local expert, blockIdx.z = pass of NT*8 activation rows.  Expert e's
  // matrices are rows [e*rows, (e+1)*rows) of each slab, its activation rows start at row e*cap of `act`, its
  // results at row e*cap of y, and only count_mul * counts[first_expert + e*expert_step] of them exist.
  const int32_t *counts;
  int32_t first_expert, expert_step, cap, count_mul;
};

// bytes of one weight row's chunk in shared memory (padded so that 8 rows x 4 words hit 32 distinct banks)
constexpr int kMmaPieceSb = 2;  // superblocks a warp buffers at a time (half a chunk)
__host__ __device__ inline int row_pitch(int qt) {
  return (qt == CMLD_Q4_K ? kMmaPieceSb * 144 : (qt == CMLD_Q6_K ? kMmaPieceSb * 208 : kMmaPieceSb * 256 + kMmaPieceSb * 16)) + 16;
}

// Byte k of w as an int (0..255).
__device__ __forceinline__ int byte_of(uint32_t w, int k) { return (int)((w >> (8 * k)) & 0xffu); }

template <int NT>
__device__ __forceinline__ void tile_q4k(const uint8_t *tile, int sbo, int ns, int lane, const uint8_t *codes, const float *xd,
                                         const int8_t *bs_hi, const int8_t *bs_lo, float (&acc)[NT][4]) {
  constexpr int m0 = 0;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int pitch = row_pitch(CMLD_Q4_K);
  const uint8_t *rlo = tile + (m0 + g8) * pitch, *rhi = rlo + 8 * pitch;
  for (int sb = 0; sb < ns; ++sb) {
    const uint8_t *plo = rlo + sb * 144, *phi = rhi + sb * 144;
    const uint4 mlo = *reinterpret_cast<const uint4 *>(plo), mhi = *reinterpret_cast<const uint4 *>(phi);
    // the eight 6-bit scales and mins of the superblock, unpacked four at a time into bytes
    // (q4_k_scale_min, src/tensor/mod.rs:5997-6006): groups 0-3 and groups 4-7
    const uint32_t sc_lo[2] = {mlo.y & 0x3f3f3f3fu, (mlo.w & 0x0f0f0f0fu) | (((mlo.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn_lo[2] = {mlo.z & 0x3f3f3f3fu, ((mlo.w >> 4) & 0x0f0f0f0fu) | (((mlo.z >> 6) & 0x03030303u) << 4)};
    const uint32_t sc_hi[2] = {mhi.y & 0x3f3f3f3fu, (mhi.w & 0x0f0f0f0fu) | (((mhi.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn_hi[2] = {mhi.z & 0x3f3f3f3fu, ((mhi.w >> 4) & 0x0f0f0f0fu) | (((mhi.z >> 6) & 0x03030303u) << 4)};
    int isum[NT][4], msum[NT][4];
    {
      // sum_g min_g * bsum32_g as one more small matrix product: A = the mins (k = group, 8 of the 16 used),
      // B = the group sums of the activation codes, split as 64*hi + lo to fit int8
      const uint32_t a0 = t4 == 0 ? mn_lo[0] : (t4 == 1 ? mn_lo[1] : 0u), a1 = t4 == 0 ? mn_hi[0] : (t4 == 1 ? mn_hi[1] : 0u);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int o = ((nt * 8 + g8) * kMmaChunkSb + sbo + sb) * 8 + (t4 & 1) * 4;
        int ch[4], cl[4];
        mma_k16(ch, a0, a1, *reinterpret_cast<const uint32_t *>(bs_hi + o));
        mma_k16(cl, a0, a1, *reinterpret_cast<const uint32_t *>(bs_lo + o));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          msum[nt][i] = 64 * ch[i] + cl[i];
          isum[nt][i] = 0;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t wl0 = *reinterpret_cast<const uint32_t *>(plo + 16 + j * 32 + t4 * 4);
      const uint32_t wl1 = *reinterpret_cast<const uint32_t *>(plo + 16 + j * 32 + 16 + t4 * 4);
      const uint32_t wh0 = *reinterpret_cast<const uint32_t *>(phi + 16 + j * 32 + t4 * 4);
      const uint32_t wh1 = *reinterpret_cast<const uint32_t *>(phi + 16 + j * 32 + 16 + t4 * 4);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int g = 2 * j + h;
        const int s_lo = byte_of(sc_lo[g >> 2], g & 3), s_hi = byte_of(sc_hi[g >> 2], g & 3);
        const uint32_t a0 = (wl0 >> (4 * h)) & 0x0f0f0f0fu, a1 = (wh0 >> (4 * h)) & 0x0f0f0f0fu;
        const uint32_t a2 = (wl1 >> (4 * h)) & 0x0f0f0f0fu, a3 = (wh1 >> (4 * h)) & 0x0f0f0f0fu;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint8_t *xc = codes + (nt * 8 + g8) * kMmaCodeStride + (sbo + sb) * 256 + g * 32 + t4 * 4;
          const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xc), b1 = *reinterpret_cast<const uint32_t *>(xc + 16);
          int c[4];
          mma_k32(c, a0, a1, a2, a3, b0, b1);
          isum[nt][0] += s_lo * c[0];
          isum[nt][1] += s_lo * c[1];
          isum[nt][2] += s_hi * c[2];
          isum[nt][3] += s_hi * c[3];
        }
      }
    }
    const float d_lo = f16_bits_to_f32((uint16_t)(mlo.x & 0xffff)), dm_lo = f16_bits_to_f32((uint16_t)(mlo.x >> 16));
    const float d_hi = f16_bits_to_f32((uint16_t)(mhi.x & 0xffff)), dm_hi = f16_bits_to_f32((uint16_t)(mhi.x >> 16));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x = xd[(nt * 8 + t4 * 2 + (i & 1)) * kMmaChunkSb + sbo + sb];
        const float d = i < 2 ? d_lo : d_hi, dm = i < 2 ? dm_lo : dm_hi;
        // src/inference.rs:23230-23236: sumf = fma(-dmin*xd, mins, sumf); sumf = fma(d*xd, dots, sumf)
        acc[nt][i] = __fmaf_rn(-__fmul_rn(dm, x), (float)msum[nt][i], acc[nt][i]);
        acc[nt][i] = __fmaf_rn(__fmul_rn(d, x), (float)isum[nt][i], acc[nt][i]);
      }
  }
}

template <int NT>
__device__ __forceinline__ void tile_q6k(const uint8_t *tile, int sbo, int ns, int lane, const uint8_t *codes, const float *xd,
                                         const int8_t *b16_hi, const int8_t *b16_lo, float d_lo[kMmaPieceSb], float d_hi[kMmaPieceSb],
                                         float (&acc)[NT][4]) {
  constexpr int m0 = 0;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int pitch = row_pitch(CMLD_Q6_K);
  const uint8_t *rlo = tile + (m0 + g8) * pitch, *rhi = rlo + 8 * pitch;
  for (int sb = 0; sb < ns; ++sb) {
    const uint8_t *plo = rlo + sb * 208, *phi = rhi + sb * 208;
    int isum[NT][4];
    {
      // codes are stored +32: sum_s sc_s * sum (q-32) x = sum_s sc_s * dot_s - 32 * sum_s sc_s * bsum16_s, and the
      // last sum is one more small matrix product: A = the 16 int8 scales, B = the 16-sums of the activation
      // codes split as 64*hi + lo
      const uint32_t a0 = *reinterpret_cast<const uint32_t *>(plo + 192 + t4 * 4), a1 = *reinterpret_cast<const uint32_t *>(phi + 192 + t4 * 4);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int o = ((nt * 8 + g8) * kMmaChunkSb + sbo + sb) * 16 + t4 * 4;
        int ch[4], cl[4];
        mma_k16(ch, a0, a1, *reinterpret_cast<const uint32_t *>(b16_hi + o));
        mma_k16(cl, a0, a1, *reinterpret_cast<const uint32_t *>(b16_lo + o));
#pragma unroll
        for (int i = 0; i < 4; ++i) isum[nt][i] = -32 * (64 * ch[i] + cl[i]);
      }
    }
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      // sub-block s of 16 values: half n, quarter qd (which 2 bits of qh, which nibble of which ql half), part lp
      const int n = s >> 3, qd = (s & 7) >> 1, lp = s & 1;
      const int qlo = n * 64 + (qd & 1) * 32 + 16 * lp + t4 * 4, qho = 128 + n * 32 + 16 * lp + t4 * 4;
      const uint32_t wl = *reinterpret_cast<const uint32_t *>(plo + qlo), wlh = *reinterpret_cast<const uint32_t *>(plo + qho);
      const uint32_t wh = *reinterpret_cast<const uint32_t *>(phi + qlo), whh = *reinterpret_cast<const uint32_t *>(phi + qho);
      const uint32_t a0 = ((wl >> (4 * (qd >> 1))) & 0x0f0f0f0fu) | (((wlh >> (2 * qd)) & 0x03030303u) << 4);
      const uint32_t a1 = ((wh >> (4 * (qd >> 1))) & 0x0f0f0f0fu) | (((whh >> (2 * qd)) & 0x03030303u) << 4);
      const int sc_lo = (int)reinterpret_cast<const int8_t *>(plo + 192)[s], sc_hi = (int)reinterpret_cast<const int8_t *>(phi + 192)[s];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(codes + (nt * 8 + g8) * kMmaCodeStride + (sbo + sb) * 256 + s * 16 + t4 * 4);
        int c[4];
        mma_k16(c, a0, a1, b0);
        isum[nt][0] += sc_lo * c[0];
        isum[nt][1] += sc_lo * c[1];
        isum[nt][2] += sc_hi * c[2];
        isum[nt][3] += sc_hi * c[3];
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x = xd[(nt * 8 + t4 * 2 + (i & 1)) * kMmaChunkSb + sbo + sb];
        acc[nt][i] = __fadd_rn(acc[nt][i], __fmul_rn(__fmul_rn(i < 2 ? d_lo[sb] : d_hi[sb], x), (float)isum[nt][i]));
      }
  }
}

template <int NT>
__device__ __forceinline__ void tile_q80(const uint8_t *tile, int sbo, int ns, int lane, const uint8_t *codes, const float *xs,
                                         float (&acc)[NT][4]) {
  constexpr int m0 = 0;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int pitch = row_pitch(CMLD_Q8_0);
  const uint8_t *rlo = tile + (m0 + g8) * pitch, *rhi = rlo + 8 * pitch;
  for (int blk = 0; blk < ns * 8; ++blk) {
    const uint32_t a0 = *reinterpret_cast<const uint32_t *>(rlo + blk * 32 + t4 * 4), a2 = *reinterpret_cast<const uint32_t *>(rlo + blk * 32 + 16 + t4 * 4);
    const uint32_t a1 = *reinterpret_cast<const uint32_t *>(rhi + blk * 32 + t4 * 4), a3 = *reinterpret_cast<const uint32_t *>(rhi + blk * 32 + 16 + t4 * 4);
    const float ws_lo = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(rlo + ns * 256 + blk * 2));
    const float ws_hi = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(rhi + ns * 256 + blk * 2));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint8_t *xc = codes + (nt * 8 + g8) * kMmaCodeStride + sbo * 256 + blk * 32 + t4 * 4;
      const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xc), b1 = *reinterpret_cast<const uint32_t *>(xc + 16);
      int c[4];
      mma_k32(c, a0, a1, a2, a3, b0, b1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x = xs[(nt * 8 + t4 * 2 + (i & 1)) * (kMmaChunkSb * 8) + sbo * 8 + blk];
        acc[nt][i] = __fadd_rn(acc[nt][i], __fmul_rn(__fmul_rn((float)c[i], i < 2 ? ws_lo : ws_hi), x));  // src/inference.rs:26198
      }
    }
  }
}

// 16-byte asynchronous global->shared copy (LDGSTS); the data is only read once, so it bypasses L1.
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Which matrix and which 16 rows unit u of the launch is.
struct MmaUnit {
  int j, row0, nrows;
};
__device__ __forceinline__ MmaUnit unit_of(const MmaArgs &a, int u) {
  int j = 0;
  if (a.n_jobs > 1 && u >= a.job[1].first_tile) j = 1;
  if (a.n_jobs > 2 && u >= a.job[2].first_tile) j = 2;
  MmaUnit m;
  m.j = j;
  m.row0 = (u - a.job[j].first_tile) * 16;
  m.nrows = min(16, a.job[j].rows - m.row0);
  return m;
}

// This warp's copy of one piece (kMmaPieceSb superblocks of the chunk, `np` of them real) of 16 weight rows
// into one of its buffers: 16-byte pieces, lanes running along a row, rows padded to the conflict-free pitch.
__device__ __forceinline__ void fetch_piece(const MmaArgs &a, const MmaUnit &m, int64_t row_base, int sb_first, int np, int lane,
                                            uint8_t *buf) {
  const MmaJob &J = a.job[m.j];
  const int pitch = row_pitch(J.qt);
  const int seg = J.qt == CMLD_Q4_K ? np * 9 : (J.qt == CMLD_Q6_K ? np * 13 : np * 16);  // 16-byte pieces of the block bytes
  const int64_t off = (int64_t)sb_first * (J.qt == CMLD_Q4_K ? 144 : (J.qt == CMLD_Q6_K ? 208 : 256));
  const int extra = J.qt == CMLD_Q8_0 ? np : 0;  // pieces of the per-block f16 scales behind the codes
  const int per_row = seg + extra;
  for (int i = lane; i < m.nrows * per_row; i += 32) {
    const int r = i / per_row, c = i % per_row;
    const uint8_t *row = J.w + (row_base * J.rows + m.row0 + r) * J.stride;
    const uint8_t *src = c < seg ? row + off + c * 16 : row + a.cols + (int64_t)sb_first * 16 + (c - seg) * 16;
    cp_async16(buf + r * pitch + c * 16, src);
  }
}

template <int NT>
__global__ void __launch_bounds__(kMmaMaxThreads, 1) gemv_mma_kernel(const MmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *codes = smem + a.off_codes;
  float *xscale = reinterpret_cast<float *>(smem + a.off_scale);
  // sums of the activation codes per 32 (Q4_K mins) and per 16 (Q6_K offset), each split as 64*hi + lo
  int8_t *bs32_hi = reinterpret_cast<int8_t *>(smem + a.off_bsum), *bs32_lo = bs32_hi + NT * 8 * kMmaChunkSb * 8;
  int8_t *bs16_hi = bs32_lo + NT * 8 * kMmaChunkSb * 8, *bs16_lo = bs16_hi + NT * 8 * kMmaChunkSb * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_warps = (int)blockDim.x >> 5, n_consumers = (int)blockDim.x;
  const int chunk = (int)blockIdx.x % a.n_chunks, slot = (int)blockIdx.x / a.n_chunks;
  const int nsb = a.cols >> 8;
  const int sb0 = chunk * kMmaChunkSb, ns = min(kMmaChunkSb, nsb - sb0);
  // units of 16 weight rows; this warp takes units first, first + stride, ...
  const int first = slot * n_warps + warp, stride = a.ctas_per_chunk * n_warps;
  uint8_t *buf0 = smem + a.off_ring + warp * 2 * a.stage_bytes, *buf1 = buf0 + a.stage_bytes;
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t astride = act_row_stride(a.cols);
  constexpr int NB = NT * 8;
  int batch = a.batch, pb = a.batch;  // rows of this launch; rows per chunk in the partial-sum layout
  int64_t e_local = 0, y_base = 0;
  const uint8_t *act = a.act;
  float *partial = a.partial;
  if (a.counts) {
    // how many rows this expert has is written by the kernel before: nothing can start before the wait
    asm volatile("griddepcontrol.wait;" ::: "memory");
    e_local = blockIdx.y;
    const int col0 = (int)blockIdx.z * NB;
    batch = min(NB, a.count_mul * __ldcg(a.counts + a.first_expert + (int)e_local * a.expert_step) - col0);
    if (batch <= 0) return;
    pb = NB;
    act += (e_local * a.cap + col0) * astride;
    y_base = e_local * a.cap + col0;
    partial += (e_local * gridDim.z + blockIdx.z) * (int64_t)a.n_chunks * NB * a.rows_cat;
  }
  // a unit (16 rows x this chunk) is worked through in pieces of kMmaPieceSb superblocks: trip `it` handles piece
  // it % n_pieces of unit first + (it / n_pieces) * stride, while the copy of trip it+1 is in flight
  const int n_pieces = (ns + kMmaPieceSb - 1) / kMmaPieceSb;
  const int n_units = first < a.total_tiles ? (a.total_tiles - first + stride - 1) / stride : 0;
  const int n_trips = n_units * n_pieces;
  // weights do not depend on the previous kernel: the first piece's copy is in flight before the wait
  if (n_trips > 0) fetch_piece(a, unit_of(a, first), e_local, sb0, min(kMmaPieceSb, ns), lane, buf0);
  cp_async_commit();
  if (!a.counts) asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---------------- this chunk's activations for every row into shared memory, once
  // (flat loops: every thread has several independent loads in flight; a loop over the rows with one row
  // per trip would serialise 32 round trips to L2)
  for (int idx = tid; idx < NB * (kMmaChunkCols / 16); idx += n_consumers) {
    const int b = idx / (kMmaChunkCols / 16), i = idx % (kMmaChunkCols / 16);
    uint4 v = make_uint4(0, 0, 0, 0);  // padding rows of the last column tile and the columns beyond a short chunk
    if (b < batch && i < ns * 16) v = __ldg(reinterpret_cast<const uint4 *>(act + b * astride + (int64_t)sb0 * 256) + i);
    *reinterpret_cast<uint4 *>(codes + b * kMmaCodeStride + i * 16) = v;
  }
  if (a.q8_0) {
    for (int idx = tid; idx < NB * (kMmaChunkSb * 8); idx += n_consumers) {
      const int b = idx / (kMmaChunkSb * 8), i = idx % (kMmaChunkSb * 8);
      float v = 0.0f;
      if (b < batch && i < ns * 8) v = __ldg(reinterpret_cast<const float *>(act + b * astride + act_scale_off(a.cols)) + sb0 * 8 + i);
      xscale[idx] = v;
    }
  } else {
    for (int idx = tid; idx < NB * kMmaChunkSb; idx += n_consumers) {
      const int b = idx / kMmaChunkSb, i = idx % kMmaChunkSb;
      float v = 0.0f;
      if (b < batch && i < ns) v = __ldg(reinterpret_cast<const float *>(act + b * astride + act_scale_off(a.cols)) + sb0 + i);
      xscale[idx] = v;
    }
    for (int idx = tid; idx < NB * (kMmaChunkSb * 8); idx += n_consumers) {
      const int b = idx / (kMmaChunkSb * 8), i = idx % (kMmaChunkSb * 8);
      int v0 = 0, v1 = 0;
      if (b < batch && i < ns * 8) {
        const int pr = __ldg(reinterpret_cast<const int *>(act + b * astride + act_bsum_off(a.cols)) + sb0 * 8 + i);  // two 16-sums
        v0 = (int)(short)(pr & 0xffff);
        v1 = pr >> 16;
      }
      const int l0 = ((v0 + 32) & 63) - 32, l1 = ((v1 + 32) & 63) - 32;
      bs16_lo[b * (kMmaChunkSb * 16) + 2 * i] = (int8_t)l0;
      bs16_hi[b * (kMmaChunkSb * 16) + 2 * i] = (int8_t)((v0 - l0) / 64);
      bs16_lo[b * (kMmaChunkSb * 16) + 2 * i + 1] = (int8_t)l1;
      bs16_hi[b * (kMmaChunkSb * 16) + 2 * i + 1] = (int8_t)((v1 - l1) / 64);
      const int v = v0 + v1, lo = ((v + 32) & 63) - 32;
      bs32_lo[idx] = (int8_t)lo;
      bs32_hi[idx] = (int8_t)((v - lo) / 64);
    }
  }
  __syncthreads();

  const int g8 = lane >> 2, t4 = lane & 3;
  float acc[NT][4];
  for (int it = 0; it < n_trips; ++it) {
    uint8_t *cur = (it & 1) ? buf1 : buf0, *nxt = (it & 1) ? buf0 : buf1;
    if (it + 1 < n_trips) {
      const int pc = (it + 1) % n_pieces;
      fetch_piece(a, unit_of(a, first + ((it + 1) / n_pieces) * stride), e_local, sb0 + pc * kMmaPieceSb,
                  min(kMmaPieceSb, ns - pc * kMmaPieceSb), lane, nxt);
    }
    cp_async_commit();
    cp_async_wait<1>();  // everything but the copy just issued has landed: this trip's piece is complete
    __syncwarp();
    const int piece = it % n_pieces, sbo = piece * kMmaPieceSb, np = min(kMmaPieceSb, ns - sbo);
    const MmaUnit m = unit_of(a, first + (it / n_pieces) * stride);
    const MmaJob &J = a.job[m.j];
    if (piece == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[nt][k] = 0.0f;
    }
    // rows beyond the matrix were not copied: their slots hold stale bytes; the integer and f32 work on
    // them is harmless and their results are not written
    if (J.qt == CMLD_Q4_K) {
      tile_q4k<NT>(cur, sbo, np, lane, codes, xscale, bs32_hi, bs32_lo, acc);
    } else if (J.qt == CMLD_Q6_K) {
      float d_lo[kMmaPieceSb], d_hi[kMmaPieceSb];
      const int r_lo = min(m.row0 + g8, J.rows - 1), r_hi = min(m.row0 + g8 + 8, J.rows - 1);
#pragma unroll
      for (int sb = 0; sb < kMmaPieceSb; ++sb) {
        const int sbc = min(sbo + sb, ns - 1);
        d_lo[sb] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(J.w + (e_local * J.rows + r_lo) * J.stride + (int64_t)nsb * 208) + sb0 + sbc));
        d_hi[sb] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(J.w + (e_local * J.rows + r_hi) * J.stride + (int64_t)nsb * 208) + sb0 + sbc));
      }
      tile_q6k<NT>(cur, sbo, np, lane, codes, xscale, bs16_hi, bs16_lo, d_lo, d_hi, acc);
    } else {
      tile_q80<NT>(cur, sbo, np, lane, codes, xscale, acc);
    }
    __syncwarp();  // every lane is done with `cur` before the next trip's copy overwrites it
    if (piece + 1 < n_pieces) continue;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int col = nt * 8 + t4 * 2 + (k & 1), r = g8 + (k >= 2 ? 8 : 0);
        if (col < batch && r < m.nrows) {
          if (a.n_chunks == 1) {
            const int64_t o = (y_base + col) * J.y_stride + m.row0 + r;
            J.y[o] = J.residual ? __fadd_rn(__ldcg(J.residual + o), acc[nt][k]) : acc[nt][k];
          } else {
            partial[((int64_t)chunk * pb + col) * a.rows_cat + J.row_off + m.row0 + r] = acc[nt][k];
          }
        }
      }
  }
  cp_async_wait<0>();
}

// y = residual + sum over chunks (in chunk order) of the partial sums.
__global__ void mma_reduce_kernel(const MmaArgs a, int nb) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  int batch = a.batch, pb = a.batch;
  int64_t y_base = 0;
  const float *partial = a.partial;
  if (a.counts) {
    const int64_t e_local = blockIdx.y;
    const int col0 = (int)blockIdx.z * nb;
    batch = min(nb, a.count_mul * __ldcg(a.counts + a.first_expert + (int)e_local * a.expert_step) - col0);
    if (batch <= 0) return;
    pb = nb;
    y_base = e_local * a.cap + col0;
    partial += (e_local * gridDim.z + blockIdx.z) * (int64_t)a.n_chunks * nb * a.rows_cat;
  }
  const int64_t total = (int64_t)batch * a.rows_cat;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int col = (int)(i / a.rows_cat), rc = (int)(i % a.rows_cat);
    int j = 0;
    if (a.n_jobs > 1 && rc >= a.job[1].row_off) j = 1;
    if (a.n_jobs > 2 && rc >= a.job[2].row_off) j = 2;
    const MmaJob &J = a.job[j];
    const int64_t o = (y_base + col) * J.y_stride + (rc - J.row_off);
    float v = __ldcg(partial + (int64_t)col * a.rows_cat + rc);
    for (int c = 1; c < a.n_chunks; ++c) v = __fadd_rn(v, __ldcg(partial + ((int64_t)c * pb + col) * a.rows_cat + rc));
    J.y[o] = J.residual ? __fadd_rn(__ldcg(J.residual + o), v) : v;
  }
}

struct MmaPlan {
  MmaArgs args;
  int smem_bytes, grid, grid_y = 1, grid_z = 1;
};

int g_mma_sms = 0;
bool g_mma_attr[5] = {false, false, false, false, false};

bool plan_mma(const GemvJob *jobs, int n_jobs, int32_t batch, MmaPlan &p) {
  if (n_jobs < 1 || n_jobs > 3 || batch < 1 || batch > 32) return false;
  const int64_t cols = jobs[0].cols;
  if (cols % 256) return false;
  MmaArgs &a = p.args;
  const bool q80 = jobs[0].qt == CMLD_Q8_0;
  int tiles = 0, stage = 0, rows_cat = 0;
  for (int k = 0; k < n_jobs; ++k) {
    const GemvJob &g = jobs[k];
    if (g.cols != cols) return false;
    if (g.qt != CMLD_Q8_0 && g.qt != CMLD_Q4_K && g.qt != CMLD_Q6_K) return false;
    if ((g.qt == CMLD_Q8_0) != q80) return false;  // one activation format per launch
    if (g.stride % 16 || (reinterpret_cast<uintptr_t>(g.w) & 15)) return false;
    MmaJob &J = a.job[k];
    J.w = g.w;
    J.qt = g.qt;
    J.rows = (int32_t)g.rows;
    J.stride = g.stride;
    J.y = g.y;
    J.residual = g.residual;
    J.y_stride = g.y_stride;
    J.first_tile = tiles;
    J.n_tiles = (int)((g.rows + 15) / 16);  // units of 16 rows: one MMA row tile, one warp
    J.row_off = rows_cat;
    tiles += J.n_tiles;
    rows_cat += (int)g.rows;
    stage = std::max(stage, 16 * row_pitch(g.qt));
  }
  stage = (stage + 127) & ~127;
  const int nt = (batch + 7) / 8;
  int off = 0;
  a.off_codes = off;
  off += nt * 8 * kMmaCodeStride;
  a.off_scale = off;
  off += nt * 8 * (q80 ? kMmaChunkSb * 8 : kMmaChunkSb) * 4;
  a.off_bsum = off;
  if (!q80) off += nt * 8 * kMmaChunkSb * (8 + 8 + 16 + 16);
  off = (off + 127) & ~127;
  a.off_ring = off;
  // every warp owns two buffers of 16 row chunks (the one it computes on and the one being filled)
  int n_warps = std::min<int>(kMmaMaxWarps, (224 * 1024 - off) / (2 * stage));
  if (const char *v = getenv("CMLD_MMA_WARPS")) n_warps = std::max(1, std::min(n_warps, atoi(v)));  // A/B runs
  if (n_warps < 2) return false;
  a.n_warps = n_warps;
  a.stage_bytes = stage;
  a.n_jobs = n_jobs;
  a.total_tiles = tiles;
  a.cols = (int32_t)cols;
  a.batch = batch;
  a.rows_cat = rows_cat;
  a.q8_0 = q80 ? 1 : 0;
  a.n_chunks = (int)((cols / 256 + kMmaChunkSb - 1) / kMmaChunkSb);
  a.ctas_per_chunk = std::max(1, std::min((tiles + n_warps - 1) / n_warps, g_mma_sms / a.n_chunks));
  p.grid = a.n_chunks * a.ctas_per_chunk;
  p.smem_bytes = off + n_warps * 2 * stage;
  return true;
}

template <int NT>
int32_t launch_nt(const MmaPlan &p, cudaStream_t s, bool pdl) {
  if (!g_mma_attr[NT]) {
    CMLD_CUDA(cudaFuncSetAttribute(gemv_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    g_mma_attr[NT] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)p.grid, (unsigned)p.grid_y, (unsigned)p.grid_z);
  cfg.blockDim = dim3((unsigned)(p.args.n_warps * 32));
  cfg.dynamicSmemBytes = (size_t)p.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, gemv_mma_kernel<NT>, p.args));
  return CMLD_OK;
}

int32_t launch_reduce(const MmaPlan &p, int nb, cudaStream_t s, bool pdl) {
  cudaLaunchConfig_t cfg{};
  const int64_t total = (int64_t)std::min(nb, p.args.counts ? nb : p.args.batch) * p.args.rows_cat;
  cfg.gridDim = dim3((unsigned)std::min<int64_t>((total + 255) / 256, p.args.counts ? 64 : 4 * 148), (unsigned)p.grid_y, (unsigned)p.grid_z);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, mma_reduce_kernel, p.args, nb));
  return CMLD_OK;
}

}  // namespace

// Floats of scratch a launch needs for its per-chunk partial sums (0 when the columns fit one chunk);
// -1 when the matrices do not fit this kernel.
int64_t gemv_mma_scratch_floats(const GemvJob *jobs, int n_jobs, int32_t batch) {
  if (g_mma_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_mma_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
  }
  MmaPlan p{};
  if (!plan_mma(jobs, n_jobs, batch, p)) return -1;
  return p.args.n_chunks > 1 ? (int64_t)p.args.n_chunks * batch * p.args.rows_cat : 0;
}

// `act`: the quantised activation rows in the global layout (Q8_0 rows for Q8_0 matrices, Q8_K rows
// otherwise).  Returns CMLD_ERR_UNSUPPORTED without a message when the shapes do not fit.
int32_t launch_gemv_mma(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, float *scratch, int64_t scratch_floats,
                        int32_t *status, cudaStream_t s, bool pdl, int64_t *launches) {
  const int64_t need = gemv_mma_scratch_floats(jobs, n_jobs, batch);
  if (need < 0) return CMLD_ERR_UNSUPPORTED;
  if (need > scratch_floats || (need > 0 && !scratch)) return CMLD_ERR_UNSUPPORTED;
  if (!act) return fail(CMLD_ERR_INVALID, "gemv: activation buffer missing");
  MmaPlan p{};
  plan_mma(jobs, n_jobs, batch, p);
  p.args.act = act;
  p.args.partial = scratch;
  p.args.status = status;
  const int nt = (batch + 7) / 8;
  int32_t rc;
  switch (nt) {
    case 1: rc = launch_nt<1>(p, s, pdl); break;
    case 2: rc = launch_nt<2>(p, s, pdl); break;
    case 3: rc = launch_nt<3>(p, s, pdl); break;
    default: rc = launch_nt<4>(p, s, pdl); break;
  }
  CMLD_TRY(rc);
  if (launches) *launches += 1;
  if (p.args.n_chunks > 1) {
    CMLD_TRY(launch_reduce(p, nt * 8, s, pdl));
    if (launches) *launches += 1;
  }
  return CMLD_OK;
}

// Expert form: `jobs` describe ONE expert's matrices (rows per expert; the slabs hold n_experts of them one
// after the other), `act` holds `cap` activation rows per local expert of which count_mul * counts[e] are
// real, y receives `cap` result rows per local expert.  nt column tiles (8 rows each) per pass, n_pass passes
// (those beyond an expert's rows exit at once).  scratch: gemv_mma_expert_scratch_floats.
int64_t gemv_mma_expert_scratch_floats(const GemvJob *jobs, int n_jobs, int nt, int n_experts, int n_pass) {
  const int64_t one = gemv_mma_scratch_floats(jobs, n_jobs, nt * 8);
  return one < 0 ? -1 : one * n_experts * n_pass;
}

int32_t launch_gemv_mma_experts(const GemvJob *jobs, int n_jobs, const uint8_t *act, int nt, int n_experts, int n_pass,
                                const int32_t *counts, int first_expert, int expert_step, int cap, int count_mul, float *scratch,
                                int64_t scratch_floats, int32_t *status, cudaStream_t s, bool pdl, int64_t *launches) {
  const int64_t need = gemv_mma_expert_scratch_floats(jobs, n_jobs, nt, n_experts, n_pass);
  if (need < 0 || need > scratch_floats || (need > 0 && !scratch)) return CMLD_ERR_UNSUPPORTED;
  if (!act || !counts || nt < 1 || nt > 4) return fail(CMLD_ERR_INVALID, "expert matvec: bad arguments");
  MmaPlan p{};
  plan_mma(jobs, n_jobs, nt * 8, p);
  MmaArgs &a = p.args;
  a.act = act;
  a.partial = scratch;
  a.status = status;
  a.counts = counts;
  a.first_expert = first_expert;
  a.expert_step = expert_step;
  a.cap = cap;
  a.count_mul = count_mul;
  // all experts stream at once: share the SMs between them
  a.ctas_per_chunk = std::max(1, std::min((a.total_tiles + a.n_warps - 1) / a.n_warps, g_mma_sms / (a.n_chunks * std::max(1, n_experts))));
  p.grid = a.n_chunks * a.ctas_per_chunk;
  p.grid_y = n_experts;
  p.grid_z = n_pass;
  int32_t rc;
  switch (nt) {
    case 1: rc = launch_nt<1>(p, s, pdl); break;
    case 2: rc = launch_nt<2>(p, s, pdl); break;
    case 3: rc = launch_nt<3>(p, s, pdl); break;
    default: rc = launch_nt<4>(p, s, pdl); break;
  }
  CMLD_TRY(rc);
  if (launches) *launches += 1;
  if (a.n_chunks > 1) {
    CMLD_TRY(launch_reduce(p, nt * 8, s, pdl));
    if (launches) *launches += 1;
  }
  return CMLD_OK;
}

}  // namespace cmld
