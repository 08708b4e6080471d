// Staged quantised matvec for sm_100a: the fast path of the decode step.
//
// Why this shape.  A decode matvec reads every weight byte once and does ~1 integer MAC per
// 4 bits: it is HBM-bound and uses no tensor cores.  What limits a simple kernel on B200 is
// the number of bytes in flight (Little's law at ~6.5 TB/s needs > 40 KB per SM) and the gaps
// between dependent launches.  So:
//   * one persistent CTA per SM walks its share of row tiles; a tile of consecutive rows is one
//     contiguous byte range of the device layout, fetched by ONE bulk asynchronous copy
//     (cp.async.bulk, the non-tensor TMA path) into a shared-memory ring of up
//     to 8 stages guarded by mbarriers (full: transaction bytes, empty: one arrival per warp);
//   * a dedicated producer warp issues the copies; it starts BEFORE the kernel waits on its
//     predecessor (griddepcontrol.wait), because weights never depend on earlier kernels — under
//     programmatic dependent launch the ring fills while the previous kernel drains;
//   * the consumer warps first build the quantised activation in shared memory — optionally
//     fused with RMSNorm or SwiGLU so no separate kernel and no global round trip is needed —
//     then each lane owns whole superblocks (Q4_K/Q6_K) or 32-value blocks (Q8_0): one f16->f32
//     and one int->f32 conversion per superblock instead of per 16 bytes, scales decoded once;
//   * per-superblock integer sums and the two f32 multiply-adds are exactly the CPU's
//     (q4_k_dot_scalar, src/diffusion_gemma/refmath.rs:504-562; q6_k_wire_row_dot and
//     q8_0_dot_rows, src/inference.rs:25535 and :26166 in the Camelid tree); lanes are combined
//     by a fixed shuffle tree, so results are deterministic and differ from the CPU's
//     block-ordered sum only by f32 reassociation.
//
//   * sixteen consumer warps in two groups that alternate tiles (a stage belongs to one group: the stage count
//     is a multiple of the group count, see plan_pipe);
//   * paired mode (gate and up of an FFN): tiles 2k and 2k+1 of a CTA are the same rows of the two matrices,
//     the two groups take them at the same time and the first writes SwiGLU(first, second);
//   * peer mode (tensor parallel): the epilogue stores this rank's partial rows into a slot on every rank and
//     the last CTA raises arrival words; the next launch's prologue waits for all ranks' words and takes the
//     sum of the partial rows as its RMSNorm input — the all-reduce of the sublayer without a collective kernel.
//
// Every wait (mbarrier, arrival word) is bounded: when the bound passes a thread records
// CMLD_ERR_TIMEOUT in *status and carries on (results are then invalid, the host reports the
// error), so a lost copy or a peer that went away can never hang the GPU.
#include "actquant.cuh"

namespace cmld {

constexpr int kPipeConsumerWarps = 8;  // warps that share one tile
constexpr int kPipeGroups = 2;         // consumer groups; group g takes this CTA's tiles g, g+2, ... (more warps to hide latency)
constexpr int kPipeAllWarps = kPipeConsumerWarps * kPipeGroups;
constexpr int kPipeConsumers = kPipeAllWarps * 32;
constexpr int kPipeThreads = kPipeConsumers + 32;  // + the producer warp
constexpr int kPipeMaxStages = 8;
constexpr int kActRec = 336;       // one Q8_K activation superblock in shared memory (21 x 16 B: conflict-free lane stride)
constexpr int kRecBsum16 = 256;    // 16 x i16 sums of 16 codes
constexpr int kRecBsum32 = 288;    // 8 x i16 sums of 32 codes
constexpr int kRecD = 304;         // f32 scale
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and flags the error) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int32_t *status) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  if (status) atomicExch(status, (int32_t)CMLD_ERR_TIMEOUT);
  return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {  // unsigned bytes x signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

struct PipeJob {
  const uint8_t *w;
  int32_t qt, rows, tile_rows, first_tile, n_tiles;
  int64_t stride;
  float *y;
  const float *residual;
  int64_t y_stride;
};

struct PipeArgs {
  PipeJob job[3];
  int32_t n_jobs, total_tiles, cols, batch, stage_bytes, n_stages;
  int32_t mode;  // 0: quantised activation given (act_in); 1: RMSNorm(x)*norm_w; 2: x as is; 3: SwiGLU(x, x2)
  const float *x, *x2, *norm_w;
  int64_t x_stride;
  float eps;
  const uint8_t *act_in;  // standard global layout, Q8_K rows (then Q8_0 rows at act_in0)
  const uint8_t *act_in0;
  int32_t need_k, need_0;
  int32_t paired;  // two matrices of equal shape and type: tiles alternate between them and the result is SwiGLU(first, second)
  int32_t off_act_k, off_act_0, off_red, off_pair, off_ring;
  float *norm_out;        // optional f32 copy of the normalised row (written by CTA 0)
  int32_t *status;
  GemvPeer peer;          // tensor-parallel sum folded into this launch (tx_n / rx_n = 0: none)
  int64_t peer_rank_stride;  // floats between the ranks' partials in the receive slot
};

// Quantises one 256-value chunk (8 values per lane) of batch row b into the shared-memory operands.
__device__ __forceinline__ void emit_chunk(const float (&v)[8], const PipeArgs &a, int b, int ch, int lane, uint8_t *act_k,
                                           uint8_t *act_0, int rec_col_stride, int act0_col_stride) {
  const int e0 = ch * 256 + lane * 8;
  if (a.need_k) {
    int q[8];
    float d;
    q8k_quantise_chunk(v, lane, q, d);
    uint8_t *rec = act_k + b * rec_col_stride + ch * kActRec;
    *reinterpret_cast<uint2 *>(rec + lane * 8) = pack8(q);
    int s16 = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
    s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) reinterpret_cast<short *>(rec + kRecBsum16)[lane >> 1] = (short)s16;
    if ((lane & 3) == 0) reinterpret_cast<short *>(rec + kRecBsum32)[lane >> 2] = (short)s32;
    if (lane == 0) *reinterpret_cast<float *>(rec + kRecD) = d;
  }
  if (a.need_0) {
    int q[8];
    float sc;
    q80_quantise_chunk(v, q, sc);
    if (e0 < a.cols) {
      *reinterpret_cast<uint2 *>(act_0 + b * act0_col_stride + e0) = pack8(q);
      if ((lane & 3) == 0) reinterpret_cast<float *>(act_0 + b * act0_col_stride + round_up16(a.cols))[e0 >> 5] = sc;
    }
  }
}

constexpr int kRxChunks = 2;  // chunks a warp holds in registers in the receiving prologue: hidden <= 16 * 2 * 256

// ---------------------------------------------------------------- per-superblock dots (shared memory operands)

template <int B>
__device__ __forceinline__ void sb_dot_q4k(const uint8_t *blk, const uint8_t *rec, int rec_col_stride, float (&acc)[B]) {
  const uint4 meta = *reinterpret_cast<const uint4 *>(blk);
  const float d = f16_bits_to_f32((uint16_t)(meta.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(meta.x >> 16));
  // 6-bit scales/mins as bytes (q4_k_scale_min, src/tensor/mod.rs:5997-6006): groups 0..3 and 4..7
  const uint32_t sc03 = meta.y & 0x3f3f3f3fu, m03 = meta.z & 0x3f3f3f3fu;
  const uint32_t sc47 = (meta.w & 0x0f0f0f0fu) | ((meta.y >> 2) & 0x30303030u);
  const uint32_t m47 = ((meta.w >> 4) & 0x0f0f0f0fu) | ((meta.z >> 2) & 0x30303030u);
  int s[B];
#pragma unroll
  for (int b = 0; b < B; ++b) s[b] = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int dl[B], dh[B];
#pragma unroll
    for (int b = 0; b < B; ++b) dl[b] = dh[b] = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 w = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * j + 16 * h);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint8_t *r = rec + b * rec_col_stride;
        const int4 xlo = *reinterpret_cast<const int4 *>(r + 64 * j + 16 * h);
        const int4 xhi = *reinterpret_cast<const int4 *>(r + 64 * j + 32 + 16 * h);
        dl[b] = __dp4a((int)(w.x & 0x0f0f0f0fu), xlo.x, dl[b]);
        dl[b] = __dp4a((int)(w.y & 0x0f0f0f0fu), xlo.y, dl[b]);
        dl[b] = __dp4a((int)(w.z & 0x0f0f0f0fu), xlo.z, dl[b]);
        dl[b] = __dp4a((int)(w.w & 0x0f0f0f0fu), xlo.w, dl[b]);
        // high nibbles left in place: bytes are 16*nibble (unsigned), the sum is shifted back below
        dh[b] = dp4a_us(w.x & 0xf0f0f0f0u, xhi.x, dh[b]);
        dh[b] = dp4a_us(w.y & 0xf0f0f0f0u, xhi.y, dh[b]);
        dh[b] = dp4a_us(w.z & 0xf0f0f0f0u, xhi.z, dh[b]);
        dh[b] = dp4a_us(w.w & 0xf0f0f0f0u, xhi.w, dh[b]);
      }
    }
    const uint32_t scw = j < 2 ? sc03 : sc47;
    const int sl = (scw >> (16 * (j & 1))) & 0xff, sh = (scw >> (16 * (j & 1) + 8)) & 0xff;
#pragma unroll
    for (int b = 0; b < B; ++b) s[b] += dl[b] * sl + (dh[b] >> 4) * sh;
  }
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const uint8_t *r = rec + b * rec_col_stride;
    const int4 bs = *reinterpret_cast<const int4 *>(r + kRecBsum32);  // 8 x i16 sums of 32 codes
    int p = __dp2a_lo(bs.x, (int)m03, 0);
    p = __dp2a_hi(bs.y, (int)m03, p);
    p = __dp2a_lo(bs.z, (int)m47, p);
    p = __dp2a_hi(bs.w, (int)m47, p);
    const float xd = *reinterpret_cast<const float *>(r + kRecD);
    // sumf = fma(-dmin, prod, sumf); sumf = fma(d, S, sumf)   (refmath.rs:529 and :560)
    acc[b] = __fmaf_rn(__fmul_rn(xd, d), (float)s[b], __fmaf_rn(-__fmul_rn(xd, dmin), (float)p, acc[b]));
  }
}

template <int B>
__device__ __forceinline__ void sb_dot_q6k(const uint8_t *blk, float dw, const uint8_t *rec, int rec_col_stride, float (&acc)[B]) {
  const int4 scw = *reinterpret_cast<const int4 *>(blk + 192);  // 16 signed scales
  int s[B];
#pragma unroll
  for (int b = 0; b < B; ++b) s[b] = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint4 qh = *reinterpret_cast<const uint4 *>(blk + 128 + 32 * h + 16 * c);
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        const uint4 ql = *reinterpret_cast<const uint4 *>(blk + 64 * h + 32 * sp + 16 * c);
        const int jlo = 8 * h + 2 * sp + c;  // 16-value group of the low-nibble stream; the high stream is jlo + 4
        // 6-bit codes: low nibble | two qh bits moved to bits 4..5
        uint4 lo, hi;
        if (sp == 0) {
          lo = make_uint4((ql.x & 0x0f0f0f0fu) | ((qh.x << 4) & 0x30303030u), (ql.y & 0x0f0f0f0fu) | ((qh.y << 4) & 0x30303030u),
                          (ql.z & 0x0f0f0f0fu) | ((qh.z << 4) & 0x30303030u), (ql.w & 0x0f0f0f0fu) | ((qh.w << 4) & 0x30303030u));
          hi = make_uint4(((ql.x >> 4) & 0x0f0f0f0fu) | (qh.x & 0x30303030u), ((ql.y >> 4) & 0x0f0f0f0fu) | (qh.y & 0x30303030u),
                          ((ql.z >> 4) & 0x0f0f0f0fu) | (qh.z & 0x30303030u), ((ql.w >> 4) & 0x0f0f0f0fu) | (qh.w & 0x30303030u));
        } else {
          lo = make_uint4((ql.x & 0x0f0f0f0fu) | ((qh.x << 2) & 0x30303030u), (ql.y & 0x0f0f0f0fu) | ((qh.y << 2) & 0x30303030u),
                          (ql.z & 0x0f0f0f0fu) | ((qh.z << 2) & 0x30303030u), (ql.w & 0x0f0f0f0fu) | ((qh.w << 2) & 0x30303030u));
          hi = make_uint4(((ql.x >> 4) & 0x0f0f0f0fu) | ((qh.x >> 2) & 0x30303030u), ((ql.y >> 4) & 0x0f0f0f0fu) | ((qh.y >> 2) & 0x30303030u),
                          ((ql.z >> 4) & 0x0f0f0f0fu) | ((qh.z >> 2) & 0x30303030u), ((ql.w >> 4) & 0x0f0f0f0fu) | ((qh.w >> 2) & 0x30303030u));
        }
        const int wsel = jlo >> 2, bsel = jlo & 3;  // scale jlo is byte bsel of word wsel; jlo+4 is the same byte of the next word
        const int w_lo = wsel == 0 ? scw.x : (wsel == 1 ? scw.y : (wsel == 2 ? scw.z : scw.w));
        const int w_hi = wsel == 0 ? scw.y : (wsel == 1 ? scw.z : (wsel == 2 ? scw.w : 0));
        const int slo = (int)(int8_t)(w_lo >> (8 * bsel)), shi = (int)(int8_t)(w_hi >> (8 * bsel));
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const uint8_t *r = rec + b * rec_col_stride;
          const int4 xlo = *reinterpret_cast<const int4 *>(r + 16 * jlo);
          const int4 xhi = *reinterpret_cast<const int4 *>(r + 16 * (jlo + 4));
          int dl = __dp4a((int)lo.x, xlo.x, 0);
          dl = __dp4a((int)lo.y, xlo.y, dl);
          dl = __dp4a((int)lo.z, xlo.z, dl);
          dl = __dp4a((int)lo.w, xlo.w, dl);
          int dh = __dp4a((int)hi.x, xhi.x, 0);
          dh = __dp4a((int)hi.y, xhi.y, dh);
          dh = __dp4a((int)hi.z, xhi.z, dh);
          dh = __dp4a((int)hi.w, xhi.w, dh);
          s[b] += slo * dl + shi * dh;
        }
      }
    }
  }
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const uint8_t *r = rec + b * rec_col_stride;
    // codes are stored +32: sum_j sc_j * sum (q-32) x = sum_j sc_j*dot_j - 32 * sum_j sc_j * bsum16_j
    const int4 b0 = *reinterpret_cast<const int4 *>(r + kRecBsum16), b1 = *reinterpret_cast<const int4 *>(r + kRecBsum16 + 16);
    int corr = __dp2a_lo(b0.x, scw.x, 0);
    corr = __dp2a_hi(b0.y, scw.x, corr);
    corr = __dp2a_lo(b0.z, scw.y, corr);
    corr = __dp2a_hi(b0.w, scw.y, corr);
    corr = __dp2a_lo(b1.x, scw.z, corr);
    corr = __dp2a_hi(b1.y, scw.z, corr);
    corr = __dp2a_lo(b1.z, scw.w, corr);
    corr = __dp2a_hi(b1.w, scw.w, corr);
    const float xd = *reinterpret_cast<const float *>(r + kRecD);
    acc[b] = __fadd_rn(acc[b], __fmul_rn(__fmul_rn(dw, xd), (float)(s[b] - 32 * corr)));
  }
}

// Sum of v over each group of `len` consecutive lanes (groups start at multiples of len); the
// result is valid in the first lane of each group.  Fixed order, so deterministic.
__device__ __forceinline__ float segment_sum(float v, int lane_in_seg, int len) {
  int cur = len;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    if (off < cur) {
      const float t = __shfl_down_sync(0xffffffffu, v, off);
      if (lane_in_seg + off < cur) v += t;
      cur = off;
    }
  }
  return v;
}

// Dot products of one staged tile: on return v[b] holds row r_local's result for batch column b in the
// lanes with `writer` set (the first lane of each row's lane segment).
template <int B>
__device__ __forceinline__ void tile_dot(const PipeArgs &a, const PipeJob &J, const uint8_t *tile, int nrows, int wg, int lane,
                                         const uint8_t *act_k, const uint8_t *act_0, int nsb, int rec_col_stride,
                                         int act0_col_stride, float (&v)[B], bool &writer, int &r_local) {
  const int n_it = J.qt == CMLD_Q8_0 ? (a.cols >> 5) : nsb;  // work items per row: blocks or superblocks
  const int L = n_it < 32 ? n_it : 32;                        // lanes per row
  const int rpw = 32 / L;                                     // rows per warp
  r_local = wg * rpw + lane / L;
  const int lis = lane % L;
  const bool active = lane < rpw * L && r_local < nrows;
  float acc[B];
#pragma unroll
  for (int b = 0; b < B; ++b) acc[b] = 0.0f;
  if (active) {
    const uint8_t *row = tile + (int64_t)r_local * J.stride;
    if (J.qt == CMLD_Q4_K) {
      for (int sb = lis; sb < nsb; sb += L) sb_dot_q4k<B>(row + sb * 144, act_k + sb * kActRec, rec_col_stride, acc);
    } else if (J.qt == CMLD_Q6_K) {
      for (int sb = lis; sb < nsb; sb += L) {
        const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(row + nsb * 208 + 2 * sb));
        sb_dot_q6k<B>(row + sb * 208, dw, act_k + sb * kActRec, rec_col_stride, acc);
      }
    } else {
      // Q8_0: a lane owns 32-value blocks; the two 16-byte halves are read in an order that
      // keeps the eight lanes of a shared-memory phase on distinct banks
      const int hs = (lane >> 2) & 1;
      for (int blk = lis; blk < n_it; blk += L) {
        const uint4 w0 = *reinterpret_cast<const uint4 *>(row + blk * 32 + 16 * hs);
        const uint4 w1 = *reinterpret_cast<const uint4 *>(row + blk * 32 + 16 * (hs ^ 1));
        const float ws = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(row + a.cols + 2 * blk));
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const uint8_t *xa = act_0 + b * act0_col_stride;
          const int4 x0 = *reinterpret_cast<const int4 *>(xa + blk * 32 + 16 * hs);
          const int4 x1 = *reinterpret_cast<const int4 *>(xa + blk * 32 + 16 * (hs ^ 1));
          int isum = __dp4a((int)w0.x, x0.x, 0);
          isum = __dp4a((int)w0.y, x0.y, isum);
          isum = __dp4a((int)w0.z, x0.z, isum);
          isum = __dp4a((int)w0.w, x0.w, isum);
          isum = __dp4a((int)w1.x, x1.x, isum);
          isum = __dp4a((int)w1.y, x1.y, isum);
          isum = __dp4a((int)w1.z, x1.z, isum);
          isum = __dp4a((int)w1.w, x1.w, isum);
          const float xs = reinterpret_cast<const float *>(xa + round_up16(a.cols))[blk];
          acc[b] = __fadd_rn(acc[b], __fmul_rn(__fmul_rn((float)isum, ws), xs));  // src/inference.rs:26198
        }
      }
    }
  }
#pragma unroll
  for (int b = 0; b < B; ++b) v[b] = segment_sum(acc[b], lis, L);
  writer = active && lis == 0;
}

// ---------------------------------------------------------------- the kernel

template <int B>
__global__ void __launch_bounds__(kPipeThreads, 1) gemv_pipe_kernel(const PipeArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + kPipeMaxStages;
  uint8_t *act_k = smem + a.off_act_k;
  uint8_t *act_0 = smem + a.off_act_0;
  float *red = reinterpret_cast<float *>(smem + a.off_red);
  uint8_t *ring = smem + a.off_ring;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.n_stages;
  // tiles this CTA takes: t = blockIdx.x + i*gridDim.x; in paired mode the unit is a (gate, up) pair of tiles
  const int n_units = a.paired ? a.job[0].n_tiles : a.total_tiles;
  const int n_my = ((int)blockIdx.x < n_units ? (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0) * (a.paired ? 2 : 1);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kPipeConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Let the next kernel of the stream get scheduled as early as the hardware allows; it blocks in
  // its own griddepcontrol.wait until this grid has completed.
  asm volatile("griddepcontrol.launch_dependents;");
  unsigned long long *tr = nullptr;  // timeline record of this launch (CTA 0, thread 0 of the consumers)
  if (a.peer.trace && blockIdx.x == 0 && tid == 0) {
    const unsigned long long idx = atomicAdd(a.peer.trace, 1ull);
    if (idx < (unsigned long long)kTraceRecords) {
      tr = a.peer.trace + 1 + idx * 8;
      tr[0] = global_ns();
      tr[6] = (unsigned long long)a.n_jobs | ((unsigned long long)a.peer.tx_n << 8) | ((unsigned long long)a.peer.rx_n << 16) |
              ((unsigned long long)a.cols << 32);
    }
  }

  if (warp == kPipeAllWarps) {
    // ---------------- producer: weights do not depend on the previous kernel, so no wait here
    if (lane == 0) {
      for (int i = 0; i < n_my; ++i) {
        const int s = i % S;
        if (i >= S) mbar_wait(&empty[s], (uint32_t)((i / S - 1) & 1), a.status);
        int j = 0, row0;
        if (a.paired) {
          j = i & 1;
          row0 = ((int)blockIdx.x + (i >> 1) * (int)gridDim.x) * a.job[0].tile_rows;
        } else {
          const int t = (int)blockIdx.x + i * (int)gridDim.x;
          if (a.n_jobs > 1 && t >= a.job[1].first_tile) j = 1;
          if (a.n_jobs > 2 && t >= a.job[2].first_tile) j = 2;
          row0 = (t - a.job[j].first_tile) * a.job[j].tile_rows;
        }
        const PipeJob &J = a.job[j];
        const int nrows = min(J.tile_rows, J.rows - row0);
        const uint32_t bytes = (uint32_t)(nrows * J.stride);
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(ring + (int64_t)s * a.stage_bytes, J.w + (int64_t)row0 * J.stride, bytes, &full[s]);
      }
    }
    return;
  }

  // ---------------- consumers
  asm volatile("griddepcontrol.wait;" ::: "memory");  // inputs written by the previous kernel are now visible
  if (tr) tr[1] = global_ns();
  const int nsb = a.cols >> 8;
  const int rec_col_stride = nsb * kActRec;
  const int act0_col_stride = (int)round_up16(a.cols) + (int)round_up16((a.cols >> 5) * 4);

  if (a.peer.rx_n > 0) {
    // the input rows are still spread over the ranks: wait for every rank's partial to have arrived
    if (tid < a.peer.rx_n) peer_wait(a.peer.rx_flag + tid, __ldcg(a.peer.rx_epoch), a.peer.timeout_ns, a.status);
    asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
  }
  if (tr) tr[2] = global_ns();

  // Prologue: quantised activation rows into shared memory.
  if (a.mode == 0) {
    // re-lay the pre-quantised global rows; flat loops over (row, piece) so that every thread has several
    // independent loads in flight instead of one L2 round trip per row
    const int64_t astride = act_row_stride(a.cols);
    if (a.need_k) {
      for (int idx = tid; idx < a.batch * nsb * 16; idx += kPipeConsumers) {  // 16-byte chunks of codes
        const int b = idx / (nsb * 16), i = idx % (nsb * 16), sb = i >> 4, c = i & 15;
        *reinterpret_cast<uint4 *>(act_k + b * rec_col_stride + sb * kActRec + c * 16) =
            __ldg(reinterpret_cast<const uint4 *>(a.act_in + b * astride + sb * 256 + c * 16));
      }
      for (int idx = tid; idx < a.batch * nsb * 8; idx += kPipeConsumers) {  // pairs of 16-sums
        const int b = idx / (nsb * 8), i = idx % (nsb * 8), sb = i >> 3, g = i & 7;
        const int pr = __ldg(reinterpret_cast<const int *>(a.act_in + b * astride + act_bsum_off(a.cols)) + i);
        uint8_t *rec = act_k + b * rec_col_stride + sb * kActRec;
        reinterpret_cast<int *>(rec + kRecBsum16)[g] = pr;
        reinterpret_cast<short *>(rec + kRecBsum32)[g] = (short)((int)(short)(pr & 0xffff) + (pr >> 16));
      }
      for (int idx = tid; idx < a.batch * nsb; idx += kPipeConsumers) {
        const int b = idx / nsb, sb = idx % nsb;
        *reinterpret_cast<float *>(act_k + b * rec_col_stride + sb * kActRec + kRecD) =
            __ldg(reinterpret_cast<const float *>(a.act_in + b * astride + act_scale_off(a.cols)) + sb);
      }
    }
    if (a.need_0) {
      const int n16 = a.cols >> 4, n32 = a.cols >> 5;
      for (int idx = tid; idx < a.batch * n16; idx += kPipeConsumers) {
        const int b = idx / n16, i = idx % n16;
        *reinterpret_cast<uint4 *>(act_0 + b * act0_col_stride + i * 16) = __ldg(reinterpret_cast<const uint4 *>(a.act_in0 + b * astride) + i);
      }
      for (int idx = tid; idx < a.batch * n32; idx += kPipeConsumers) {
        const int b = idx / n32, i = idx % n32;
        reinterpret_cast<float *>(act_0 + b * act0_col_stride + round_up16(a.cols))[i] =
            __ldg(reinterpret_cast<const float *>(a.act_in0 + b * astride + act_scale_off(a.cols)) + i);
      }
    }
  }
  const bool chunked_norm = a.mode == 1 && (a.cols & 255) == 0 && a.cols <= kRxChunks * kPipeAllWarps * 256;
  for (int b = 0; b < a.batch; ++b) {
    if (a.peer.rx_n > 0 || chunked_norm) {
      // RMSNorm with ONE load of the row: each warp keeps its chunks in registers between the mean-square
      // pass and the scaling pass.  The squares are added per lane over the warp's chunks, by the shuffle
      // tree within the warp, then the sixteen warp sums by one more shuffle tree — the order the
      // stand-alone norm kernel reproduces, so both give the same bits.  With a peer sum the row is the sum
      // of the ranks' partial rows (added in rank order, so every rank gets the same bits).
      float hv[kRxChunks][8];
      float ss = 0.0f;
#pragma unroll
      for (int k = 0; k < kRxChunks; ++k) {
        const int ch = warp + k * kPipeAllWarps;
        if (ch * 256 < a.cols) {
          const float *src = (a.peer.rx_n > 0 ? a.peer.rx_part + (int64_t)b * a.cols : a.x + (int64_t)b * a.x_stride) + ch * 256 + lane * 8;
          float4 s0 = __ldcg(reinterpret_cast<const float4 *>(src)), s1 = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
          for (int r = 1; r < a.peer.rx_n; ++r) {
            const float4 t0 = __ldcg(reinterpret_cast<const float4 *>(src + r * a.peer_rank_stride));
            const float4 t1 = __ldcg(reinterpret_cast<const float4 *>(src + r * a.peer_rank_stride) + 1);
            s0.x = __fadd_rn(s0.x, t0.x), s0.y = __fadd_rn(s0.y, t0.y), s0.z = __fadd_rn(s0.z, t0.z), s0.w = __fadd_rn(s0.w, t0.w);
            s1.x = __fadd_rn(s1.x, t1.x), s1.y = __fadd_rn(s1.y, t1.y), s1.z = __fadd_rn(s1.z, t1.z), s1.w = __fadd_rn(s1.w, t1.w);
          }
          const float t[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            hv[k][i] = t[i];
            ss = __fmaf_rn(t[i], t[i], ss);
          }
          if (blockIdx.x == 0 && a.peer.rx_out) {
            float4 *o4 = reinterpret_cast<float4 *>(a.peer.rx_out + (int64_t)b * a.cols + ch * 256 + lane * 8);
            o4[0] = s0;
            o4[1] = s1;
          }
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
      float t = lane < kPipeAllWarps ? red[lane] : 0.0f;
      t = warp_sum(t);
      const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)a.cols), a.eps)));
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
#pragma unroll
      for (int k = 0; k < kRxChunks; ++k) {
        const int ch = warp + k * kPipeAllWarps;
        if (ch * 256 < a.cols) {
          const int e0 = ch * 256 + lane * 8;
          const float4 wa = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0)), wb = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0) + 1);
          const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(hv[k][i], scale), wv[i]);
          if (a.norm_out && blockIdx.x == 0) {
            float4 *o4 = reinterpret_cast<float4 *>(a.norm_out + (int64_t)b * a.cols + e0);
            o4[0] = make_float4(v[0], v[1], v[2], v[3]);
            o4[1] = make_float4(v[4], v[5], v[6], v[7]);
          }
          emit_chunk(v, a, b, ch, lane, act_k, act_0, rec_col_stride, act0_col_stride);
        }
      }
      continue;
    }
    if (a.mode == 0) continue;  // copied above
    const float *x = a.x + (int64_t)b * a.x_stride;
    const float *x2 = a.mode == 3 ? a.x2 + (int64_t)b * a.x_stride : nullptr;
    float scale = 1.0f;
    if (a.mode == 1) {
      // the mean square is summed by the first 256 threads in the same order as the stand-alone
      // norm kernel, so both paths produce the same bits
      float ss = 0.0f;
      if (tid < 256)
#pragma unroll 8
        for (int i = tid; i < a.cols; i += 256) {
          const float v = __ldcg(x + i);
          ss = __fmaf_rn(v, v, ss);
        }
      ss = warp_sum(ss);
      if (lane == 0 && warp < 8) red[warp] = ss;
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
      float t = lane < 8 ? red[lane] : 0.0f;
      t = warp_sum(t);
      scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)a.cols), a.eps)));
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
    }
    const int n_chunks = (a.cols + 255) >> 8;
    for (int ch = warp; ch < n_chunks; ch += kPipeAllWarps) {
      const int e0 = ch * 256 + lane * 8;
      float v[8];
      if (e0 + 8 <= a.cols) {
        // 8 consecutive values per lane: two 128-bit loads per operand (cols is a multiple of 32)
        const float4 xa = __ldcg(reinterpret_cast<const float4 *>(x + e0)), xb = __ldcg(reinterpret_cast<const float4 *>(x + e0) + 1);
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        if (a.mode == 1) {
          const float4 wa = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0)), wb = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0) + 1);
          const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(xv[i], scale), wv[i]);
        } else if (a.mode == 3) {
          const float4 ua = __ldcg(reinterpret_cast<const float4 *>(x2 + e0)), ub = __ldcg(reinterpret_cast<const float4 *>(x2 + e0) + 1);
          const float uv[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = swiglu(xv[i], uv[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = xv[i];
        }
        if (a.norm_out && blockIdx.x == 0) {
          float4 *o4 = reinterpret_cast<float4 *>(a.norm_out + (int64_t)b * a.cols + e0);
          o4[0] = make_float4(v[0], v[1], v[2], v[3]);
          o4[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
      }
      emit_chunk(v, a, b, ch, lane, act_k, act_0, rec_col_stride, act0_col_stride);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
  if (tr) tr[3] = global_ns();

  // Main loop over this CTA's tiles; the two consumer groups alternate.
  const int group = warp / kPipeConsumerWarps, wg = warp % kPipeConsumerWarps;
  if (a.paired) {
    // gate and up tiles of the same rows are consecutive tiles 2k, 2k+1 of this CTA: group 0 takes the gate tile,
    // group 1 the up tile, at the same time; group 1 hands its results over through shared memory (two
    // buffers, one barrier of all consumers per pair) and group 0 writes SwiGLU(gate, up) — the f32 operand
    // of the down projection — so neither product goes through memory on its own.
    float *pairbuf = reinterpret_cast<float *>(smem + a.off_pair);  // [2][tile_rows][B]
    const int tile_rows = a.job[0].tile_rows;
    for (int k = 0; 2 * k < n_my; ++k) {
      const int pair = (int)blockIdx.x + k * (int)gridDim.x;
      const int row0 = pair * tile_rows;
      const int nrows = min(tile_rows, a.job[0].rows - row0);
      const int i = 2 * k + group, s = i % S;
      const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[s], (uint32_t)((i / S) & 1), a.status));
      float v[B];
      bool writer = false;
      int r_local = 0;
      if (ready) {
        tile_dot<B>(a, a.job[group], ring + (int64_t)s * a.stage_bytes, nrows, wg, lane, act_k, act_0, nsb, rec_col_stride,
                    act0_col_stride, v, writer, r_local);
      } else {
#pragma unroll
        for (int b = 0; b < B; ++b) v[b] = 0.0f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      float *slot = pairbuf + ((k & 1) * tile_rows + r_local) * B;
      if (group == 1 && writer) {
#pragma unroll
        for (int b = 0; b < B; ++b) slot[b] = v[b];
      }
      asm volatile("bar.sync 2, %0;" ::"n"(kPipeConsumers));
      if (group == 0 && writer) {
#pragma unroll
        for (int b = 0; b < B; ++b) a.job[0].y[(int64_t)b * a.job[0].y_stride + row0 + r_local] = swiglu(v[b], slot[b]);
      }
    }
  } else {
    for (int i = group; i < n_my; i += kPipeGroups) {
      const int s = i % S;
      const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[s], (uint32_t)((i / S) & 1), a.status));
      const int t = (int)blockIdx.x + i * (int)gridDim.x;
      int j = 0;
      if (a.n_jobs > 1 && t >= a.job[1].first_tile) j = 1;
      if (a.n_jobs > 2 && t >= a.job[2].first_tile) j = 2;
      const PipeJob &J = a.job[j];
      const int row0 = (t - J.first_tile) * J.tile_rows;
      const int nrows = min(J.tile_rows, J.rows - row0);
      if (ready) {
        float v[B];
        bool writer;
        int r_local;
        tile_dot<B>(a, J, ring + (int64_t)s * a.stage_bytes, nrows, wg, lane, act_k, act_0, nsb, rec_col_stride, act0_col_stride, v, writer, r_local);
        if (writer) {
#pragma unroll
          for (int b = 0; b < B; ++b) {
            const int64_t o = (int64_t)b * J.y_stride + row0 + r_local;
            const float out = J.residual ? __fadd_rn(__ldcg(J.residual + o), v[b]) : v[b];
            if (a.peer.tx_n > 0) {
              for (int p = 0; p < a.peer.tx_n; ++p) a.peer.tx_part[p][o] = out;  // this rank's partial, onto every rank
            } else {
              J.y[o] = out;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  if (tr) tr[4] = global_ns();
  if (a.peer.tx_n > 0) {
    // The CTA barrier orders every consumer's stores before thread 0's system-scope fence (fences are
    // cumulative), and the fence before this CTA's ticket; the CTA that takes the last ticket has
    // therefore seen the whole launch's rows leave, and raises this rank's arrival word everywhere.
    // (One fence per CTA: a system-scope fence in every thread costs tens of microseconds.)
    asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
    if (tid == 0) {
      __threadfence_system();
      if (atomicAdd(a.peer.tx_ticket, 1u) == gridDim.x - 1) {
        __threadfence_system();
        *a.peer.tx_ticket = 0;
        const uint32_t epoch = *a.peer.tx_epoch + 1;
        *a.peer.tx_epoch = epoch;
        // one fence (above) orders every row before every arrival word; the words themselves go out as plain
        // stores (a release store per rank would wait for the previous rank's round trip each time: ~3 us x ranks)
        for (int p = 0; p < a.peer.tx_n; ++p) st_relaxed_sys(a.peer.tx_flag[p], epoch);
      }
      if (tr) tr[5] = global_ns();
    }
  }
}

// ---------------------------------------------------------------- host side

struct PipePlan {
  PipeArgs args;
  int smem_bytes;
};

static int g_sm_count = 0;
static bool g_attr_set[9] = {false};

template <int B>
static int32_t launch_pipe_b(const PipePlan &p, int grid, cudaStream_t s, bool pdl) {
  if (!g_attr_set[B]) {
    CMLD_CUDA(cudaFuncSetAttribute(gemv_pipe_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    g_attr_set[B] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kPipeThreads);
  cfg.dynamicSmemBytes = (size_t)p.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, gemv_pipe_kernel<B>, p.args));
  return CMLD_OK;
}

// Tile geometry and shared-memory map for these matrices at this batch; false if it does not fit.
static bool plan_pipe(const GemvJob *jobs, int n_jobs, int32_t batch, PipePlan &p, bool &need_k, bool &need_0, int &tiles_out,
                      bool paired = false) {
  if (n_jobs < 1 || n_jobs > 3 || batch < 1 || batch > 8) return false;
  const int64_t cols = jobs[0].cols;
  if (cols % 32) return false;
  PipeArgs &a = p.args;
  need_k = need_0 = false;
  int stage = 0, tiles = 0;
  for (int k = 0; k < n_jobs; ++k) {
    const GemvJob &g = jobs[k];
    if (g.cols != cols) return false;
    if (g.qt == CMLD_Q8_0) need_0 = true;
    else {
      need_k = true;
      if (cols % 256) return false;
    }
    const int n_it = g.qt == CMLD_Q8_0 ? (int)(cols >> 5) : (int)(cols >> 8);
    const int L = n_it < 32 ? n_it : 32;
    PipeJob &J = a.job[k];
    J.w = g.w;
    J.qt = g.qt;
    J.rows = (int32_t)g.rows;
    J.tile_rows = kPipeConsumerWarps * (32 / L);
    J.stride = g.stride;
    J.y = g.y;
    J.residual = g.residual;
    J.y_stride = g.y_stride;
    J.first_tile = tiles;
    J.n_tiles = (int)((g.rows + J.tile_rows - 1) / J.tile_rows);
    tiles += J.n_tiles;
    stage = std::max<int>(stage, (int)(J.tile_rows * g.stride));
    if (g.stride % 16 || (reinterpret_cast<uintptr_t>(g.w) & 15)) return false;
  }
  stage = (stage + 127) & ~127;
  const int nsb = (int)(cols >> 8);
  int off = 2 * kPipeMaxStages * 8;
  a.off_act_k = off;
  if (need_k) off += batch * nsb * kActRec;
  off = (off + 15) & ~15;
  a.off_act_0 = off;
  if (need_0) off += batch * ((int)round_up16(cols) + (int)round_up16((cols >> 5) * 4));
  a.off_red = off;
  off += 64 * 4;
  a.off_pair = off;
  if (paired) off += 2 * a.job[0].tile_rows * batch * 4;
  off = (off + 127) & ~127;
  a.off_ring = off;
  // Prefer a footprint that lets two kernels share an SM (the next one prefetches under PDL).
  // The stage count must be a multiple of the number of consumer groups: tile i lives in stage i % S and
  // belongs to group i % kPipeGroups, so with S even every stage is only ever used by one group and a
  // group meets the phases of its stages in order (an mbarrier parity wait cannot tell phase n from n+2).
  int n_stages = 0;
  for (int budget : {110 * 1024, 224 * 1024}) {
    n_stages = std::min<int>(kPipeMaxStages, (budget - off) / stage);
    n_stages -= n_stages % kPipeGroups;
    if (n_stages >= 4) break;
  }
  if (n_stages < 2) return false;
  if (paired && (n_jobs != 2 || jobs[0].rows != jobs[1].rows || jobs[0].qt != jobs[1].qt || jobs[0].stride != jobs[1].stride)) return false;
  p.smem_bytes = off + n_stages * stage;
  a.stage_bytes = stage;
  a.n_stages = n_stages;
  tiles_out = tiles;
  return true;
}

int gemv_pipe_fit_batch(const GemvJob *jobs, int n_jobs, bool paired) {
  for (int b = 8; b >= 1; --b) {
    PipePlan p{};
    bool nk, n0;
    int tiles;
    if (plan_pipe(jobs, n_jobs, b, p, nk, n0, tiles, paired)) return b;
  }
  return 0;
}

// Plans and launches the staged kernel.  Returns CMLD_ERR_UNSUPPORTED (without setting an error
// message the caller would see) when the shape does not fit; the caller then uses the
// direct-load kernel.
int32_t launch_gemv_pipe(const GemvJob *jobs, int n_jobs, int32_t batch, const GemvPrologue &pro, int32_t *status,
                         cudaStream_t s, bool pdl, const GemvPeer *peer) {
  if (g_sm_count == 0) {
    int dev = 0;
    CMLD_CUDA(cudaGetDevice(&dev));
    CMLD_CUDA(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  PipePlan p{};
  PipeArgs &a = p.args;
  bool need_k = false, need_0 = false;
  int tiles = 0;
  if (!plan_pipe(jobs, n_jobs, batch, p, need_k, need_0, tiles, pro.pair_swiglu != 0)) return CMLD_ERR_UNSUPPORTED;
  const int64_t cols = jobs[0].cols;
  a.n_jobs = n_jobs;
  a.total_tiles = tiles;
  a.cols = (int32_t)cols;
  a.batch = batch;
  a.mode = pro.mode;
  a.x = pro.x;
  a.x2 = pro.x2;
  a.norm_w = pro.norm_w;
  a.x_stride = pro.x_stride;
  a.eps = pro.eps;
  a.act_in = pro.act_k;
  a.act_in0 = pro.act_0;
  a.need_k = need_k;
  a.need_0 = need_0;
  a.norm_out = pro.norm_out;
  a.status = status;
  a.paired = pro.pair_swiglu ? 1 : 0;
  if (a.paired && peer && peer->tx_n > 0) return fail(CMLD_ERR_INVALID, "gemv: a paired launch does not send");
  if (peer) {
    a.peer = *peer;
    a.peer_rank_stride = (int64_t)kPeerRows * cols;
    if (peer->tx_n > 0 && (n_jobs != 1 || !status)) return fail(CMLD_ERR_INVALID, "gemv: a sending launch takes one matrix and a status word");
    if (peer->rx_n > 0 && (pro.mode != 1 || cols % 256 || cols > kRxChunks * kPipeAllWarps * 256 || !status))
      return fail(CMLD_ERR_INVALID, "gemv: a receiving launch is an RMSNorm prologue over at most %d columns", kRxChunks * kPipeAllWarps * 256);
  }
  if (a.mode == 0 && ((need_k && !a.act_in) || (need_0 && !a.act_in0))) return fail(CMLD_ERR_INVALID, "gemv: activation buffer missing");
  const int grid = std::min(a.paired ? a.job[0].n_tiles : tiles, g_sm_count);
  switch (batch) {
    case 1: return launch_pipe_b<1>(p, grid, s, pdl);
    case 2: return launch_pipe_b<2>(p, grid, s, pdl);
    case 3: return launch_pipe_b<3>(p, grid, s, pdl);
    case 4: return launch_pipe_b<4>(p, grid, s, pdl);
    case 5: return launch_pipe_b<5>(p, grid, s, pdl);
    case 6: return launch_pipe_b<6>(p, grid, s, pdl);
    case 7: return launch_pipe_b<7>(p, grid, s, pdl);
    default: return launch_pipe_b<8>(p, grid, s, pdl);
  }
}

}  // namespace cmld
