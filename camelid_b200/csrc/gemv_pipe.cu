// Staged quantised matvec for sm_100a: the fast path of the decode step, with every f32 operation
// in the order of Camelid's CPU path, so its results are the CPU path's bits.
//
// Why this shape.  A decode matvec reads every weight byte once and does ~1 integer MAC per
// 4 bits: it is HBM-bound and uses no tensor cores.  What limits a simple kernel on B200 is
// the number of bytes in flight (Little's law at ~6.5 TB/s needs > 40 KB per SM) and the gaps
// between dependent launches.  So:
//   * one persistent CTA per SM walks its share of row tiles; a tile is a few consecutive rows, or for
//     long rows a run of up to 32 superblocks of each of them (a "piece"), fetched by bulk
//     asynchronous copies (cp.async.bulk, the non-tensor TMA path: one copy when the piece is whole
//     rows, else one per row) into a shared-memory ring of 4 or 8 stages guarded by mbarriers
//     (full: transaction bytes, empty: one arrival per warp);
//   * a dedicated producer warp issues the copies; it starts BEFORE the kernel waits on its
//     predecessor (griddepcontrol.wait), because weights never depend on earlier kernels — under
//     programmatic dependent launch the ring fills while the previous kernel drains;
//   * the consumer warps first build the quantised activation in shared memory — optionally
//     fused with RMSNorm or SwiGLU so no separate kernel and no global round trip is needed —
//     then each lane owns whole superblocks (Q4_K/Q6_K) or 32-value blocks (Q8_0) and computes their
//     integer dot products with dp4a;
//   * the f32 part of a row is a dependent chain in block order on the CPU (q4_k_dot_scalar,
//     src/diffusion_gemma/refmath.rs:504-562: two fused multiply-adds per superblock;
//     q6_k_wire_row_dot, src/inference.rs:25535-25581: eight accumulators by index mod 8, then their
//     left-to-right sum; q8_0_dot_rows, src/inference.rs:26191-26199: ((isum*ws)*xs) added block by
//     block, in the Camelid tree).  The lanes hand their per-block terms over through a small
//     per-warp buffer and a few "chain lanes" walk them in that order, so the result has the CPU's
//     bits; the chains cost latency only, which the other warps cover;
//   * sixteen consumer warps in four groups; group g takes units g, g+4, ... of the CTA's sequence (a
//     ring stage belongs to one group: the stage count is a multiple of the group count);
//   * paired mode (gate and up of an FFN): two neighbouring groups take the same rows of the two
//     matrices at the same time and the first writes SwiGLU(first, second);
//   * peer mode (tensor parallel): the epilogue stores this rank's partial rows into a slot on every rank and
//     the last CTA raises arrival words; the next launch's prologue waits for all ranks' words and takes the
//     sum of the partial rows as its RMSNorm input — the all-reduce of the sublayer without a collective kernel.
//
// Every wait (mbarrier, arrival word) is bounded: when the bound passes a thread records
// CMLD_ERR_TIMEOUT in *status and carries on (results are then invalid, the host reports the
// error), so a lost copy or a peer that went away can never hang the GPU.
#include "actquant.cuh"
#include "exact_sum.cuh"

namespace cmld {

constexpr int kPipeGroups = 4;      // consumer groups; group g takes this CTA's units g, g+4, ...
constexpr int kPipeGroupWarps = 4;  // warps that share one tile
constexpr int kPipeAllWarps = kPipeGroupWarps * kPipeGroups;
constexpr int kPipeConsumers = kPipeAllWarps * 32;
constexpr int kPipeThreads = kPipeConsumers + 32;  // + the producer warp
constexpr int kPipeMaxStages = 8;
constexpr int kActRec = 336;       // one Q8_K activation superblock for Q4_K rows (21 x 16 B: conflict-free lane stride)
constexpr int kRecBsum16 = 256;    // 16 x i16 sums of 16 codes
constexpr int kRecBsum32 = 288;    // 8 x i16 sums of 32 codes
constexpr int kRecD = 304;         // f32 scale
// The same superblock for Q6_K rows: q6_k_wire_row_dot keeps eight accumulators by (index mod 8), so
// the integer dot of a 16-value scale group is needed as eight pair sums x[l]*w[l] + x[l+8]*w[l+8].
// Group j holds eight words: Ylo_k = [x(2k), x(2k+8), 0, 0] for k = 0..3, then Yhi_k =
// [0, 0, x(2k+1), x(2k+9)]: a dp4a of the pair-interleaved weight word [w(2k), w(2k+8), w(2k+1),
// w(2k+9)] with Ylo_k / Yhi_k is the pair sum for l = 2k / 2k+1.
constexpr int kActRec6 = 528;      // 16 groups x 32 B + scale (33 x 16 B: conflict-free lane stride)
constexpr int kRec6D = 512;
constexpr int kTermBytes = 2048;   // per consumer warp: the terms of one pass over 32 blocks
constexpr int kPieceBlocks = 32;   // superblocks (K-quants) per row in a piece
constexpr int kPieceBlocks0 = 256; // 32-value blocks (Q8_0) per row in a piece (rows of up to 8192 values stay whole)
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
  int32_t n_it;          // blocks (Q8_0) or superblocks (K-quants) per row
  int32_t n_pieces;      // pieces a row is cut into
  int32_t piece_blocks;  // blocks per piece (the last piece may be shorter)
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
  int32_t need_k4, need_k6, need_0;
  int32_t paired;  // two matrices of equal shape and type: the result is SwiGLU(first, second)
  int32_t off_act_k, off_act_6, off_act_0, off_red, off_pair, off_term, off_ring;
  float *norm_out;        // optional f32 copy of the normalised row (written by CTA 0)
  int32_t *status;
  GemvPeer peer;          // tensor-parallel sum folded into this launch (tx_n / rx_n = 0: none)
  int64_t peer_rank_stride;  // floats between the ranks' partials in the receive slot
  KvPrefetch pf;
};

// One Q8_K chunk (the codes of 256 values, 8 per lane, scale d) into the shared-memory operand records.
__device__ __forceinline__ void emit_q8k(uint2 pk, float d, int lane, bool k4, bool k6, uint8_t *rec4, uint8_t *rec6) {
  if (k4) {
    *reinterpret_cast<uint2 *>(rec4 + lane * 8) = pk;
    int s16 = __dp4a((int)pk.y, 0x01010101, __dp4a((int)pk.x, 0x01010101, 0));
    s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) reinterpret_cast<short *>(rec4 + kRecBsum16)[lane >> 1] = (short)s16;
    if ((lane & 3) == 0) reinterpret_cast<short *>(rec4 + kRecBsum32)[lane >> 2] = (short)s32;
    if (lane == 0) *reinterpret_cast<float *>(rec4 + kRecD) = d;
  }
  if (k6) {
    // a 16-value group lives in two neighbouring lanes: the even one holds values 0..7, the odd one 8..15
    const uint32_t ox = __shfl_xor_sync(0xffffffffu, pk.x, 1), oy = __shfl_xor_sync(0xffffffffu, pk.y, 1);
    const bool odd = lane & 1;
    const uint32_t a0 = odd ? ox : pk.x, a1 = odd ? oy : pk.y, b0 = odd ? pk.x : ox, b1 = odd ? pk.y : oy;
    uint4 o;
    if (!odd) {  // Ylo_k = [x(2k), x(2k+8), 0, 0]
      o.x = __byte_perm(a0, b0, 0x0040) & 0x0000ffffu;
      o.y = __byte_perm(a0, b0, 0x0062) & 0x0000ffffu;
      o.z = __byte_perm(a1, b1, 0x0040) & 0x0000ffffu;
      o.w = __byte_perm(a1, b1, 0x0062) & 0x0000ffffu;
    } else {     // Yhi_k = [0, 0, x(2k+1), x(2k+9)]
      o.x = __byte_perm(a0, b0, 0x5100) & 0xffff0000u;
      o.y = __byte_perm(a0, b0, 0x7300) & 0xffff0000u;
      o.z = __byte_perm(a1, b1, 0x5100) & 0xffff0000u;
      o.w = __byte_perm(a1, b1, 0x7300) & 0xffff0000u;
    }
    *reinterpret_cast<uint4 *>(rec6 + 32 * (lane >> 1) + 16 * (int)odd) = o;
    if (lane == 0) *reinterpret_cast<float *>(rec6 + kRec6D) = d;
  }
}

// Quantises one 256-value chunk (8 values per lane) of batch row b into the shared-memory operands.
__device__ __forceinline__ void emit_chunk(const float (&v)[8], const PipeArgs &a, int b, int ch, int lane, uint8_t *act_k,
                                           uint8_t *act_6, uint8_t *act_0, int nsb, int act0_col_stride) {
  const int e0 = ch * 256 + lane * 8;
  if (a.need_k4 | a.need_k6) {
    int q[8];
    float d;
    q8k_quantise_chunk(v, lane, q, d);
    emit_q8k(pack8(q), d, lane, a.need_k4 != 0, a.need_k6 != 0, act_k + (b * nsb + ch) * kActRec, act_6 + (b * nsb + ch) * kActRec6);
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

constexpr int kRxChunks = 2;  // chunks a warp holds in registers in the norm prologue: hidden <= 16 * 2 * 256

// ---------------------------------------------------------------- per-superblock integer dots (shared memory operands)

// Q4_K: S[b] = sum_g sc_g * dot32_g and P[b] = sum_g min_g * bsum32_g, the two integers of refmath.rs:504-562.
template <int B>
__device__ __forceinline__ void sb_ints_q4k(const uint8_t *blk, const uint8_t *rec, int rec_col_stride, int (&S)[B], int (&P)[B],
                                            float &dw, float &dmw) {
  const uint4 meta = *reinterpret_cast<const uint4 *>(blk);
  dw = f16_bits_to_f32((uint16_t)(meta.x & 0xffff));
  dmw = f16_bits_to_f32((uint16_t)(meta.x >> 16));
  // 6-bit scales/mins as bytes (q4_k_scale_min, src/tensor/mod.rs:5997-6006): groups 0..3 and 4..7
  const uint32_t sc03 = meta.y & 0x3f3f3f3fu, m03 = meta.z & 0x3f3f3f3fu;
  const uint32_t sc47 = (meta.w & 0x0f0f0f0fu) | ((meta.y >> 2) & 0x30303030u);
  const uint32_t m47 = ((meta.w >> 4) & 0x0f0f0f0fu) | ((meta.z >> 2) & 0x30303030u);
#pragma unroll
  for (int b = 0; b < B; ++b) S[b] = 0;
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
    for (int b = 0; b < B; ++b) S[b] += dl[b] * sl + (dh[b] >> 4) * sh;
  }
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int4 bs = *reinterpret_cast<const int4 *>(rec + b * rec_col_stride + kRecBsum32);  // 8 x i16 sums of 32 codes
    int p = __dp2a_lo(bs.x, (int)m03, 0);
    p = __dp2a_hi(bs.y, (int)m03, p);
    p = __dp2a_lo(bs.z, (int)m47, p);
    P[b] = __dp2a_hi(bs.w, (int)m47, p);
  }
}

// One 16-value scale group of a Q6_K superblock: n = its four code words as 4*(q-32) in natural
// order.  aux[b][l] += sc * (pair sum l) * 4.
template <int B>
__device__ __forceinline__ void q6k_group(const uint4 &n, int sc, const uint8_t *y, int rec6_col_stride, int (&aux)[B][8]) {
  const int v0 = (int)__byte_perm(n.x, n.z, 0x5140), v1 = (int)__byte_perm(n.x, n.z, 0x7362);
  const int v2 = (int)__byte_perm(n.y, n.w, 0x5140), v3 = (int)__byte_perm(n.y, n.w, 0x7362);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int4 ylo = *reinterpret_cast<const int4 *>(y + b * rec6_col_stride);
    const int4 yhi = *reinterpret_cast<const int4 *>(y + b * rec6_col_stride + 16);
    aux[b][0] += sc * __dp4a(v0, ylo.x, 0);
    aux[b][1] += sc * __dp4a(v0, yhi.x, 0);
    aux[b][2] += sc * __dp4a(v1, ylo.y, 0);
    aux[b][3] += sc * __dp4a(v1, yhi.y, 0);
    aux[b][4] += sc * __dp4a(v2, ylo.z, 0);
    aux[b][5] += sc * __dp4a(v2, yhi.z, 0);
    aux[b][6] += sc * __dp4a(v3, ylo.w, 0);
    aux[b][7] += sc * __dp4a(v3, yhi.w, 0);
  }
}

// Q6_K: aux[b][l] = 4 * sum_j sc_j * (x[16j+l]*a[16j+l] + x[16j+8+l]*a[16j+8+l]), the eight integers of
// src/inference.rs:25560-25575 (times four: the signed codes are built as (q ^ 32) << 2, which is
// 4*(q-32) as a signed byte, so no offset correction is needed).
template <int B>
__device__ __forceinline__ void sb_ints_q6k(const uint8_t *blk, const uint8_t *rec6, int rec6_col_stride, int (&aux)[B][8]) {
  const int4 scw = *reinterpret_cast<const int4 *>(blk + 192);  // 16 signed scales
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int l = 0; l < 8; ++l) aux[b][l] = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint4 qh = *reinterpret_cast<const uint4 *>(blk + 128 + 32 * h + 16 * c);
      // flip the top bit of every 2-bit field: q ^ 32
      qh.x ^= 0xaaaaaaaau, qh.y ^= 0xaaaaaaaau, qh.z ^= 0xaaaaaaaau, qh.w ^= 0xaaaaaaaau;
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        const uint4 ql = *reinterpret_cast<const uint4 *>(blk + 64 * h + 32 * sp + 16 * c);
        const int jlo = 8 * h + 2 * sp + c;  // 16-value group of the low-nibble stream; the high stream is jlo + 4
        const int sl = 6 - 2 * sp, sh = 2 - 2 * sp;  // field sp / field 2+sp of qh moved to bits 6..7
        uint4 lo, hi;
        lo.x = ((ql.x << 2) & 0x3c3c3c3cu) | ((qh.x << sl) & 0xc0c0c0c0u);
        lo.y = ((ql.y << 2) & 0x3c3c3c3cu) | ((qh.y << sl) & 0xc0c0c0c0u);
        lo.z = ((ql.z << 2) & 0x3c3c3c3cu) | ((qh.z << sl) & 0xc0c0c0c0u);
        lo.w = ((ql.w << 2) & 0x3c3c3c3cu) | ((qh.w << sl) & 0xc0c0c0c0u);
        hi.x = ((ql.x >> 2) & 0x3c3c3c3cu) | ((qh.x << sh) & 0xc0c0c0c0u);
        hi.y = ((ql.y >> 2) & 0x3c3c3c3cu) | ((qh.y << sh) & 0xc0c0c0c0u);
        hi.z = ((ql.z >> 2) & 0x3c3c3c3cu) | ((qh.z << sh) & 0xc0c0c0c0u);
        hi.w = ((ql.w >> 2) & 0x3c3c3c3cu) | ((qh.w << sh) & 0xc0c0c0c0u);
        const int wsel = jlo >> 2, bsel = jlo & 3;  // scale jlo is byte bsel of word wsel; jlo+4 is the same byte of the next word
        const int w_lo = wsel == 0 ? scw.x : (wsel == 1 ? scw.y : (wsel == 2 ? scw.z : scw.w));
        const int w_hi = wsel == 0 ? scw.y : (wsel == 1 ? scw.z : (wsel == 2 ? scw.w : 0));
        const int slo = (int)(int8_t)(w_lo >> (8 * bsel)), shi = (int)(int8_t)(w_hi >> (8 * bsel));
        q6k_group<B>(lo, slo, rec6 + 32 * jlo, rec6_col_stride, aux);
        q6k_group<B>(hi, shi, rec6 + 32 * (jlo + 4), rec6_col_stride, aux);
      }
    }
  }
}

// Shape of a job's lane assignment: L lanes per row, rpw rows per warp.
__host__ __device__ __forceinline__ int lanes_per_row(int n_it) { return n_it < 32 ? n_it : 32; }
// K-quant rows shorter than a few superblocks (column shards of a tensor-parallel split) keep a minimum of lanes per
// row, the spare ones idle: the chain lanes of a warp serve at most 8 (Q4_K) / 2 (Q6_K) rows (see chain_slot).
__host__ __device__ __forceinline__ int lanes_per_row_k(int qt, int n_it) {
  const int L = lanes_per_row(n_it), lo = qt == CMLD_Q6_K ? 16 : 4;
  return L < lo ? lo : L;
}

// The chain lanes.  After tile_dot, res[k] of a chain lane is a finished or running row sum; this says which
// (row of the tile, batch column) it belongs to.  Q4_K: rounds of up to 4 columns; Q8_0: one round of all
// columns; Q6_K: rounds of 2 columns (at most two rows per warp), eight lanes per (row, column), result in the first of them.
template <int B>
__device__ __forceinline__ bool chain_slot(int qt, int rpw, int k, int lane, int &r, int &b) {
  if (qt == CMLD_Q4_K) {
    const int nb = min(4, B - 4 * k);
    if (nb <= 0 || lane >= rpw * nb) return false;
    r = lane / nb;
    b = 4 * k + lane % nb;
    return true;
  }
  if (qt == CMLD_Q6_K) {
    const int nb = min(2, B - 2 * k);
    if (nb <= 0 || lane >= rpw * nb * 8 || (lane & 7)) return false;
    r = (lane >> 3) / nb;
    b = 2 * k + (lane >> 3) % nb;
    return true;
  }
  if (k != 0 || lane >= rpw * B) return false;
  r = lane / B;
  b = lane % B;
  return true;
}

// One staged piece: rows wg*rpw .. of the tile, blocks [it0, it0+cnt_it) of each.  res[] carries the chain
// lanes' running sums from piece to piece; `last` finishes them (Q6_K: the left-to-right sum of the eight).
// The warp gives the stage back (one arrival on empty_bar) as soon as it has read its last byte of it — before
// the chains, which only use the term buffer — so the producer can refill the stage while the chains run.
// Piece layout in the stage: whole rows (stride J.stride) when the job has one piece; else per row
// [blocks | scales]: Q4_K cnt*144; Q6_K cnt*208 then cnt f16 d; Q8_0 cnt*32 codes then cnt f16 scales.
template <int B>
__device__ __forceinline__ void tile_dot(const PipeArgs &a, const PipeJob &J, const uint8_t *tile, int nrows, int wg, int lane,
                                         int it0, int cnt_it, bool last, const uint8_t *act_k, const uint8_t *act_6,
                                         const uint8_t *act_0, int nsb, int act0_col_stride, float *tb, float (&res)[B],
                                         uint64_t *empty_bar, bool release, int L, int rpw, int lis, int rsub) {
  const int r_local = wg * rpw + rsub;
  const bool row_ok = lane < rpw * L && r_local < nrows;
  const int rec_col_stride = nsb * kActRec, rec6_col_stride = nsb * kActRec6;
  const bool whole = J.n_pieces == 1;
  if (J.qt == CMLD_Q4_K) {
    const int row_bytes = whole ? (int)J.stride : cnt_it * 144;
    const uint8_t *row = tile + (int64_t)r_local * row_bytes;
    float4 *t4 = reinterpret_cast<float4 *>(tb);
    constexpr int R = (B + 3) / 4;
    for (int p0 = 0; p0 < cnt_it; p0 += 32) {
      const int i = p0 + lis, cnt = min(L, cnt_it - p0);
      const bool act = row_ok && i < cnt_it;
      int S[B], P[B];
      float dw = 0.0f, dmw = 0.0f;
      if (act) sb_ints_q4k<B>(row + i * 144, act_k + (it0 + i) * kActRec, rec_col_stride, S, P, dw, dmw);
      if (release && p0 + 32 >= cnt_it) {
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar);
      }
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const int nb = (B - 4 * k) < 4 ? (B - 4 * k) : 4;
        if (act) {
#pragma unroll
          for (int bb = 0; bb < nb; ++bb) {
            const int b = 4 * k + bb;
            const float xd = *reinterpret_cast<const float *>(act_k + b * rec_col_stride + (it0 + i) * kActRec + kRecD);
            // sumf = fma(-dmin, prod, sumf); sumf = fma(d, S, sumf) with d = xd*dw, dmin = xd*dminw (refmath.rs:529, :560)
            t4[lane * nb + bb] = make_float4(__fmul_rn(xd, dw), (float)S[b], -__fmul_rn(xd, dmw), (float)P[b]);
          }
        }
        __syncwarp();
        if (lane < rpw * nb) {
          const int r = lane / nb, bb = lane % nb;
          if (wg * rpw + r < nrows) {
            float s = res[k];
            const float4 *tp = t4 + r * L * nb + bb;
            int j = 0;
            for (; j + 8 <= cnt; j += 8) {  // eight terms loaded, then their sixteen dependent multiply-adds
              float4 t[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) t[u] = tp[(j + u) * nb];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                s = __fmaf_rn(t[u].z, t[u].w, s);
                s = __fmaf_rn(t[u].x, t[u].y, s);
              }
            }
            for (; j < cnt; ++j) {
              const float4 t = tp[j * nb];
              s = __fmaf_rn(t.z, t.w, s);
              s = __fmaf_rn(t.x, t.y, s);
            }
            res[k] = s;
          }
        }
        __syncwarp();
      }
    }
  } else if (J.qt == CMLD_Q6_K) {
    const int row_bytes = whole ? (int)J.stride : (int)round_up16(cnt_it * 208 + cnt_it * 2);
    const uint8_t *row = tile + (int64_t)r_local * row_bytes;
    const uint16_t *dws = reinterpret_cast<const uint16_t *>(row + (whole ? J.n_it : cnt_it) * 208);
    constexpr int R = (B + 1) / 2;
    for (int p0 = 0; p0 < cnt_it; p0 += 32) {
      const int i = p0 + lis, cnt = min(L, cnt_it - p0);
      const bool act = row_ok && i < cnt_it;
      int aux[B][8];
      float dw = 0.0f;
      if (act) {
        sb_ints_q6k<B>(row + i * 208, act_6 + (it0 + i) * kActRec6, rec6_col_stride, aux);
        dw = f16_bits_to_f32(dws[i]);
      }
      if (release && p0 + 32 >= cnt_it) {
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar);
      }
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const int nb = (B - 2 * k) < 2 ? (B - 2 * k) : 2;
        if (act) {
#pragma unroll
          for (int bb = 0; bb < nb; ++bb) {
            const int b = 2 * k + bb;
            const float xd = *reinterpret_cast<const float *>(act_6 + b * rec6_col_stride + (it0 + i) * kActRec6 + kRec6D);
            const float dd = __fmul_rn(dw, xd);  // src/inference.rs:25545
            // sums[l] += dd * (float)aux[l]: the product here, the addition in block order by the chain lanes
            float4 *dst = reinterpret_cast<float4 *>(tb + (lane * nb + bb) * 8);
            dst[0] = make_float4(__fmul_rn(dd, (float)(aux[b][0] >> 2)), __fmul_rn(dd, (float)(aux[b][1] >> 2)),
                                 __fmul_rn(dd, (float)(aux[b][2] >> 2)), __fmul_rn(dd, (float)(aux[b][3] >> 2)));
            dst[1] = make_float4(__fmul_rn(dd, (float)(aux[b][4] >> 2)), __fmul_rn(dd, (float)(aux[b][5] >> 2)),
                                 __fmul_rn(dd, (float)(aux[b][6] >> 2)), __fmul_rn(dd, (float)(aux[b][7] >> 2)));
          }
        }
        __syncwarp();
        if (lane < rpw * nb * 8) {
          const int l = lane & 7, r = (lane >> 3) / nb, bb = (lane >> 3) % nb;
          if (wg * rpw + r < nrows) {
            float s = res[k];
            const float *tp = tb + (r * L * nb + bb) * 8 + l;
            int j = 0;
            for (; j + 8 <= cnt; j += 8) {
              float t[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) t[u] = tp[(j + u) * nb * 8];
#pragma unroll
              for (int u = 0; u < 8; ++u) s = __fadd_rn(s, t[u]);
            }
            for (; j < cnt; ++j) s = __fadd_rn(s, tp[j * nb * 8]);
            res[k] = s;
          }
        }
        __syncwarp();
      }
    }
    if (last) {
#pragma unroll
      for (int k = 0; k < R; ++k) {
        float tot = 0.0f;  // 0 + sums[0] + sums[1] + ... (src/inference.rs:25578-25580)
#pragma unroll
        for (int l = 0; l < 8; ++l) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, res[k], (lane & ~7) + l));
        res[k] = tot;
      }
    }
  } else {
    // Q8_0: a lane owns 32-value blocks
    const int row_bytes = whole ? (int)J.stride : (int)round_up16(cnt_it * 32 + cnt_it * 2);
    const uint8_t *row = tile + (int64_t)r_local * row_bytes;
    const uint16_t *wss = reinterpret_cast<const uint16_t *>(row + (whole ? a.cols : cnt_it * 32));
    for (int p0 = 0; p0 < cnt_it; p0 += 32) {
      const int i = p0 + lis, cnt = min(L, cnt_it - p0);
      const bool act = row_ok && i < cnt_it;
      if (act) {
        // the two 16-byte halves are read in an order that keeps the eight lanes of a shared-memory phase on distinct banks
        const int hs = (lane >> 2) & 1;
        const uint4 w0 = *reinterpret_cast<const uint4 *>(row + i * 32 + 16 * hs);
        const uint4 w1 = *reinterpret_cast<const uint4 *>(row + i * 32 + 16 * (hs ^ 1));
        const float ws = f16_bits_to_f32(wss[i]);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const uint8_t *xa = act_0 + b * act0_col_stride;
          const int4 x0 = *reinterpret_cast<const int4 *>(xa + (it0 + i) * 32 + 16 * hs);
          const int4 x1 = *reinterpret_cast<const int4 *>(xa + (it0 + i) * 32 + 16 * (hs ^ 1));
          int isum = __dp4a((int)w0.x, x0.x, 0);
          isum = __dp4a((int)w0.y, x0.y, isum);
          isum = __dp4a((int)w0.z, x0.z, isum);
          isum = __dp4a((int)w0.w, x0.w, isum);
          isum = __dp4a((int)w1.x, x1.x, isum);
          isum = __dp4a((int)w1.y, x1.y, isum);
          isum = __dp4a((int)w1.z, x1.z, isum);
          isum = __dp4a((int)w1.w, x1.w, isum);
          const float xs = reinterpret_cast<const float *>(xa + round_up16(a.cols))[it0 + i];
          tb[b * 32 + lane] = __fmul_rn(__fmul_rn((float)isum, ws), xs);  // src/inference.rs:26198
        }
      }
      __syncwarp();
      if (release && p0 + 32 >= cnt_it && lane == 0) mbar_arrive(empty_bar);
      if (lane < rpw * B) {
        const int r = lane / B, bb = lane % B;
        if (wg * rpw + r < nrows) {
          float s = res[0];
          const float *tp = tb + bb * 32 + r * L;
          int j = 0;
          for (; j + 8 <= cnt; j += 8) {
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = tp[j + u];
#pragma unroll
            for (int u = 0; u < 8; ++u) s = __fadd_rn(s, t[u]);
          }
          for (; j < cnt; ++j) s = __fadd_rn(s, tp[j]);
          res[0] = s;
        }
      }
      __syncwarp();
    }
  }
}

// Where unit i of a CTA's sequence lies: units come in rounds of kPipeGroups tiles (one per group), the
// pieces of a group's tile one after another, so that unit i always belongs to group i % kPipeGroups and a
// group meets the pieces of its tile in order.  Returns the index of the tile in this CTA's list.
__device__ __forceinline__ int unit_tile(int i, int n_pieces, int &piece) {
  const int per_round = kPipeGroups * n_pieces;
  piece = (i % per_round) / kPipeGroups;
  return (i / per_round) * kPipeGroups + i % kPipeGroups;
}

// Job and first row of tile t of the launch (the jobs' tiles are numbered one after another).
__device__ __forceinline__ int tile_job(const PipeArgs &a, int t) {
  int j = 0;
  if (a.n_jobs > 1 && t >= a.job[1].first_tile) j = 1;
  if (a.n_jobs > 2 && t >= a.job[2].first_tile) j = 2;
  return j;
}

// ---------------------------------------------------------------- the kernel

template <int B, bool SHORT_ROWS>
__global__ void __launch_bounds__(kPipeThreads, 1) gemv_pipe_kernel(const PipeArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + kPipeMaxStages;
  uint8_t *act_k = smem + a.off_act_k;
  uint8_t *act_6 = smem + a.off_act_6;
  uint8_t *act_0 = smem + a.off_act_0;
  float *red = reinterpret_cast<float *>(smem + a.off_red);
  uint8_t *ring = smem + a.off_ring;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.n_stages;
  // Tiles this CTA takes: t = blockIdx.x + k*gridDim.x.  In paired mode the unit of distribution is a pair of
  // tiles (the same rows of the two matrices), which occupies two neighbouring groups.
  const int n_dist = a.paired ? a.job[0].n_tiles : a.total_tiles;
  const int n_mine = (int)blockIdx.x < n_dist ? (n_dist - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int n_my_tiles = a.paired ? 2 * n_mine : n_mine;  // entries of this CTA's tile list
  const int n_pieces = a.job[0].n_pieces;                 // the same for every job of a launch
  const int n_units = ((n_my_tiles + kPipeGroups - 1) / kPipeGroups) * kPipeGroups * n_pieces;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kPipeGroupWarps);
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

  // per-CTA timeline (same option): CTA b's k-th launch -> four stamps after the per-launch records
  unsigned long long *trc = nullptr;
  if (a.peer.trace && tid == 0 && blockIdx.x < kTraceCtas) {
    unsigned long long *base = a.peer.trace + 1 + 8 * (size_t)kTraceRecords + (size_t)blockIdx.x * (1 + 4 * (size_t)kTraceCtaRecords);
    const unsigned long long k = base[0];
    base[0] = k + 1;
    trc = base + 1 + 4 * (k % kTraceCtaRecords);
    trc[0] = global_ns();
  }

  if (warp == kPipeAllWarps) {
    // ---------------- producer: weights do not depend on the previous kernel, so no wait here
    if (lane != 0 && a.pf.k) {
      // side job: the KV rows of the attention kernel that follows, into L2, 2 KB per request
      constexpr int kChunk = 2048;
      for (int b = 0; b < a.pf.batch; ++b) {
        const int64_t row_bytes = (int64_t)a.pf.head_dim * 2, head_bytes = (int64_t)a.pf.positions[b] * row_bytes;  // rows before the new one
        const int per_head = (int)((head_bytes + kChunk - 1) / kChunk);
        const int total = a.pf.n_kv_heads * 2 * per_head;
        for (int c = (int)blockIdx.x * 31 + lane - 1; c < total; c += (int)gridDim.x * 31) {
          const int h = c / per_head, ck = c % per_head, kvh = h >> 1;
          const __half *base = (h & 1 ? a.pf.v : a.pf.k) + (((int64_t)a.pf.slots[b] * a.pf.n_kv_heads + kvh) * a.pf.max_pos) * a.pf.head_dim;
          const int64_t off = (int64_t)ck * kChunk;
          const uint32_t bytes = (uint32_t)min((int64_t)kChunk, head_bytes - off);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t *>(base) + off), "r"(bytes) : "memory");
        }
      }
    }
    if (lane == 0) {
      for (int i = 0; i < n_units; ++i) {
        int piece;
        const int tl = unit_tile(i, n_pieces, piece);
        if (tl >= n_my_tiles) continue;  // the last round may be short (only at the end of the sequence)
        const int s = i % S;
        if (i >= S) mbar_wait(&empty[s], (uint32_t)((i / S - 1) & 1), a.status);
        int j, row0;
        if (a.paired) {
          j = tl & 1;
          row0 = ((int)blockIdx.x + (tl >> 1) * (int)gridDim.x) * a.job[0].tile_rows;
        } else {
          const int t = (int)blockIdx.x + tl * (int)gridDim.x;
          j = tile_job(a, t);
          row0 = (t - a.job[j].first_tile) * a.job[j].tile_rows;
        }
        const PipeJob &J = a.job[j];
        const int nrows = min(J.tile_rows, J.rows - row0);
        uint8_t *dst = ring + (int64_t)s * a.stage_bytes;
        if (J.n_pieces == 1) {
          const uint32_t bytes = (uint32_t)(nrows * J.stride);
          mbar_expect_tx(&full[s], bytes);
          bulk_g2s(dst, J.w + (int64_t)row0 * J.stride, bytes, &full[s]);
        } else {
          const int it0 = piece * J.piece_blocks, cnt = min(J.piece_blocks, J.n_it - it0);
          // per row: the piece's blocks, then its per-block scales (Q6_K, Q8_0), at a 16-byte aligned row pitch
          const int blk = J.qt == CMLD_Q4_K ? 144 : (J.qt == CMLD_Q6_K ? 208 : 32);
          const int main_bytes = cnt * blk, sc_bytes = J.qt == CMLD_Q4_K ? 0 : cnt * 2;
          const int pitch = (int)round_up16(main_bytes + sc_bytes);
          const int64_t sc_off = J.qt == CMLD_Q6_K ? (int64_t)J.n_it * 208 : a.cols;
          mbar_expect_tx(&full[s], (uint32_t)(nrows * (main_bytes + sc_bytes)));
          for (int r = 0; r < nrows; ++r) {
            const uint8_t *src = J.w + (int64_t)(row0 + r) * J.stride;
            bulk_g2s(dst + r * pitch, src + (int64_t)it0 * blk, (uint32_t)main_bytes, &full[s]);
            if (sc_bytes) bulk_g2s(dst + r * pitch + main_bytes, src + sc_off + it0 * 2, (uint32_t)sc_bytes, &full[s]);
          }
        }
      }
    }
    return;
  }

  // ---------------- consumers
  asm volatile("griddepcontrol.wait;" ::: "memory");  // inputs written by the previous kernel are now visible
  if (tr) tr[1] = global_ns();
  if (trc) trc[1] = global_ns();
  const int nsb = a.cols >> 8;
  const int act0_col_stride = (int)round_up16(a.cols) + (int)round_up16((a.cols >> 5) * 4);

  if (a.peer.rx_n > 0) {
    // the input rows are still spread over the ranks: wait for every rank's partial to have arrived
    if (tid < a.peer.rx_n) peer_wait(a.peer.rx_flag + tid, __ldcg(a.peer.rx_epoch), a.peer.timeout_ns, a.status);
    asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
  }
  if (tr) tr[2] = global_ns();

  // Prologue: quantised activation rows into shared memory.
  if (a.mode == 0) {
    // re-lay the pre-quantised global rows
    const int64_t astride = act_row_stride(a.cols);
    if (a.need_k4 | a.need_k6) {
      for (int idx = warp; idx < a.batch * nsb; idx += kPipeAllWarps) {
        const int b = idx / nsb, ch = idx % nsb;
        const uint2 pk = __ldg(reinterpret_cast<const uint2 *>(a.act_in + b * astride + ch * 256) + lane);
        const float d = __ldg(reinterpret_cast<const float *>(a.act_in + b * astride + act_scale_off(a.cols)) + ch);
        emit_q8k(pk, d, lane, a.need_k4 != 0, a.need_k6 != 0, act_k + idx * kActRec, act_6 + idx * kActRec6);
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
    if (chunked_norm) {
      // RMSNorm with ONE load of the row: each warp keeps its chunks in registers between the mean-square
      // pass and the scaling pass.  The squares are summed with the bits of the CPU's one-accumulator loop
      // (rms_norm_into, src/tensor/mod.rs:2740-2764; see exact_sum.cuh).  With a peer sum the row is the sum
      // of the ranks' partial rows (added in rank order, so every rank gets the same bits).
      float *sq = reinterpret_cast<float *>(smem + a.off_term);  // the term buffers are idle during the prologue
      uint8_t *ws = smem + a.off_term + a.cols * 4;
      float hv[kRxChunks][8];
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
          float4 q0, q1;
#pragma unroll
          for (int i = 0; i < 8; ++i) hv[k][i] = t[i];
          q0 = make_float4(__fmul_rn(t[0], t[0]), __fmul_rn(t[1], t[1]), __fmul_rn(t[2], t[2]), __fmul_rn(t[3], t[3]));
          q1 = make_float4(__fmul_rn(t[4], t[4]), __fmul_rn(t[5], t[5]), __fmul_rn(t[6], t[6]), __fmul_rn(t[7], t[7]));
          reinterpret_cast<float4 *>(sq + ch * 256 + lane * 8)[0] = q0;
          reinterpret_cast<float4 *>(sq + ch * 256 + lane * 8)[1] = q1;
          if (blockIdx.x == 0 && a.peer.rx_out) {
            float4 *o4 = reinterpret_cast<float4 *>(a.peer.rx_out + (int64_t)b * a.cols + ch * 256 + lane * 8);
            o4[0] = s0;
            o4[1] = s1;
          }
        }
      }
      if (tr) tr[5] = global_ns();
      const float ss = xsum::cta_sum<kPipeAllWarps>(sq, a.cols, warp, lane, 1, ws);
      if (tr) tr[7] = global_ns();
      const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.cols), a.eps)));
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
          emit_chunk(v, a, b, ch, lane, act_k, act_6, act_0, nsb, act0_col_stride);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));  // sq is reused by the next row
      continue;
    }
    if (a.mode == 0) continue;  // copied above
    const float *x = a.x + (int64_t)b * a.x_stride;
    const float *x2 = a.mode == 3 ? a.x2 + (int64_t)b * a.x_stride : nullptr;
    float scale = 1.0f;
    if (a.mode == 1) {
      // a width the chunked form does not take: the CPU's loop itself, by one thread
      if (tid == 0) {
        float t = 0.0f;
        for (int i = 0; i < a.cols; ++i) {
          const float v = __ldcg(x + i);
          t = __fadd_rn(t, __fmul_rn(v, v));
        }
        red[0] = t;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
      scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(red[0], (float)a.cols), a.eps)));
      asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
    }
    const int n_chunks = (a.cols + 255) >> 8;
    // the next chunk's values are requested before the current chunk is quantised: one exposed memory latency per
    // row instead of one per chunk (the down projection's 14336 values are 3.5 chunks per warp)
    float4 nxa = make_float4(0.0f, 0.0f, 0.0f, 0.0f), nxb = nxa;
    if (warp < n_chunks && warp * 256 + lane * 8 + 8 <= a.cols) {
      nxa = __ldcg(reinterpret_cast<const float4 *>(x + warp * 256 + lane * 8));
      nxb = __ldcg(reinterpret_cast<const float4 *>(x + warp * 256 + lane * 8) + 1);
    }
    for (int ch = warp; ch < n_chunks; ch += kPipeAllWarps) {
      const int e0 = ch * 256 + lane * 8;
      float v[8];
      const float4 xa = nxa, xb = nxb;
      {
        const int e1 = e0 + kPipeAllWarps * 256;
        if (ch + kPipeAllWarps < n_chunks && e1 + 8 <= a.cols) {
          nxa = __ldcg(reinterpret_cast<const float4 *>(x + e1));
          nxb = __ldcg(reinterpret_cast<const float4 *>(x + e1) + 1);
        }
      }
      if (e0 + 8 <= a.cols) {
        // 8 consecutive values per lane: two 128-bit loads per operand (cols is a multiple of 32)
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
      emit_chunk(v, a, b, ch, lane, act_k, act_6, act_0, nsb, act0_col_stride);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));
  if (tr) tr[3] = global_ns();
  if (trc) trc[2] = global_ns();

  // Main loop over this CTA's units; group g takes units g, g + kPipeGroups, ...
  const int group = warp / kPipeGroupWarps, wg = warp % kPipeGroupWarps;
  float *tb = reinterpret_cast<float *>(smem + a.off_term + warp * kTermBytes);
  float *pairbuf = reinterpret_cast<float *>(smem + a.off_pair);  // paired mode: [pair slot][tile_rows][B]
  float res[B];
  int done_pairs = 0;
  // lane geometry of the two block sizes a launch can hold (every job has the same number of columns), once:
  // the divisions are not repeated per tile
  // (SHORT_ROWS: K-quant rows of fewer superblocks than 16, with a Q6_K matrix in the launch, or 4 keep that many
  // lanes per row; a separate instantiation, so that the usual shapes run the code they always ran)
  const int Lk = SHORT_ROWS ? max(lanes_per_row(nsb > 0 ? nsb : 1), a.need_k6 ? 16 : 4) : lanes_per_row(nsb > 0 ? nsb : 1);
  const int rpwk = 32 / Lk, lisk = lane % Lk, rsubk = lane / Lk;
  const int L0 = lanes_per_row(a.cols >> 5), rpw0 = 32 / L0, lis0 = lane % L0, rsub0 = lane / L0;
  // unit i -> (tile tl of this CTA's list, piece): advanced without divisions; a group's units are kPipeGroups apart
  // likewise the unit's stage i % S and the parity (i / S) & 1 of its use of that stage: S is a multiple of the
  // group count, so the stage advances by kPipeGroups and wraps
  int tl = group, piece = 0, s = group;
  uint32_t use_parity = 0;
  for (int i = group; i < n_units; i += kPipeGroups, s += kPipeGroups, use_parity ^= (s >= S ? 1u : 0u), s -= (s >= S ? S : 0)) {
    if (i != group) {
      if (++piece == n_pieces) {
        piece = 0;
        tl += kPipeGroups;
      }
    }
    if (tl >= n_my_tiles) break;
    int j, row0;
    if (a.paired) {
      j = tl & 1;
      row0 = ((int)blockIdx.x + (tl >> 1) * (int)gridDim.x) * a.job[0].tile_rows;
    } else {
      const int t = (int)blockIdx.x + tl * (int)gridDim.x;
      j = tile_job(a, t);
      row0 = (t - a.job[j].first_tile) * a.job[j].tile_rows;
    }
    const PipeJob &J = a.job[j];
    const int nrows = min(J.tile_rows, J.rows - row0);
    const int it0 = piece * J.piece_blocks, cnt_it = min(J.piece_blocks, J.n_it - it0);
    const bool last = piece == J.n_pieces - 1;
    const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[s], use_parity, a.status));
    const bool is0 = J.qt == CMLD_Q8_0;
    const int L = is0 ? L0 : Lk, rpw = is0 ? rpw0 : rpwk, lis = is0 ? lis0 : lisk, rsub = is0 ? rsub0 : rsubk;
    {
      const int wge = wg;
      if (piece == 0) {
#pragma unroll
        for (int k = 0; k < B; ++k) res[k] = 0.0f;
      }
      const bool release = true;
      if (ready) {
        tile_dot<B>(a, J, ring + (int64_t)s * a.stage_bytes, nrows, wge, lane, it0, cnt_it, last, act_k, act_6, act_0, nsb,
                    act0_col_stride, tb, res, &empty[s], release, L, rpw, lis, rsub);
      } else {
        __syncwarp();
        if (release && lane == 0) mbar_arrive(&empty[s]);
      }
      if (!last) continue;
      if (a.paired) {
        // groups 2p (first matrix) and 2p+1 (second) hold the same rows: the second hands its results over through
        // shared memory (double-buffered, one barrier of the two groups per row set) and the first writes
        // SwiGLU(first, second) — the f32 operand of the down projection — so neither product goes through memory.
        const int slot = group >> 1;
        float *buf = pairbuf + ((slot * 2 + (done_pairs & 1)) * kPipeGroupWarps * rpw) * B;
        if (group & 1) {
#pragma unroll
          for (int k = 0; k < B; ++k) {
            int r, b;
            if (chain_slot<B>(J.qt, rpw, k, lane, r, b) && wge * rpw + r < nrows) buf[(wg * rpw + r) * B + b] = res[k];
          }
        }
        if (slot == 0) asm volatile("bar.sync 2, %0;" ::"n"(2 * kPipeGroupWarps * 32));
        else asm volatile("bar.sync 3, %0;" ::"n"(2 * kPipeGroupWarps * 32));
        if (!(group & 1)) {
#pragma unroll
          for (int k = 0; k < B; ++k) {
            int r, b;
            if (chain_slot<B>(J.qt, rpw, k, lane, r, b) && wge * rpw + r < nrows)
              a.job[0].y[(int64_t)b * a.job[0].y_stride + row0 + wge * rpw + r] = swiglu(res[k], buf[(wg * rpw + r) * B + b]);
          }
        }
        ++done_pairs;
      } else if (ready) {
#pragma unroll
        for (int k = 0; k < B; ++k) {
          int r, b;
          if (chain_slot<B>(J.qt, rpw, k, lane, r, b) && wge * rpw + r < nrows) {
            const int64_t o = (int64_t)b * J.y_stride + row0 + wge * rpw + r;
            const float out = J.residual ? __fadd_rn(__ldcg(J.residual + o), res[k]) : res[k];
            if (a.peer.tx_n > 0) {
              for (int p = 0; p < a.peer.tx_n; ++p) a.peer.tx_part[p][o] = out;  // this rank's partial, onto every rank
            } else {
              J.y[o] = out;
            }
          }
        }
      }
    }
  }
  if (tr) tr[4] = global_ns();
  if (a.peer.trace) {
    asm volatile("bar.sync 1, %0;" ::"n"(kPipeConsumers));  // the CTA's last row, not thread 0's
    if (trc) trc[3] = global_ns();
  }
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
  bool short_rows;  // K-quant rows shorter than the lanes a row keeps: the SHORT_ROWS instantiation
};

static int g_sm_count = 0;
static bool g_attr_set[9] = {false};

template <int B>
static int32_t launch_pipe_b(const PipePlan &p, int grid, cudaStream_t s, bool pdl) {
  if (!g_attr_set[B]) {
    CMLD_CUDA(cudaFuncSetAttribute(gemv_pipe_kernel<B, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    CMLD_CUDA(cudaFuncSetAttribute(gemv_pipe_kernel<B, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
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
  if (p.short_rows) CMLD_CUDA(cudaLaunchKernelEx(&cfg, gemv_pipe_kernel<B, true>, p.args));
  else CMLD_CUDA(cudaLaunchKernelEx(&cfg, gemv_pipe_kernel<B, false>, p.args));
  return CMLD_OK;
}

// Tile geometry and shared-memory map for these matrices at this batch; false if it does not fit.
static bool plan_pipe(const GemvJob *jobs, int n_jobs, int32_t batch, PipePlan &p, bool &need_k4, bool &need_k6, bool &need_0,
                      int &tiles_out, bool paired, bool norm) {
  if (n_jobs < 1 || n_jobs > 3 || batch < 1 || batch > 8) return false;
  const int64_t cols = jobs[0].cols;
  if (cols % 32) return false;
  PipeArgs &a = p.args;
  need_k4 = need_k6 = need_0 = false;
  int stage = 0, tiles = 0, n_pieces = -1;
  // one lane geometry for the K-quant jobs of a launch (they share the number of superblocks per row)
  int lanes_k = 1;
  for (int k = 0; k < n_jobs; ++k)
    if (jobs[k].qt == CMLD_Q4_K || jobs[k].qt == CMLD_Q6_K) lanes_k = std::max(lanes_k, lanes_per_row_k(jobs[k].qt, (int)(cols >> 8)));
  p.short_rows = lanes_k > lanes_per_row((int)(cols >> 8) > 0 ? (int)(cols >> 8) : 1);
  for (int k = 0; k < n_jobs; ++k) {
    const GemvJob &g = jobs[k];
    if (g.cols != cols) return false;
    const int n_it = g.qt == CMLD_Q8_0 ? (int)(cols >> 5) : (int)(cols >> 8);
    const int L = g.qt == CMLD_Q8_0 ? lanes_per_row(n_it) : lanes_k, rpw = 32 / L;
    // the chain lanes of a warp must fit in it (see chain_slot)
    if (g.qt == CMLD_Q8_0) {
      need_0 = true;
      if (rpw * batch > 32) return false;
    } else {
      if (cols % 256) return false;
      if (g.qt == CMLD_Q4_K) {
        need_k4 = true;
        if (rpw > 8) return false;
      } else if (g.qt == CMLD_Q6_K) {
        need_k6 = true;
        if (rpw > 2) return false;
      } else {
        return false;
      }
    }
    const int per_piece = g.qt == CMLD_Q8_0 ? kPieceBlocks0 : kPieceBlocks;
    PipeJob &J = a.job[k];
    J.w = g.w;
    J.qt = g.qt;
    J.rows = (int32_t)g.rows;
    J.tile_rows = kPipeGroupWarps * rpw;
    J.n_it = n_it;
    J.stride = g.stride;
    J.y = g.y;
    J.residual = g.residual;
    J.y_stride = g.y_stride;
    J.first_tile = tiles;
    J.n_tiles = (int)((g.rows + J.tile_rows - 1) / J.tile_rows);
    tiles += J.n_tiles;
    if (g.stride % 16 || (reinterpret_cast<uintptr_t>(g.w) & 15)) return false;
    // whole rows when a tile of them is a moderate stage; else pieces of per_piece blocks
    const int blk = g.qt == CMLD_Q4_K ? 144 : (g.qt == CMLD_Q6_K ? 208 : 32);
    int np = 1, st = (int)(J.tile_rows * g.stride);
    J.piece_blocks = n_it;
    if (n_it > per_piece) {
      np = (n_it + per_piece - 1) / per_piece;
      J.piece_blocks = per_piece;
      // every piece's scale run must start on a 16-byte boundary and be a multiple of 16 bytes long
      if (g.qt != CMLD_Q4_K && (n_it % 8)) return false;
      st = J.tile_rows * (int)round_up16(per_piece * blk + (g.qt == CMLD_Q4_K ? 0 : per_piece * 2));
    }
    J.n_pieces = np;
    if (n_pieces < 0) n_pieces = np;
    if (np != n_pieces) return false;  // jobs of one launch are cut alike (they share cols; types may differ)
    stage = std::max(stage, st);
  }
  stage = (stage + 127) & ~127;
  const int nsb = (int)(cols >> 8);
  int off = 2 * kPipeMaxStages * 8;
  a.off_act_k = off;
  if (need_k4) off += batch * nsb * kActRec;
  off = (off + 15) & ~15;
  a.off_act_6 = off;
  if (need_k6) off += batch * nsb * kActRec6;
  off = (off + 15) & ~15;
  a.off_act_0 = off;
  if (need_0) off += batch * ((int)round_up16(cols) + (int)round_up16((cols >> 5) * 4));
  a.off_red = off;
  off += 64 * 4;
  a.off_pair = off;
  if (paired) off += 4 * a.job[0].tile_rows * batch * 4;
  off = (off + 15) & ~15;
  a.off_term = off;
  {
    int term = kPipeAllWarps * kTermBytes;
    // the norm prologue borrows this region for the squares and the exact sum's workspace
    if (norm && cols % 256 == 0 && cols <= kRxChunks * kPipeAllWarps * 256)
      term = std::max(term, (int)cols * 4 + xsum::workspace_bytes((int)cols));
    off += term;
  }
  off = (off + 127) & ~127;
  a.off_ring = off;
  // The stage count must be a multiple of the number of consumer groups: unit i lives in stage i % S and
  // belongs to group i % kPipeGroups, so every stage is only ever used by one group and a group meets the
  // phases of its stages in order (an mbarrier parity wait cannot tell phase n from n+2).
  int n_stages = std::min<int>(kPipeMaxStages, (226 * 1024 - off) / stage);
  n_stages -= n_stages % kPipeGroups;
  if (n_stages < kPipeGroups) return false;
  if (paired && (n_jobs != 2 || jobs[0].rows != jobs[1].rows || jobs[0].qt != jobs[1].qt || jobs[0].stride != jobs[1].stride)) return false;
  p.smem_bytes = off + n_stages * stage;
  a.stage_bytes = stage;
  a.n_stages = n_stages;
  tiles_out = tiles;
  return true;
}

int gemv_pipe_fit_batch(const GemvJob *jobs, int n_jobs, bool paired, bool norm) {
  for (int b = 8; b >= 1; --b) {
    PipePlan p{};
    bool k4, k6, n0;
    int tiles;
    if (plan_pipe(jobs, n_jobs, b, p, k4, k6, n0, tiles, paired, norm)) return b;
  }
  return 0;
}

// Plans and launches the staged kernel.  Returns CMLD_ERR_UNSUPPORTED (without setting an error
// message the caller would see) when the shape does not fit; the caller then uses the
// generic kernel.
int32_t launch_gemv_pipe(const GemvJob *jobs, int n_jobs, int32_t batch, const GemvPrologue &pro, int32_t *status,
                         cudaStream_t s, bool pdl, const GemvPeer *peer, const KvPrefetch *pf) {
  if (g_sm_count == 0) {
    int dev = 0;
    CMLD_CUDA(cudaGetDevice(&dev));
    CMLD_CUDA(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  PipePlan p{};
  PipeArgs &a = p.args;
  bool need_k4 = false, need_k6 = false, need_0 = false;
  int tiles = 0;
  if (!plan_pipe(jobs, n_jobs, batch, p, need_k4, need_k6, need_0, tiles, pro.pair_swiglu != 0, pro.mode == 1)) return CMLD_ERR_UNSUPPORTED;
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
  a.need_k4 = need_k4;
  a.need_k6 = need_k6;
  a.need_0 = need_0;
  a.norm_out = pro.norm_out;
  a.status = status;
  if (pf) a.pf = *pf;
  a.paired = pro.pair_swiglu ? 1 : 0;
  if (a.paired && peer && peer->tx_n > 0) return fail(CMLD_ERR_INVALID, "gemv: a paired launch does not send");
  if (peer) {
    a.peer = *peer;
    a.peer_rank_stride = (int64_t)kPeerRows * cols;
    if (peer->tx_n > 0 && (n_jobs != 1 || !status)) return fail(CMLD_ERR_INVALID, "gemv: a sending launch takes one matrix and a status word");
    if (peer->rx_n > 0 && (pro.mode != 1 || cols % 256 || cols > kRxChunks * kPipeAllWarps * 256 || !status))
      return fail(CMLD_ERR_INVALID, "gemv: a receiving launch is an RMSNorm prologue over at most %d columns", kRxChunks * kPipeAllWarps * 256);
  }
  if (a.mode == 0 && (((need_k4 || need_k6) && !a.act_in) || (need_0 && !a.act_in0))) return fail(CMLD_ERR_INVALID, "gemv: activation buffer missing");
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
