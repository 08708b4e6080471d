// Batched quantised matvec on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in
// tensor memory): 9..32 activation rows in one pass over the weights, with the CPU path's order of f32
// operations in the epilogue, so that a row's result is bit-identical to the one-row kernels'.
//
// What the tensor cores compute is the INTEGER part of the reference's dot products, which is exact in
// any order; the f32 steps that follow are done per (weight row, activation row) in block order:
//   Q8_0 (src/inference.rs:26191-26199): per 32-value block, isum = sum q*y is one K=32 MMA into its own
//     accumulator columns; then acc += ((float)isum * ws) * xs, block after block.
//   Q4_K (src/diffusion_gemma/refmath.rs:504-562): per superblock S = sum_g sc_g * (q.y)_g and
//     P = sum_g min_g * bsum_g; then acc = fma(-(xd*dmin), P, acc); acc = fma(xd*d, S, acc).
//     The 6-bit scale is split sc = 8*s1 + s0 and the A operand holds s1*q and s0*q (<= 105, one packed
//     multiply per four nibbles), so S = 8*S1 + S0 comes from two accumulators that run over the whole
//     superblock; P comes from one more MMA whose A operand is the eight mins and whose B operand the
//     activation group sums split as 64*h + l.
//   Q6_K (src/inference.rs:25545-25581): eight f32 lanes by (index mod 8): per superblock
//     aux[l] = sum_g sc_g * sum_{k in g, k = l mod 8} (q_k - 32) * y_k, then sums[l] += (d*xd) * aux[l],
//     and at the end 0 + sums[0] + ... + sums[7].  The K dimension is permuted so that MMA l covers the 32
//     values with index = l mod 8; the A operand holds u = sc*(q-32) + 4096 (in 32..8192) split as
//     128*uh + ul, and aux[l] = 128*D_hi + D_lo - 4096 * (sum of those 32 activation codes).
//
// One CTA per SM, tile = 128 weight rows x all columns, K step = 256 columns.  Warp roles:
//   warps 0-7   epilogue: two groups of four warps (a warp reads the 32 TMEM lanes of its quarter), each
//               group owns half of the CTA's activation columns; tcgen05.ld, integer fix-up, f32 chains.
//   warp 8      one lane issues the MMAs of a K step and commits them to the mbarriers.
//   warp 9      one lane brings the step's packed activation record with one bulk copy.
//   warps 10-17 weight path: cp.async of the raw wire bytes three steps ahead into a private ring (a thread
//               unpacks only what it loaded itself, so no barrier), unpack into the canonical K-major
//               operand layout; Q8_0 codes are copied straight into that layout.
// A launch with few tiles splits the activation columns over several CTAs per tile (the weights then
// come from L2 for all but one of them) so that idle SMs take part.
// Every wait is bounded: a wait that runs out sets the status word and an abort flag, all roles leave
// their loops, tensor memory is freed and the kernel returns.
#include "common.cuh"

namespace cmld {

namespace {

// Warp roles for EW epilogue warps (8: two groups of four, each with half of the CTA's activation columns; 4: one group,
// for launches of eight columns per CTA, whose threads can then have more registers): epilogue 0..EW-1, MMA issue EW,
// activation records EW+1, weight path EW+2..EW+9.
constexpr int tc_threads(int ew) { return (ew + 10) * 32; }
constexpr int kTcUnpackThreads = 256;
constexpr int kTcRows = 128;
constexpr int kTcRawStages = 3;
constexpr int kTcPrefetchAhead = 6;  // K steps by which a row's wire bytes are asked into L2 before they are copied
constexpr int kTcMaxActStages = 8;
constexpr int kScaleAhead = 4;  // steps by which the epilogue asks for a row's scales ahead of their use
constexpr int kTcPlane = kTcRows * 256;  // one operand plane of a K step: 128 rows x 256 bytes
constexpr uint32_t kTcSpin = 1u << 22;

// packed activation record of one K step and one group of eight activation rows
constexpr int kRecB1 = 2048;                         // codes, [k/16][row%8][16]
constexpr int kRecQ4 = kRecB1 + 512 + 32;            // + group-sum pieces [piece][k/16 of 2][8][16] + xd[8]
constexpr int kRecQ6 = kRecB1 + 256 + 32;            // + class sums i32 [8 l][8] + xd[8]
constexpr int kRecQ8 = kRecB1 + 256;                 // + xs f32 [8 blocks][8]

__host__ __device__ constexpr int rec_bytes(int qt) { return qt == CMLD_Q4_K ? kRecQ4 : qt == CMLD_Q6_K ? kRecQ6 : kRecQ8; }

struct TcJob {
  const uint8_t *w;
  int32_t rows, first_tile, n_tiles;
  int64_t stride;
  float *y;
  const float *residual;
  int64_t y_stride;
};

struct TcArgs {
  TcJob job[3];
  int32_t n_jobs, total_tiles, nks, batch;
  int32_t groups_total;  // activation row groups (of eight) in the packed records
  int32_t ng;            // groups one CTA takes (1, 2 or 4)
  int32_t n_splits;      // CTAs per tile = groups_total / ng
  int32_t a_stages;      // operand ring depth: 2 (K-quants), 4 (Q8_0)
  int32_t a_stage_bytes, off_a, off_raw, off_act, act_stage_bytes, act_stages, off_scale, off_bar;
  const uint8_t *pack;
  int32_t *status;
};

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(s32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait.  Gives up when the limit is reached or another role has already given up.
__device__ __forceinline__ bool bar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int32_t *status) {
  for (uint32_t i = 0; i < kTcSpin; ++i) {
    if (bar_try(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
    __nanosleep(40);  // leave the issue slots to the warps that have work
  }
  *abort_flag = 1;
  if (status) atomicExch(status, (int32_t)CMLD_ERR_TIMEOUT);
  return false;
}

__device__ __forceinline__ void cp16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp4(void *dst_smem, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand without swizzle: 8 rows x 16 bytes are contiguous; LBO = bytes between the 16-byte chunks
// along K, SBO = bytes between groups of eight rows (descriptor version 1 in bits 46-47).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// kind::i8, D = S32, B signed, both K-major, M = 128
__device__ __forceinline__ uint32_t instr_desc(int n, bool a_unsigned) {
  return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
// tcgen05.ld is asynchronous: its registers are valid only after tcgen05.wait::ld.  Load(s) and wait sit in ONE
// asm statement, so the compiler cannot move a use of the registers between them, and every output is an
// early clobber: an address operand sharing a register with an output of an earlier load in the same statement
// would be overwritten whenever that load's write-back lands first.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8x2(uint32_t t0, int (&a)[8], uint32_t t1, int (&b)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%16];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%17];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=&r"(a[0]), "=&r"(a[1]), "=&r"(a[2]), "=&r"(a[3]), "=&r"(a[4]), "=&r"(a[5]), "=&r"(a[6]), "=&r"(a[7]), "=&r"(b[0]), "=&r"(b[1]),
        "=&r"(b[2]), "=&r"(b[3]), "=&r"(b[4]), "=&r"(b[5]), "=&r"(b[6]), "=&r"(b[7])
      : "r"(t0), "r"(t1)
      : "memory");
}

__device__ __forceinline__ void tmem_ld8x4(uint32_t t0, int (&a)[8], uint32_t t1, int (&b)[8], uint32_t t2, int (&c)[8], uint32_t t3, int (&d)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%32];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%33];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%16,%17,%18,%19,%20,%21,%22,%23}, [%34];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%24,%25,%26,%27,%28,%29,%30,%31}, [%35];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=&r"(a[0]), "=&r"(a[1]), "=&r"(a[2]), "=&r"(a[3]), "=&r"(a[4]), "=&r"(a[5]), "=&r"(a[6]), "=&r"(a[7]), "=&r"(b[0]), "=&r"(b[1]),
        "=&r"(b[2]), "=&r"(b[3]), "=&r"(b[4]), "=&r"(b[5]), "=&r"(b[6]), "=&r"(b[7]), "=&r"(c[0]), "=&r"(c[1]), "=&r"(c[2]), "=&r"(c[3]),
        "=&r"(c[4]), "=&r"(c[5]), "=&r"(c[6]), "=&r"(c[7]), "=&r"(d[0]), "=&r"(d[1]), "=&r"(d[2]), "=&r"(d[3]), "=&r"(d[4]), "=&r"(d[5]),
        "=&r"(d[6]), "=&r"(d[7])
      : "r"(t0), "r"(t1), "r"(t2), "r"(t3)
      : "memory");
}

// The epilogue gives a step's accumulator slot and activation record back.  Called AFTER the step's f32 work, so
// that every value read from the record has been consumed by an instruction: a shared-memory load that is merely
// issued is not ordered before the arrival, and the next bulk copy into the stage (async proxy) overtook such
// loads now and then, handing the chain the scale of a later step.  The proxy fence orders this thread's generic
// reads before async-proxy writes that follow the arrival.
__device__ __forceinline__ void release_step(uint64_t *acc_empty, uint64_t *b_empty, int lane) {
  tc_fence_before();
  fence_async_smem();
  __syncwarp();
  if (lane == 0) {
    bar_arrive(acc_empty);
    bar_arrive(b_empty);
  }
}

__device__ __forceinline__ int tc_tile_job(const TcArgs &a, int t) {
  int j = 0;
  if (a.n_jobs > 1 && t >= a.job[1].first_tile) j = 1;
  if (a.n_jobs > 2 && t >= a.job[2].first_tile) j = 2;
  return j;
}

// accumulator columns of one K step
__host__ __device__ constexpr int slot_cols(int qt, int nc) { return qt == CMLD_Q4_K ? 4 * nc : qt == CMLD_Q6_K ? 16 * nc : 8 * nc; }

// ---------------------------------------------------------------- activation packing

// One CTA per K step: the quantised activation rows (global layout: codes | f32 scales | i16 sums of 16)
// rearranged into the records the matvec CTAs fetch with one bulk copy.  Rows past `batch` are zero.
template <int QT>
__global__ void __launch_bounds__(256) tc5_pack_kernel(const uint8_t *act, int64_t cols, int batch, int groups_total, uint8_t *pack) {
  constexpr int REC = rec_bytes(QT);
  const int ks = blockIdx.x;
  const int64_t astride = act_row_stride(cols);
  uint8_t *out = pack + (int64_t)ks * groups_total * REC;
  for (int idx = threadIdx.x; idx < groups_total * (kRecB1 / 4); idx += blockDim.x) {
    const int g = idx / (kRecB1 / 4), w = idx % (kRecB1 / 4);
    const int c = w >> 5, i = (w >> 2) & 7, x0 = (w & 3) * 4;  // chunk, row in group, first byte of the word
    const int n = g * 8 + i;
    uint32_t v = 0;
    if (n < batch) {
      const int8_t *codes = reinterpret_cast<const int8_t *>(act + n * astride) + (int64_t)ks * 256;
      if (QT == CMLD_Q6_K) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int k = 16 * c + x0 + x, l = k >> 5, p = k & 31;  // MMA l takes the values with index = l mod 8
          v |= (uint32_t)(uint8_t)codes[8 * p + l] << (8 * x);
        }
      } else {
        v = *reinterpret_cast<const uint32_t *>(codes + 16 * c + x0);
      }
    }
    *reinterpret_cast<uint32_t *>(out + (int64_t)g * REC + w * 4) = v;
  }
  for (int idx = threadIdx.x; idx < groups_total * 8; idx += blockDim.x) {
    const int g = idx >> 3, i = idx & 7, n = g * 8 + i;
    uint8_t *rec = out + (int64_t)g * REC + kRecB1;
    const uint8_t *row = act + n * astride;
    if (QT == CMLD_Q4_K) {
      // group sums of 32 codes as 64*h + l, h in -64..63, l in 0..63: [piece][chunk][i][16], bytes 0..7 of chunk 0
      const int16_t *b16 = reinterpret_cast<const int16_t *>(row + act_bsum_off(cols)) + ks * 16;
      uint32_t hw[4] = {0, 0, 0, 0}, lw[4] = {0, 0, 0, 0};
      if (n < batch) {
#pragma unroll
        for (int gq = 0; gq < 8; ++gq) {
          const int bs = (int)b16[2 * gq] + (int)b16[2 * gq + 1];
          hw[gq >> 2] |= (uint32_t)(uint8_t)(int8_t)(bs >> 6) << (8 * (gq & 3));
          lw[gq >> 2] |= (uint32_t)(bs & 63) << (8 * (gq & 3));
        }
      }
      *reinterpret_cast<uint4 *>(rec + 0 * 256 + 0 * 128 + i * 16) = make_uint4(hw[0], hw[1], 0, 0);
      *reinterpret_cast<uint4 *>(rec + 0 * 256 + 1 * 128 + i * 16) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4 *>(rec + 1 * 256 + 0 * 128 + i * 16) = make_uint4(lw[0], lw[1], 0, 0);
      *reinterpret_cast<uint4 *>(rec + 1 * 256 + 1 * 128 + i * 16) = make_uint4(0, 0, 0, 0);
      reinterpret_cast<float *>(rec + 512)[i] = n < batch ? reinterpret_cast<const float *>(row + act_scale_off(cols))[ks] : 0.0f;
    } else if (QT == CMLD_Q6_K) {
      const int8_t *codes = reinterpret_cast<const int8_t *>(row) + (int64_t)ks * 256;
      int *ys = reinterpret_cast<int *>(rec);
#pragma unroll
      for (int l = 0; l < 8; ++l) {
        int s = 0;
        if (n < batch)
          for (int p = 0; p < 32; ++p) s += codes[8 * p + l];
        ys[l * 8 + i] = s;
      }
      reinterpret_cast<float *>(rec + 256)[i] = n < batch ? reinterpret_cast<const float *>(row + act_scale_off(cols))[ks] : 0.0f;
    } else {
      float *xs = reinterpret_cast<float *>(rec);
#pragma unroll
      for (int j = 0; j < 8; ++j) xs[j * 8 + i] = n < batch ? reinterpret_cast<const float *>(row + act_scale_off(cols))[ks * 8 + j] : 0.0f;
    }
  }
}

// ---------------------------------------------------------------- weight path

// A raw stage is the plain image of the tile's superblocks of one K step: row r at r * SB bytes (SB = 144 or
// 208; both are odd multiples of 16, so lanes reading the same field of consecutive rows hit distinct banks).
// 16-byte chunk c of row r in an operand plane:
__device__ __forceinline__ uint8_t *plane_chunk(uint8_t *plane, int c, int r) { return plane + c * 2048 + (r >> 3) * 128 + (r & 7) * 16; }

__device__ __forceinline__ uint4 mul4(uint4 v, uint32_t s) { return make_uint4(v.x * s, v.y * s, v.z * s, v.w * s); }

__device__ __forceinline__ void unpack_q4k(const uint8_t *raw_stage, uint8_t *a_stage, int r, int h) {
  const uint8_t *blk = raw_stage + r * 144;
  const uint4 meta = *reinterpret_cast<const uint4 *>(blk);
  // 6-bit scales and mins as bytes (q4_k_scale_min, src/tensor/mod.rs:5997-6006)
  const uint32_t scw = h ? ((meta.w & 0x0f0f0f0fu) | ((meta.y >> 2) & 0x30303030u)) : (meta.y & 0x3f3f3f3fu);
  uint8_t *hi = a_stage, *lo = a_stage + kTcPlane;
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint4 w = *reinterpret_cast<const uint4 *>(blk + 16 + 64 * h + 16 * s);
    const int jl = s >> 1, e16 = s & 1;  // 32-byte chunk within the half, 16-byte half of the chunk
    const int g_lo = 4 * h + 2 * jl;     // low nibbles: this group; high nibbles: the next
    const uint32_t sc_lo = (scw >> (16 * jl)) & 0xffu, sc_hi = (scw >> (16 * jl + 8)) & 0xffu;
    const uint4 ql = make_uint4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu);
    const uint4 qh = make_uint4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, (w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu);
    // sc = 8*s1 + s0: bytes s1*q and s0*q stay below 106, so the four bytes of a word multiply at once
    *reinterpret_cast<uint4 *>(plane_chunk(hi, 2 * g_lo + e16, r)) = mul4(ql, sc_lo >> 3);
    *reinterpret_cast<uint4 *>(plane_chunk(lo, 2 * g_lo + e16, r)) = mul4(ql, sc_lo & 7u);
    *reinterpret_cast<uint4 *>(plane_chunk(hi, 2 * (g_lo + 1) + e16, r)) = mul4(qh, sc_hi >> 3);
    *reinterpret_cast<uint4 *>(plane_chunk(lo, 2 * (g_lo + 1) + e16, r)) = mul4(qh, sc_hi & 7u);
  }
  if (h == 0) {
    const uint32_t m03 = meta.z & 0x3f3f3f3fu, m47 = ((meta.w >> 4) & 0x0f0f0f0fu) | ((meta.z >> 2) & 0x30303030u);
    *reinterpret_cast<uint4 *>(plane_chunk(a_stage + 2 * kTcPlane, 0, r)) = make_uint4(m03, m47, 0, 0);
  }
}

// prmt in its default mode: a selector nibble with bit 3 set yields the sign of the selected byte replicated
// (0x00 for the codes here, which are below 128).  __byte_perm documents only the three low bits of a nibble.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ void unpack_q6k(const uint8_t *raw_stage, uint8_t *a_stage, int r, int h) {
  const uint8_t *blk = raw_stage + r * 208;
  uint32_t QL[16], QH[8];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint4 v = *reinterpret_cast<const uint4 *>(blk + 64 * h + 16 * s);
    QL[4 * s] = v.x, QL[4 * s + 1] = v.y, QL[4 * s + 2] = v.z, QL[4 * s + 3] = v.w;
  }
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const uint4 v = *reinterpret_cast<const uint4 *>(blk + 128 + 32 * h + 16 * s);
    QH[4 * s] = v.x, QH[4 * s + 1] = v.y, QH[4 * s + 2] = v.z, QH[4 * s + 3] = v.w;
  }
  const int8_t *scales = reinterpret_cast<const int8_t *>(blk + 192) + 8 * h;
  // The 128 values of this half are four quarters of 32; value l' of quarter qd has the 6-bit code
  // (ql[32*(qd&1) + l'] >> 4*(qd>>1)) & 15 | ((qh[l'] >> 2*qd) & 3) << 4 and the scale 2*qd + l'/16.
  // Q[qd][m] = the codes l' = 4m..4m+3 as bytes.
  uint32_t Q[4][8];
#pragma unroll
  for (int qd = 0; qd < 4; ++qd)
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const uint32_t lo4 = (QL[8 * (qd & 1) + m] >> (4 * (qd >> 1))) & 0x0f0f0f0fu;
      const uint32_t hi2 = qd < 2 ? (QH[m] << (4 - 2 * qd)) : (QH[m] >> (2 * qd - 4));
      Q[qd][m] = lo4 | (hi2 & 0x30303030u);
    }
  uint8_t *hi = a_stage, *lo = a_stage + kTcPlane;
  // Class l (index mod 8) takes from each quarter the values l' = l, 8+l, 16+l, 24+l, i.e. byte l%4 of the words
  // l/4, 2+l/4 (scale 2qd) and 4+l/4, 6+l/4 (scale 2qd+1): u = sc*q + (4096 - 32*sc) = sc*(q-32) + 4096 in two
  // 16-bit lanes per multiply-add, then the low seven bits and the rest as the two operand bytes.
#pragma unroll
  for (int l = 0; l < 8; ++l) {
    uint32_t oh[4], ol[4];
    const uint32_t sel = (uint32_t)(l & 3) | 0x80u | ((uint32_t)(4 + (l & 3)) << 8) | 0x8000u;  // [x.b, 0, y.b, 0] (codes are below 128)
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      const int sa = scales[2 * qd], sb = scales[2 * qd + 1];
      const uint32_t p01 = prmt(Q[qd][l >> 2], Q[qd][2 + (l >> 2)], sel);
      const uint32_t p23 = prmt(Q[qd][4 + (l >> 2)], Q[qd][6 + (l >> 2)], sel);
      const uint32_t u01 = p01 * (uint32_t)sa + (uint32_t)(4096 - 32 * sa) * 0x10001u;
      const uint32_t u23 = p23 * (uint32_t)sb + (uint32_t)(4096 - 32 * sb) * 0x10001u;
      ol[qd] = __byte_perm(u01, u23, 0x6420) & 0x7f7f7f7fu;
      oh[qd] = __byte_perm(u01 >> 7, u23 >> 7, 0x6420);
    }
    *reinterpret_cast<uint4 *>(plane_chunk(hi, 2 * l + h, r)) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
    *reinterpret_cast<uint4 *>(plane_chunk(lo, 2 * l + h, r)) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
  }
}

// ---------------------------------------------------------------- the kernel

// GW: groups of eight activation rows per epilogue warp group (1 or 2).
template <int QT, int GW, int EW>
__global__ void __launch_bounds__(tc_threads(EW), 1) gemv_tc5_kernel(const TcArgs a) {
  constexpr int kTcThreads = tc_threads(EW), kTcEpiWarps = EW, kTcMmaWarp = EW, kTcActWarp = EW + 1, kTcUnpackWarp0 = EW + 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int REC = rec_bytes(QT);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + a.off_bar);
  uint64_t *a_full = bars, *a_empty = bars + 4, *b_full = bars + 8, *b_empty = bars + 16, *acc_full = bars + 24, *acc_empty = bars + 26;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 28);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 29);
  const int SB = a.act_stages;
  uint8_t *a_ring = smem + a.off_a, *raw = smem + a.off_raw, *act_ring = smem + a.off_act;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NA = a.a_stages, nc = a.ng * 8;
  const int split = (int)blockIdx.x % a.n_splits, cta = (int)blockIdx.x / a.n_splits, n_ctas = (int)gridDim.x / a.n_splits;
  const int n_mine = cta < a.total_tiles ? (a.total_tiles - cta + n_ctas - 1) / n_ctas : 0;
  const int total_steps = n_mine * a.nks;
  const int scols = slot_cols(QT, nc);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < 2 * scols) tmem_cols <<= 1;

  if (tid == 0) {
    for (int i = 0; i < 4; ++i) {
      bar_init(&a_full[i], kTcUnpackThreads / 32);
      bar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < kTcMaxActStages; ++i) {
      bar_init(&b_full[i], 1);
      bar_init(&b_empty[i], kTcEpiWarps);
    }
    for (int i = 0; i < 2; ++i) {
      bar_init(&acc_full[i], 1);
      bar_init(&acc_empty[i], kTcEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (QT == CMLD_Q4_K) {
    // the mins operand: only bytes 0..7 of chunk 0 are ever written again
    for (int i = tid; i < NA * 4096 / 16; i += kTcThreads) {
      const int st = i / 256, o = i % 256;
      *reinterpret_cast<uint4 *>(a_ring + (int64_t)st * a.a_stage_bytes + 2 * kTcPlane + o * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
  }
  if (warp == kTcMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;
#pragma unroll

  if (warp >= kTcUnpackWarp0) {
    // ------------------------------------------------ weight path
    const int tu = tid - kTcUnpackWarp0 * 32, r = tu & 127, h = tu >> 7;
    constexpr int SBYTES = QT == CMLD_Q4_K ? 144 : QT == CMLD_Q6_K ? 208 : 256;  // wire bytes of a row per K step (Q8_0: codes)
    constexpr int SEG = SBYTES / 16;
    // Loads run kAhead steps before their use.  K-quants: into the raw ring (kAhead + 1 stages); Q8_0: into the
    // operand ring itself (its slot must have been read by the MMAs of kAhead + 1 steps ago).
    constexpr int kAhead = QT == CMLD_Q8_0 ? 3 : kTcRawStages - 1;
    auto row_ptr = [&](int q, int rr) -> const uint8_t * {
      const int t = cta + (q / a.nks) * n_ctas;
      const TcJob &J = a.job[tc_tile_job(a, t)];
      return J.w + (int64_t)min((t - J.first_tile) * kTcRows + rr, J.rows - 1) * J.stride;
    };
    bool ok = true;
    // The copies are spread over the 256 threads so that the lanes of a warp ask for consecutive 16-byte pieces of
    // a row (a warp instruction that touches 32 different rows costs 32 cache-line lookups).
    auto load_step = [&](int q) {
      if (q < total_steps) {
        const int ks = q % a.nks;
        if (tu < kTcRows && q + kTcPrefetchAhead < total_steps) {  // a later step's bytes into L2, one request per row
          const int qp = q + kTcPrefetchAhead;
          const uint8_t *pa = row_ptr(qp, tu) + (int64_t)(qp % a.nks) * SBYTES;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pa));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pa + SBYTES - 16));
        }
        if (QT == CMLD_Q8_0) {
          if (q >= NA) ok = ok && bar_wait(&a_empty[q % NA], (uint32_t)((q / NA - 1) & 1), abort_flag, a.status);
          if (ok) {
            // codes are int8 in K order already: straight into the operand layout.  A warp instruction covers 8 rows x
            // 4 chunks: 64 contiguous bytes per row from memory, four contiguous 128-byte pieces in shared memory.
            uint8_t *a_stage = a_ring + (int64_t)(q % NA) * a.a_stage_bytes;
            const int wu = tu >> 5, r8 = lane & 7, cc = lane >> 3;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rr = 16 * wu + 8 * (j >> 2) + r8, c = 4 * (j & 3) + cc;
              cp16(plane_chunk(a_stage, c, rr), row_ptr(q, rr) + (int64_t)ks * 256 + 16 * c);
            }
          }
        } else {
          uint8_t *dst = raw + (q % kTcRawStages) * (kTcRows * SBYTES);
#pragma unroll
          for (int j = 0; j < (kTcRows * SEG + kTcUnpackThreads - 1) / kTcUnpackThreads; ++j) {
            const int ci = tu + kTcUnpackThreads * j;
            if (ci < kTcRows * SEG) {
              const int rr = ci / SEG, sg = ci % SEG;
              cp16(dst + ci * 16, row_ptr(q, rr) + (int64_t)ks * SBYTES + 16 * sg);
            }
          }
        }
      }
      cp_commit();
    };
    for (int q = 0; q < kAhead; ++q) load_step(q);
    for (int q = 0; q < total_steps && ok; ++q) {
      uint8_t *a_stage = a_ring + (int64_t)(q % NA) * a.a_stage_bytes;
      if (QT == CMLD_Q8_0) {
        load_step(q + kAhead);
        cp_wait<kAhead>();
        if (!ok) break;
      } else {
        cp_wait<kAhead - 1>();  // this thread's pieces of step q have landed
        if (q >= NA) ok = bar_wait(&a_empty[q % NA], (uint32_t)((q / NA - 1) & 1), abort_flag, a.status);
        // One barrier per step over the 256 threads: everybody's pieces of step q are visible, everybody is done
        // reading step q-1 (whose stage the next load overwrites), and the verdict of the bounded wait is shared.
        uint32_t all_ok;
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(all_ok)
                     : "r"(ok ? 1u : 0u)
                     : "memory");
        ok = all_ok != 0;
        if (!ok) break;
        const uint8_t *raw_stage = raw + (q % kTcRawStages) * (kTcRows * SBYTES);
        if (QT == CMLD_Q4_K) unpack_q4k(raw_stage, a_stage, r, h);
        else unpack_q6k(raw_stage, a_stage, r, h);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) bar_arrive(&a_full[q % NA]);
      // the copies of a later step are asked for off the critical path (their stage, that of step q-1, is free since
      // the barrier above)
      if (QT != CMLD_Q8_0) load_step(q + kAhead);
    }
    cp_wait<0>();
  } else if (warp == kTcActWarp) {
    // ------------------------------------------------ activation records
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)(a.ng * REC);
      for (int q = 0; q < total_steps; ++q) {
        const int st = q % SB;
        if (q >= SB && !bar_wait(&b_empty[st], (uint32_t)((q / SB - 1) & 1), abort_flag, a.status)) break;
        bar_expect_tx(&b_full[st], bytes);
        const uint8_t *src = a.pack + ((int64_t)(q % a.nks) * a.groups_total + split * a.ng) * REC;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         s32(act_ring + (int64_t)st * a.act_stage_bytes)),
                     "l"(src), "r"(bytes), "r"(s32(&b_full[st]))
                     : "memory");
      }
    }
  } else if (warp == kTcMmaWarp) {
    // ------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t id_n = instr_desc(nc, true), id_p = instr_desc(16, true);
      for (int q = 0; q < total_steps; ++q) {
        const int sa = q % NA, sb = q % SB, sc = q & 1;
        if (!bar_wait(&a_full[sa], (uint32_t)((q / NA) & 1), abort_flag, a.status)) break;
        if (!bar_wait(&b_full[sb], (uint32_t)((q / SB) & 1), abort_flag, a.status)) break;
        if (q >= 2 && !bar_wait(&acc_empty[sc], (uint32_t)((q / 2 - 1) & 1), abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t a_addr = s32(a_ring + (int64_t)sa * a.a_stage_bytes), b_addr = s32(act_ring + (int64_t)sb * a.act_stage_bytes);
        const uint32_t d0 = tbase + (uint32_t)(sc * scols);
        if (QT == CMLD_Q4_K) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint64_t db = smem_desc(b_addr + g * 256, 128, REC);
            mma_i8(d0, smem_desc(a_addr + g * 4096, 2048, 128), db, id_n, g > 0);
            mma_i8(d0 + nc, smem_desc(a_addr + kTcPlane + g * 4096, 2048, 128), db, id_n, g > 0);
          }
          for (int gl = 0; gl < a.ng; ++gl)  // P: sixteen columns per group of rows, [h pieces | l pieces]
            mma_i8(d0 + 2 * nc + 16 * gl, smem_desc(a_addr + 2 * kTcPlane, 2048, 128), smem_desc(b_addr + gl * REC + kRecB1, 128, 256), id_p, false);
        } else if (QT == CMLD_Q6_K) {
#pragma unroll
          for (int l = 0; l < 8; ++l) {
            const uint64_t db = smem_desc(b_addr + l * 256, 128, REC);
            mma_i8(d0 + (2 * l) * nc, smem_desc(a_addr + l * 4096, 2048, 128), db, id_n, false);
            mma_i8(d0 + (2 * l + 1) * nc, smem_desc(a_addr + kTcPlane + l * 4096, 2048, 128), db, id_n, false);
          }
        } else {
          const uint32_t id_s = instr_desc(nc, false);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            mma_i8(d0 + j * nc, smem_desc(a_addr + j * 4096, 2048, 128), smem_desc(b_addr + j * 256, 128, REC), id_s, false);
        }
        mma_commit(&a_empty[sa]);
        mma_commit(&acc_full[sc]);
      }
    }
  } else {
    // ------------------------------------------------ epilogue
    const int wg = warp >> 2, quarter = warp & 3, r = quarter * 32 + lane;
    const int n_wg = (EW == 8 && a.ng >= 2) ? 2 : 1;   // warp groups with columns of their own
    const bool has_cols = wg < n_wg;
    const int g_first = has_cols ? wg * (a.ng / n_wg) : 0;  // first group (of eight columns) of this warp group
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    constexpr int kScaleSlot = QT == CMLD_Q8_0 ? 16 : 4;
    uint8_t *scale_ring = smem + a.off_scale;
    // One commit group per step (empty past the end), so that the group count tells which steps have landed.
    auto fetch_scales = [&](int q2) {
      if (q2 < total_steps) {
        const int t2 = cta + (q2 / a.nks) * n_ctas, ks2 = q2 % a.nks;
        const TcJob &J2 = a.job[tc_tile_job(a, t2)];
        const uint8_t *w2 = J2.w + (int64_t)min((t2 - J2.first_tile) * kTcRows + r, J2.rows - 1) * J2.stride;
        uint8_t *slot = scale_ring + ((q2 % kScaleAhead) * (kTcEpiWarps * 32) + tid) * kScaleSlot;
        if (QT == CMLD_Q4_K) cp4(slot, w2 + (int64_t)ks2 * 144);                          // f16 d, f16 dmin
        else if (QT == CMLD_Q6_K) cp4(slot, w2 + (int64_t)a.nks * 208 + 4 * (ks2 >> 1));  // the word holding f16 d of ks2
        else cp16(slot, w2 + (int64_t)a.nks * 256 + 16 * ks2);                            // eight f16 block scales
      }
      cp_commit();
    };
    for (int q2 = 0; q2 < kScaleAhead - 1; ++q2) fetch_scales(q2);
    for (int it = 0; it < n_mine; ++it) {
      const int t = cta + it * n_ctas;
      const TcJob &J = a.job[tc_tile_job(a, t)];
      const int row = (t - J.first_tile) * kTcRows + r;
      const bool row_ok = row < J.rows;
      float acc[QT == CMLD_Q6_K ? 8 : GW * 8][QT == CMLD_Q6_K ? 8 : 1];
#pragma unroll
      for (int i = 0; i < (QT == CMLD_Q6_K ? 8 : GW * 8); ++i)
#pragma unroll
        for (int l = 0; l < (QT == CMLD_Q6_K ? 8 : 1); ++l) acc[i][l] = 0.0f;
      bool ok = true;
      for (int ks = 0; ks < a.nks && ok; ++ks) {
        const int q = it * a.nks + ks, sc = q & 1, sb = q % SB;
        // the row's own scales of this step: asked for kScaleAhead steps ago, in this thread's private slot
        cp_wait<kScaleAhead - 2>();
        float dw = 0.0f, dmw = 0.0f;
        uint4 ws8 = make_uint4(0, 0, 0, 0);
        {
          const uint8_t *slot = scale_ring + ((q % kScaleAhead) * (kTcEpiWarps * 32) + tid) * kScaleSlot;
          if (QT == CMLD_Q4_K) {
            const uint32_t m = *reinterpret_cast<const uint32_t *>(slot);
            dw = f16_bits_to_f32((uint16_t)(m & 0xffff));
            dmw = f16_bits_to_f32((uint16_t)(m >> 16));
          } else if (QT == CMLD_Q6_K) {
            const uint32_t m = *reinterpret_cast<const uint32_t *>(slot);
            dw = f16_bits_to_f32((uint16_t)((m >> (16 * (ks & 1))) & 0xffff));
          } else {
            ws8 = *reinterpret_cast<const uint4 *>(slot);
          }
        }
        ok = bar_wait(&acc_full[sc], (uint32_t)((q / 2) & 1), abort_flag, a.status);
        // the record's bytes arrive through the async proxy: each reader observes the copy's own barrier (its phase
        // completed before the step's MMAs were issued, and is not re-armed before this warp gives the stage back)
        ok = ok && bar_wait(&b_full[sb], (uint32_t)((q / SB) & 1), abort_flag, a.status);
        // The lanes leave the polling loops at different iterations; tcgen05.ld is a .sync.aligned instruction and
        // must be executed by the whole warp together, so the warp is brought back together here (a diverged warp
        // returned wrong values in the last registers of a load now and then).
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d0 = tbase + lane_base + (uint32_t)(sc * scols);
        const uint8_t *recs = act_ring + (int64_t)sb * a.act_stage_bytes;
        if (QT == CMLD_Q4_K) {
          int S[GW * 8], P[GW * 8];
          float xd[GW * 8];
#pragma unroll
          for (int gi = 0; gi < GW; ++gi) {
            const int g = g_first + gi;
            int s1[8], s0[8], ph[8], pl[8];
            if (has_cols) {
              tmem_ld8x4(d0 + g * 8, s1, d0 + nc + g * 8, s0, d0 + 2 * nc + 16 * g, ph, d0 + 2 * nc + 16 * g + 8, pl);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                S[gi * 8 + i] = 8 * s1[i] + s0[i];
                P[gi * 8 + i] = 64 * ph[i] + pl[i];
                xd[gi * 8 + i] = reinterpret_cast<const float *>(recs + g * REC + kRecB1 + 512)[i];
              }
            }
          }
          if (has_cols) {
#pragma unroll
            for (int i = 0; i < GW * 8; ++i) {
              // sumf = fma(-dmin, P, sumf); sumf = fma(d, S, sumf) with d = xd*dw, dmin = xd*dminw (refmath.rs:529, :560)
              acc[i][0] = __fmaf_rn(-__fmul_rn(xd[i], dmw), (float)P[i], acc[i][0]);
              acc[i][0] = __fmaf_rn(__fmul_rn(xd[i], dw), (float)S[i], acc[i][0]);
            }
          }
          release_step(&acc_empty[sc], &b_empty[sb], lane);
          fetch_scales(q + kScaleAhead - 1);  // off the critical path
        } else if (QT == CMLD_Q6_K) {
          const int g = g_first;
          if (has_cols) {
            const int *ys = reinterpret_cast<const int *>(recs + g * REC + kRecB1);
            float dd[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) dd[i] = __fmul_rn(dw, reinterpret_cast<const float *>(recs + g * REC + kRecB1 + 256)[i]);  // src/inference.rs:25545
#pragma unroll
            for (int l = 0; l < 8; l += 2) {
              int dh[8], dl[8], eh[8], el[8];
              tmem_ld8x4(d0 + (2 * l) * nc + g * 8, dh, d0 + (2 * l + 1) * nc + g * 8, dl, d0 + (2 * l + 2) * nc + g * 8, eh,
                         d0 + (2 * l + 3) * nc + g * 8, el);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                // sums[l] += (d*xd) * (float)aux[l], each of the eight lanes on its own (independent chains)
                acc[i][l] = __fadd_rn(acc[i][l], __fmul_rn(dd[i], (float)(128 * dh[i] + dl[i] - 4096 * ys[l * 8 + i])));
                acc[i][l + 1] = __fadd_rn(acc[i][l + 1], __fmul_rn(dd[i], (float)(128 * eh[i] + el[i] - 4096 * ys[(l + 1) * 8 + i])));
              }
            }
          }
          release_step(&acc_empty[sc], &b_empty[sb], lane);
          fetch_scales(q + kScaleAhead - 1);  // off the critical path
        } else {
          const uint32_t wsw[4] = {ws8.x, ws8.y, ws8.z, ws8.w};
#pragma unroll
          for (int gi = 0; gi < GW; ++gi) {
            const int g = g_first + gi;
            if (has_cols) {
              const float *xs = reinterpret_cast<const float *>(recs + g * REC + kRecB1);
              // all eight blocks of the step are read before the slot is given back only for the last group
#pragma unroll
              for (int j0 = 0; j0 < 8; j0 += 4) {
                int isum[4][8];
                tmem_ld8x4(d0 + j0 * nc + g * 8, isum[0], d0 + (j0 + 1) * nc + g * 8, isum[1], d0 + (j0 + 2) * nc + g * 8, isum[2],
                           d0 + (j0 + 3) * nc + g * 8, isum[3]);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                  const int j = j0 + jj;
                  const float ws = f16_bits_to_f32((uint16_t)((wsw[j >> 1] >> (16 * (j & 1))) & 0xffff));
#pragma unroll
                  for (int i = 0; i < 8; ++i)  // src/inference.rs:26198
                    acc[gi * 8 + i][0] = __fadd_rn(acc[gi * 8 + i][0], __fmul_rn(__fmul_rn((float)isum[jj][i], ws), xs[j * 8 + i]));
                }
              }
            }
          }
          release_step(&acc_empty[sc], &b_empty[sb], lane);
          fetch_scales(q + kScaleAhead - 1);  // off the critical path
        }
      }
      if (!ok) break;
      if (has_cols && row_ok) {
#pragma unroll
        for (int i = 0; i < (QT == CMLD_Q6_K ? 8 : GW * 8); ++i) {
          const int b = (split * a.ng + g_first) * 8 + i;
          if (b < a.batch) {
            float res = acc[i][0];
            if (QT == CMLD_Q6_K) {
              res = 0.0f;  // 0 + sums[0] + ... + sums[7] (src/inference.rs:25578-25580)
#pragma unroll
              for (int l = 0; l < 8; ++l) res = __fadd_rn(res, acc[i][l]);
            }
            const int64_t o = (int64_t)b * J.y_stride + row;
            J.y[o] = J.residual ? __fadd_rn(__ldcg(J.residual + o), res) : res;
          }
        }
      }
    }
  }
  cp_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == kTcMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(tmem_cols) : "memory");
  }
}

int g_tc_sms = 0;

struct TcPlan {
  TcArgs args;
  int grid, smem, gw;
};

}  // namespace

static bool tc5_qt_ok(int qt) { return qt == CMLD_Q4_K || qt == CMLD_Q6_K || qt == CMLD_Q8_0; }

// Bytes of packed activation records one matrix type needs for `cols` columns and up to 32 rows.
int64_t gemv_tc5_pack_bytes(int64_t cols) { return cols / 256 * 4 * (int64_t)kRecQ4; }

bool gemv_tc5_fits(const GemvJob *jobs, int n_jobs, int32_t batch) {
  if (n_jobs < 1 || n_jobs > 3 || batch < 1 || batch > 32) return false;
  for (int i = 0; i < n_jobs; ++i) {
    if (!tc5_qt_ok(jobs[i].qt) || jobs[i].cols != jobs[0].cols || jobs[i].cols % 256 != 0 || jobs[i].cols < 256 || jobs[i].rows < 1) return false;
  }
  return true;
}

template <int QT, int GW, int EW>
static int32_t launch_tc(const TcPlan &p, cudaStream_t s) {
  static bool attr = false;
  if (!attr) {
    CMLD_CUDA(cudaFuncSetAttribute(gemv_tc5_kernel<QT, GW, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr = true;
  }
  gemv_tc5_kernel<QT, GW, EW><<<p.grid, tc_threads(EW), p.smem, s>>>(p.args);
  CMLD_CUDA(cudaGetLastError());
  return CMLD_OK;
}

// Matrices of ONE type.  `pack`: room for gemv_tc5_pack_bytes(cols).
static int32_t launch_tc5_qt(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, uint8_t *pack, int32_t *status,
                             cudaStream_t s, int64_t *launches) {
  const int qt = jobs[0].qt;
  const int64_t cols = jobs[0].cols;
  TcPlan p{};
  TcArgs &a = p.args;
  a.n_jobs = n_jobs;
  int tiles = 0;
  for (int i = 0; i < n_jobs; ++i) {
    TcJob &J = a.job[i];
    J.w = jobs[i].w;
    J.rows = (int32_t)jobs[i].rows;
    J.stride = jobs[i].stride;
    J.y = jobs[i].y;
    J.residual = jobs[i].residual;
    J.y_stride = jobs[i].y_stride;
    J.first_tile = tiles;
    J.n_tiles = (int32_t)((jobs[i].rows + kTcRows - 1) / kTcRows);
    tiles += J.n_tiles;
  }
  a.total_tiles = tiles;
  a.nks = (int32_t)(cols / 256);
  a.batch = batch;
  a.groups_total = batch <= 8 ? 1 : batch <= 16 ? 2 : 4;
  // columns per CTA: as many as the type allows, fewer (more CTAs per tile) while SMs would stay idle
  const int ng_max = qt == CMLD_Q6_K ? 2 : 4;
  int ng = std::min(a.groups_total, ng_max);
  while (ng > 1 && tiles * (a.groups_total / (ng / 2)) <= g_tc_sms) ng /= 2;
  // Q6_K keeps 64 f32 sums and 64 integers of a step per epilogue thread: with eight columns per CTA one warp group of
  // epilogue threads is enough, and the 448-thread form of the kernel gives each thread 144 registers instead of 96
  // (no spills).  Taken whenever the launch stays within one wave of CTAs.
  if (qt == CMLD_Q6_K && ng == 2 && tiles * a.groups_total <= g_tc_sms) ng = 1;
  const int ew = ng == 1 ? 4 : 8;
  a.ng = ng;
  a.n_splits = a.groups_total / ng;
  a.a_stages = qt == CMLD_Q8_0 ? 4 : 2;
  a.a_stage_bytes = qt == CMLD_Q4_K ? 2 * kTcPlane + 4096 : qt == CMLD_Q6_K ? 2 * kTcPlane : kTcPlane;
  a.act_stage_bytes = ng * rec_bytes(qt);
  a.off_a = 0;
  a.off_raw = a.off_a + a.a_stages * a.a_stage_bytes;
  const int raw_bytes = qt == CMLD_Q4_K ? kTcRawStages * kTcRows * 144 : qt == CMLD_Q6_K ? kTcRawStages * kTcRows * 208 : 0;
  a.off_act = a.off_raw + raw_bytes;
  // as many activation stages as fit (the copy of a record starts when the epilogue has given its stage back and
  // takes about a microsecond: the ring must cover that)
  const int scale_bytes = kScaleAhead * ew * 32 * (qt == CMLD_Q8_0 ? 16 : 4);
  a.act_stages = std::min<int>(kTcMaxActStages, (227 * 1024 - 256 - scale_bytes - a.off_act) / a.act_stage_bytes);
  if (a.act_stages < 2) return CMLD_ERR_UNSUPPORTED;
  a.off_scale = (a.off_act + a.act_stages * a.act_stage_bytes + 15) & ~15;
  a.off_bar = a.off_scale + scale_bytes;
  p.smem = a.off_bar + 256;
  if (p.smem > 227 * 1024) return CMLD_ERR_UNSUPPORTED;
  a.pack = pack;
  a.status = status;
  const int ctas_per_split = std::max(1, std::min(tiles, g_tc_sms / a.n_splits));
  p.grid = ctas_per_split * a.n_splits;
  p.gw = ng == 4 ? 2 : 1;
  // pack the activation rows for this type
  switch (qt) {
    case CMLD_Q4_K: tc5_pack_kernel<CMLD_Q4_K><<<a.nks, 256, 0, s>>>(act, cols, batch, a.groups_total, pack); break;
    case CMLD_Q6_K: tc5_pack_kernel<CMLD_Q6_K><<<a.nks, 256, 0, s>>>(act, cols, batch, a.groups_total, pack); break;
    default: tc5_pack_kernel<CMLD_Q8_0><<<a.nks, 256, 0, s>>>(act, cols, batch, a.groups_total, pack); break;
  }
  CMLD_CUDA(cudaGetLastError());
  int32_t rc;
  if (qt == CMLD_Q4_K) rc = p.gw == 2 ? launch_tc<CMLD_Q4_K, 2, 8>(p, s) : ew == 4 ? launch_tc<CMLD_Q4_K, 1, 4>(p, s) : launch_tc<CMLD_Q4_K, 1, 8>(p, s);
  else if (qt == CMLD_Q6_K) rc = ew == 4 ? launch_tc<CMLD_Q6_K, 1, 4>(p, s) : launch_tc<CMLD_Q6_K, 1, 8>(p, s);
  else rc = p.gw == 2 ? launch_tc<CMLD_Q8_0, 2, 8>(p, s) : ew == 4 ? launch_tc<CMLD_Q8_0, 1, 4>(p, s) : launch_tc<CMLD_Q8_0, 1, 8>(p, s);
  CMLD_TRY(rc);
  if (launches) *launches += 2;
  return CMLD_OK;
}

// `act`: the quantised activation rows in the global layout (Q8_0 rows for Q8_0 matrices, Q8_K rows
// otherwise).  `pack`: scratch of gemv_tc5_pack_bytes(cols) bytes, overwritten by every call.  Matrices of
// different types are served by one launch per type.  CMLD_ERR_UNSUPPORTED (no message) when the shapes do
// not fit.
int32_t launch_gemv_tc5(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, uint8_t *pack, int64_t pack_bytes,
                        int32_t *status, cudaStream_t s, int64_t *launches) {
  if (!gemv_tc5_fits(jobs, n_jobs, batch)) return CMLD_ERR_UNSUPPORTED;
  if (!act || !pack || pack_bytes < gemv_tc5_pack_bytes(jobs[0].cols)) return CMLD_ERR_UNSUPPORTED;
  if (g_tc_sms == 0) {
    int dev = 0;
    CMLD_CUDA(cudaGetDevice(&dev));
    CMLD_CUDA(cudaDeviceGetAttribute(&g_tc_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  bool done[3] = {false, false, false};
  for (int i = 0; i < n_jobs; ++i) {
    if (done[i]) continue;
    GemvJob same[3];
    int n = 0;
    for (int k = i; k < n_jobs; ++k)
      if (!done[k] && jobs[k].qt == jobs[i].qt) {
        same[n++] = jobs[k];
        done[k] = true;
      }
    CMLD_TRY(launch_tc5_qt(same, n, act, batch, pack, status, s, launches));
  }
  return CMLD_OK;
}

}  // namespace cmld
