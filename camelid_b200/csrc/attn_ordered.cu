// Single-query grouped-query attention over the f16 KV cache with every f32 operation in the order of
// Camelid's CPU path (attention_context_for_head_into_with_kernels, src/inference.rs:30287-30466 with
// dot_product, src/tensor/mod.rs:3464-3480, in the Camelid tree), so the output has the CPU's bits:
//
//   score_p = (((0 + q0*k0) + q1*k1) + ...) * scale          one accumulator over the head dimension
//   m = max_p score_p;  e_p = expf(score_p - m);  S = ((e_0 + e_1) + ...)   one accumulator over positions
//   out_d = ((0 + (e_0/S)*v_0d) + (e_1/S)*v_1d) + ...        one accumulator over positions, per d
//
// The dependent chains are what they are — 4 cycles per addition — so the kernel is organised around
// having as many of them in flight as the arithmetic allows and nothing else on the critical path:
//   * one thread-block cluster of 8 CTAs per (sequence, kv head), serving the G query heads of the group;
//   * scores: positions are cut into 8 ranges, one per CTA; a thread owns one (position, head) chain over the
//     head dimension; K rows are staged by cp.async into shared memory at a bank-conflict-free pitch;
//   * softmax: range maxima meet through distributed shared memory; e_p is written straight into the
//     shared memory of the CTAs that need it; the sum over positions is a sequential f32 sum of non-negative
//     terms, computed with its exact bits by all warps of one CTA per head (exact_sum.cuh);
//   * output: CTA r of the cluster owns dims [r*hd/8, (r+1)*hd/8) of ALL G heads (G*hd/8 chains), so a V element
//     it loads serves G chains and the V bytes a CTA needs are 1/8 of the rows.  V is copied by cp.async into
//     shared memory from the moment the kernel starts, so it arrives while the scores are still being computed.
//     Contexts of up to 2048 positions keep the CTA's whole V slice there and a chain lane forms its own products
//     (e_p/S)*v_pd; longer contexts stream V through a ring: producer warps form the products into
//     double-buffered shared memory and a chain warp walks 32 chains with one 16-byte load per four additions.
// RoPE of q and k and the f16 KV append can be folded in (fuse_rope), as in the split-range kernel.
#include <cooperative_groups.h>

#include "common.cuh"
#include "exact_sum.cuh"
#include "expf_exact.cuh"

namespace cmld {

namespace cg = cooperative_groups;

constexpr int kOaThreads = 512;
constexpr int kOaWarps = kOaThreads / 32;
constexpr int kOaCluster = 8;
constexpr int kOaKBlock = 128;  // positions per staged K block (at most)
constexpr int kOaBatch = 64;    // positions per product buffer
// V ring slots per producer warp (one slot per batch of 64 positions): as many as shared memory allows, so that for
// contexts of up to 2048 positions every V byte is requested when the kernel starts
__host__ __device__ constexpr int oa_vdepth(int64_t cap) { return cap <= 2048 ? 32 : (cap <= 4096 ? 16 : 8); }

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// RoPE pair partner and sign: x'[d] = x[d]*c + sgn * x[partner]*s  (src/inference/rope.rs:495-530)
__device__ __forceinline__ float oa_rope_elem(const float *x, int d, int rope_dim, int split_half, const float *ct, const float *st) {
  if (d >= rope_dim) return x[d];
  const int half = rope_dim >> 1;
  int p, partner;
  bool first;
  if (split_half) {
    first = d < half;
    p = first ? d : d - half;
    partner = first ? d + half : d - half;
  } else {
    first = (d & 1) == 0;
    p = d >> 1;
    partner = first ? d + 1 : d - 1;
  }
  const float c = ct[p], sn = st[p];
  return first ? __fsub_rn(__fmul_rn(x[d], c), __fmul_rn(x[partner], sn)) : __fadd_rn(__fmul_rn(x[partner], sn), __fmul_rn(x[d], c));
}

__device__ __forceinline__ void cp_async4(void *dst_smem, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

// One output chain over a V slice that is wholly in shared memory as [dim pair][position] half2 words (va: the
// pair's row; PAR: which half is this chain's dim) with the weights of its head at wa: out = ((0 + w_0*v_0) +
// w_1*v_1) + ...  Eight positions per trip: four 16-byte loads, issued one trip ahead of the eight dependent
// additions they feed, so the chain runs at the pace the warp can issue its ~3.5 instructions per position.
template <int PAR>
__device__ __forceinline__ float oa_resident_chain(uint32_t va, uint32_t wa, int n_pre) {
  float o = 0.0f;
#define OR_CV(X) (PAR ? __high2float(*reinterpret_cast<const __half2 *>(&(X))) : __low2float(*reinterpret_cast<const __half2 *>(&(X))))
#define OR_LOAD(U, V0, V1, W0, W1)                                                                                            \
  do {                                                                                                                        \
    const uint32_t off_ = (uint32_t)(U) * 32u;                                                                                \
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(V0.x), "=r"(V0.y), "=r"(V0.z), "=r"(V0.w) : "r"(va + off_));        \
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(V1.x), "=r"(V1.y), "=r"(V1.z), "=r"(V1.w) : "r"(va + off_ + 16u));  \
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(W0.x), "=f"(W0.y), "=f"(W0.z), "=f"(W0.w) : "r"(wa + off_));        \
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(W1.x), "=f"(W1.y), "=f"(W1.z), "=f"(W1.w) : "r"(wa + off_ + 16u));  \
  } while (0)
#define OR_ADD(V0, V1, W0, W1)                          \
  do {                                                  \
    o = __fadd_rn(o, __fmul_rn(W0.x, OR_CV(V0.x)));     \
    o = __fadd_rn(o, __fmul_rn(W0.y, OR_CV(V0.y)));     \
    o = __fadd_rn(o, __fmul_rn(W0.z, OR_CV(V0.z)));     \
    o = __fadd_rn(o, __fmul_rn(W0.w, OR_CV(V0.w)));     \
    o = __fadd_rn(o, __fmul_rn(W1.x, OR_CV(V1.x)));     \
    o = __fadd_rn(o, __fmul_rn(W1.y, OR_CV(V1.y)));     \
    o = __fadd_rn(o, __fmul_rn(W1.z, OR_CV(V1.z)));     \
    o = __fadd_rn(o, __fmul_rn(W1.w, OR_CV(V1.w)));     \
  } while (0)
  const int nu = n_pre >> 3;  // whole units of eight positions
  if (nu > 0) {
    uint4 A0, A1, B0, B1;
    float4 WA0, WA1, WB0, WB1;
    OR_LOAD(0, A0, A1, WA0, WA1);
    int u = 0;
    for (; u + 2 < nu; u += 2) {
      OR_LOAD(u + 1, B0, B1, WB0, WB1);
      OR_ADD(A0, A1, WA0, WA1);
      OR_LOAD(u + 2, A0, A1, WA0, WA1);
      OR_ADD(B0, B1, WB0, WB1);
    }
    if (u + 1 < nu) {
      OR_LOAD(u + 1, B0, B1, WB0, WB1);
      OR_ADD(A0, A1, WA0, WA1);
      OR_ADD(B0, B1, WB0, WB1);
    } else {
      OR_ADD(A0, A1, WA0, WA1);
    }
  }
  for (int p = nu * 8; p < n_pre; ++p) {
    uint32_t vw;
    float w;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(vw) : "r"(va + 4u * p));
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(w) : "r"(wa + 4u * p));
    o = __fadd_rn(o, __fmul_rn(w, OR_CV(vw)));
  }
#undef OR_CV
#undef OR_LOAD
#undef OR_ADD
  return o;
}

struct OaLayout {
  int cap_range;   // positions a CTA's range can hold
  int cap_pad;     // positions per weight array (multiple of 256)
  int off_q, off_sc, off_a, off_prod, off_ws, off_mx, off_inv, off_klast, off_v, total;
};

// Shared-memory map.  Region A holds the K staging buffers while the scores are computed and, after that, the
// softmax weights of all G heads (written by the whole cluster once nobody scores any more).
__host__ __device__ inline OaLayout oa_layout(int G, int HD, int64_t cap) {
  OaLayout L;
  const int dpc = HD / kOaCluster;
  L.cap_range = (int)((cap + kOaCluster - 1) / kOaCluster);
  L.cap_pad = (int)((cap + 255) / 256 * 256);
  int off = 0;
  L.off_q = off;
  off += G * HD * 4;
  L.off_sc = off;
  off += G * L.cap_range * 4;
  off = (off + 15) & ~15;
  L.off_a = off;
  {
    const int kbytes = 2 * kOaKBlock * (HD * 2 + 16), wbytes = G * L.cap_pad * 4;
    off += kbytes > wbytes ? kbytes : wbytes;
  }
  const bool resident = oa_vdepth(cap) == 32;  // the CTA's whole V slice stays in shared memory: no product buffers
  L.off_prod = off;
  if (!resident) off += 2 * (kOaBatch / 4) * (G * dpc * 4 + 4) * 4;  // products: [buffer][4 positions][chain][position in the four] + 4 floats of padding
  L.off_ws = off;
  off += xsum::workspace_bytes(L.cap_pad);
  off = (off + 15) & ~15;
  L.off_mx = off;
  off += kOaCluster * 8 * 4;
  L.off_inv = off;
  off += 48;
  L.off_klast = off;
  off += HD * 2;
  off = (off + 127) & ~127;
  L.off_v = off;
  if (resident) off += (dpc / 2) * (L.cap_pad * 4 + 16);  // [dim pair][position] half2 words; the row pitch keeps 16-byte loads of eight rows on distinct banks
  else off += (2 * (dpc / 8)) * oa_vdepth(cap) * 512;     // producer warps x slots x (32 lanes x 16 bytes)
  L.total = off;
  return L;
}

template <int G, int HD, int VD>
__global__ void __launch_bounds__(kOaThreads, 1) attn_ordered_kernel(AttnArgs a, int64_t cap) {
  asm volatile("griddepcontrol.launch_dependents;");
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int DPC = HD / kOaCluster;       // dims of every head this CTA owns in the output phase
  constexpr int CPC = G * DPC;               // its chains: (head g, dim dd) -> g * DPC + dd
  constexpr int NP = DPC / 8;                // 16-byte pieces of a V row it needs
  constexpr int NCW = (CPC + 31) / 32;       // warps that walk chains
  constexpr int NPW = 2 * NP;                // producer warps: each takes 32/NP positions of every 64-position batch
  constexpr int PPB = 32 / NP;               // positions per producer warp and batch
  constexpr int QP = CPC * 4 + 4;            // floats per group of four positions: [chain][position in the group], padded so that
                                             // the producers' scalar stores (neighbouring positions) spread over the banks
  constexpr int KP = HD * 2 + 16;            // K row pitch in shared memory
  static_assert(DPC % 8 == 0 && NPW >= 1 && NPW + NCW <= kOaWarps, "shape not supported");
  const OaLayout L = oa_layout(G, HD, cap);
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = a.positions[b];
  const int n_pos = pos + 1;
  const int slot = a.slots[b];
  if (pos < 0 || pos >= a.max_pos || n_pos > cap) return;  // the same for every CTA of the cluster
  float(*s_q)[HD] = reinterpret_cast<float(*)[HD]>(smem + L.off_q);
  float *s_sc = reinterpret_cast<float *>(smem + L.off_sc);   // [G][cap_range]
  uint8_t *s_k = smem + L.off_a;                              // K staging ...
  float *s_w = reinterpret_cast<float *>(smem + L.off_a);     // ... then [G][cap_pad] weights
  float *s_prod = reinterpret_cast<float *>(smem + L.off_prod);  // [2][kOaBatch / 4][QP]
  uint8_t *s_ws = smem + L.off_ws;
  float *s_mx = reinterpret_cast<float *>(smem + L.off_mx);   // [cluster rank][8]
  float *s_inv = reinterpret_cast<float *>(smem + L.off_inv); // [8]
  __half *s_klast = reinterpret_cast<__half *>(smem + L.off_klast);
  uint8_t *s_v = smem + L.off_v;                              // [producer warp][VD][32 lanes x 16 bytes]

  unsigned long long *ph = (a.phase_ns && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0) ? a.phase_ns : nullptr;
  if (ph) ph[0] = global_ns();
  __half *kbase = const_cast<__half *>(a.k_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  __half *vbase = const_cast<__half *>(a.v_cache) + ((int64_t)slot * a.n_kv_heads + kvh) * a.max_pos * HD;
  const int n_pre = a.fuse_rope ? n_pos - 1 : n_pos;  // positions whose K/V rows are already in the cache
  const int d0 = crank * DPC;                         // this CTA's first dim

  // ---- V rings of the producer warps (the last NPW warps).  Producer warp j owns positions [j*PPB, (j+1)*PPB) of
  // every 64-position batch; a lane copies one 16-byte piece (8 dims of one position), and later multiplies the
  // very bytes it copied itself, so the producers never wait for each other.
  const int pw = warp - (kOaWarps - NPW);  // producer index, < 0 for the other warps
  const int n_batches = (n_pre + kOaBatch - 1) / kOaBatch;
  const int v_pp = lane % PPB, v_k = lane / PPB;  // this lane's position within the warp's block, and piece
  uint8_t *vring = s_v + (pw < 0 ? 0 : pw) * VD * 512;
  auto issue_v = [&](int bt) {
    if (bt < n_batches) {
      const int p = bt * kOaBatch + pw * PPB + v_pp;
      if (p < n_pre) cp_async16(vring + (bt % VD) * 512 + lane * 16, vbase + (int64_t)p * HD + d0 + 8 * v_k);
    }
    cp_async_commit();
  };
  // Contexts of up to 2048 positions (VD == 32): every thread copies 4-byte pieces (two dims of one position) straight
  // into the [dim pair][position] layout the chain lanes read, as one group.
  constexpr bool kResident = VD == 32;
  constexpr int HP = DPC / 2;
  const int vt_pitch = L.cap_pad * 4 + 16;
  auto issue_v_resident = [&]() {
    for (int idx = tid; idx < n_pre * HP; idx += kOaThreads) {
      const int p = idx / HP, j = idx % HP;
      cp_async4(s_v + j * vt_pitch + p * 4, vbase + (int64_t)p * HD + d0 + 2 * j);
    }
    cp_async_commit();
  };
  // ranges: CTA r scores positions [r*len, (r+1)*len), in n_blocks blocks of bsz positions
  const int len = (n_pos + kOaCluster - 1) / kOaCluster;
  const int lo = crank * len, hi = min(n_pos, lo + len);
  // contexts of up to 2048 positions: a CTA's range (at most 256 positions) is one block filling both staging
  // buffers — one wait and one pass instead of two; longer contexts: blocks of up to 128, double-buffered
  const int kblk = kResident ? 2 * kOaKBlock : kOaKBlock;
  const int n_blocks = hi > lo ? (hi - lo + kblk - 1) / kblk : 0;
  const int bsz = n_blocks > 0 ? (hi - lo + n_blocks - 1) / n_blocks : 0;
  auto issue_k = [&](int blk) {
    if (blk < n_blocks) {
      uint8_t *dst = s_k + (blk & 1) * kOaKBlock * KP;
      for (int i = tid; i < bsz * (HD / 8); i += kOaThreads) {
        const int pp = i / (HD / 8), gdx = i % (HD / 8), p = lo + blk * bsz + pp;
        if (p < hi && p < n_pre) cp_async16(dst + pp * KP + gdx * 16, kbase + (int64_t)p * HD + gdx * 8);
      }
    }
    cp_async_commit();
  };
  // With the KV append folded in, every row this kernel prefetches was written by an earlier step: the loads
  // can start before the kernel waits for its predecessor (which produces q and the new k / v rows).
  if (a.fuse_rope) {
    issue_k(0);
    issue_k(1);
    if (kResident) issue_v_resident();
    else if (pw >= 0)
      for (int c = 0; c < VD; ++c) issue_v(c);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (!a.fuse_rope) {
    issue_k(0);
    issue_k(1);
    if (kResident) issue_v_resident();
    else if (pw >= 0)
      for (int c = 0; c < VD; ++c) issue_v(c);
  }

  // ---- q (rotated), and the row's own K/V: appended to the cache, K kept for the scores
  const float *q = a.q + (int64_t)b * a.q_stride + (int64_t)kvh * G * HD;
  if (a.fuse_rope) {
    const int half = a.rope_dim >> 1;
    const float *ct = a.cos_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    const float *st = a.sin_tab + (int64_t)(a.index_by_position ? pos : b) * half;
    for (int i = tid; i < G * HD; i += kOaThreads) s_q[i / HD][i % HD] = oa_rope_elem(q + (i / HD) * HD, i % HD, a.rope_dim, a.split_half, ct, st);
    if (pos >= lo && pos < hi) {
      const float *kn = a.k_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      const float *vn = a.v_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD;
      for (int d = tid; d < HD; d += kOaThreads) {
        const __half kh = __float2half_rn(oa_rope_elem(kn, d, a.rope_dim, a.split_half, ct, st));
        s_klast[d] = kh;
        kbase[(int64_t)pos * HD + d] = kh;
        vbase[(int64_t)pos * HD + d] = __float2half_rn(vn[d]);
      }
    }
  } else {
    for (int i = tid; i < G * HD; i += kOaThreads) s_q[i / HD][i % HD] = q[i];
  }

  // ---- scores of this CTA's range, K staged block by block; a thread owns one (position, head) chain
  for (int blk = 0; blk < n_blocks; ++blk) {
    // groups in flight, oldest first: K block blk, K block blk+1, then (producer warps) the V ring's first VD slots
    // or, from the second pass on, nothing younger: wait until block blk has landed
    // (resident form: K block 0, K block 1, the V group, then one K group per pass)
    if (kResident && blk < 2) cp_async_wait<2>();
    else if (!kResident && blk == 0 && pw >= 0) cp_async_wait<VD + 1>();
    else cp_async_wait<1>();
    __syncthreads();  // block blk has landed for everyone (the first pass also publishes s_q and s_klast)
    const uint8_t *kb = s_k + (blk & 1) * kOaKBlock * KP;
    for (int pair = tid; pair < bsz * G; pair += kOaThreads) {
      const int pp = pair % bsz, g = pair / bsz, p = lo + blk * bsz + pp;
      if (p < hi) {
        const uint4 *kr = p < n_pre ? reinterpret_cast<const uint4 *>(kb + pp * KP) : reinterpret_cast<const uint4 *>(s_klast);
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
          const uint4 raw = kr[j];
          const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
          const float4 qa = *reinterpret_cast<const float4 *>(&s_q[g][8 * j]), qb = *reinterpret_cast<const float4 *>(&s_q[g][8 * j + 4]);
          const float2 k0 = __half22float2(h2[0]), k1 = __half22float2(h2[1]), k2 = __half22float2(h2[2]), k3 = __half22float2(h2[3]);
          s = __fadd_rn(s, __fmul_rn(qa.x, k0.x));
          s = __fadd_rn(s, __fmul_rn(qa.y, k0.y));
          s = __fadd_rn(s, __fmul_rn(qa.z, k1.x));
          s = __fadd_rn(s, __fmul_rn(qa.w, k1.y));
          s = __fadd_rn(s, __fmul_rn(qb.x, k2.x));
          s = __fadd_rn(s, __fmul_rn(qb.y, k2.y));
          s = __fadd_rn(s, __fmul_rn(qb.z, k3.x));
          s = __fadd_rn(s, __fmul_rn(qb.w, k3.y));
        }
        s_sc[g * L.cap_range + (p - lo)] = __fmul_rn(s, a.scale);
      }
    }
    __syncthreads();  // everyone is done with the buffer
    issue_k(blk + 2);
  }
  if (n_blocks == 0) __syncthreads();
  cp_async_wait<0>();
  if (ph) ph[1] = global_ns();  // scores done

  // ---- range maxima to every CTA
  if (warp < G) {
    float m = -INFINITY;
    for (int i = lane; i < hi - lo; i += 32) m = fmaxf(m, s_sc[warp * L.cap_range + i]);
    m = warp_max(m);
    if (lane < kOaCluster) cluster.map_shared_rank(s_mx, lane)[crank * 8 + warp] = m;
  }
  cluster.sync();  // also: nobody reads its K staging area any more, so the weights may now be written over it
  if (ph) ph[2] = global_ns();  // maxima exchanged
  // ---- e_p = expf(score - max) into every CTA of the cluster (each needs all heads' weights for its chains)
  for (int i = tid; i < G * (hi - lo); i += kOaThreads) {
    const int g = i / (hi - lo), pi = i % (hi - lo);
    float m = -INFINITY;
#pragma unroll
    for (int r = 0; r < kOaCluster; ++r) m = fmaxf(m, s_mx[r * 8 + g]);
    const float e = expf_exact(__fsub_rn(s_sc[g * L.cap_range + pi], m));
#pragma unroll
    for (int r = 0; r < kOaCluster; ++r) cluster.map_shared_rank(s_w, r)[g * L.cap_pad + lo + pi] = e;
  }
  cluster.sync();
  if (ph) ph[3] = global_ns();  // weights delivered
  // ---- S = e_0 + e_1 + ... in order: head g by CTA g; 1/S to all
  if (crank < G) {
    float *w = s_w + crank * L.cap_pad;
    const int n_pad = (n_pos + 255) & ~255;
    for (int i = n_pos + tid; i < n_pad; i += kOaThreads) w[i] = 0.0f;  // adding +0 leaves a sum as it is
    const float ssum = xsum::cta_sum<kOaWarps>(w, n_pad, warp, lane, 1, s_ws);
    if (tid < kOaCluster) cluster.map_shared_rank(s_inv, tid)[crank] = __fdiv_rn(1.0f, ssum);
  }
  cluster.sync();
  if (ph) ph[4] = global_ns();  // sums done
  // ---- prob_p = e_p * (1/S), in place (the padding of the summed head is scaled too: harmless)
  for (int i = tid; i < G * n_pos; i += kOaThreads) {
    const int g = i / n_pos, p = i % n_pos;
    s_w[g * L.cap_pad + p] = __fmul_rn(s_w[g * L.cap_pad + p], s_inv[g]);
  }
  __syncthreads();
  if (ph) ph[6] = global_ns();  // probabilities ready
  // ---- out_d = sum over positions, in order.  Producer warps write the products (e_p/S)*v_pd of 64 positions at a
  // time into one of two buffers, laid out [four positions][chain][position in the four]; a chain lane then gets
  // the four next terms of its chain with one 16-byte load.  Hand-over by named barriers: 2 + b = buffer b is
  // full, 4 + b = buffer b is free again.
  constexpr int kHandover = (NPW + NCW) * 32;
  constexpr int HW = (G * HP + 31) / 32;  // resident form: chain warps per parity of the dim
  static_assert(2 * HW <= kOaWarps, "too many chains");
  if (kResident) {
    // Warp w walks the chains of the even (w even) or odd dims: lane -> (head g, dim pair j); the parity being uniform
    // in a warp, the f16 -> f32 conversion picks its half of the word without a select.
    if (warp < 2 * HW) {
      const int parity = warp & 1, li = (warp >> 1) * 32 + lane;
      const bool valid = li < G * HP;
      const int g = (valid ? li : 0) / HP, j = (valid ? li : 0) % HP, d = d0 + 2 * j + parity;
      const uint32_t va = (uint32_t)__cvta_generic_to_shared(s_v + j * vt_pitch);
      const uint32_t wa = (uint32_t)__cvta_generic_to_shared(s_w + g * L.cap_pad);
      // the row's own V (rounded through f16 as the cache holds it): requested before the chain, used after it
      const float v_own = a.fuse_rope ? __ldg(a.v_new + (int64_t)b * a.kv_stride + (int64_t)kvh * HD + d) : 0.0f;
      float o = parity ? oa_resident_chain<1>(va, wa, n_pre) : oa_resident_chain<0>(va, wa, n_pre);
      if (a.fuse_rope) {
        const float vl = __half2float(__float2half_rn(v_own));
        o = n_pos == 1 ? vl : __fadd_rn(o, __fmul_rn(s_w[g * L.cap_pad + pos], vl));
      } else if (n_pos == 1) {
        o = __half2float(vbase[d]);  // a single cached position: the context is a copy of V (src/inference.rs:29858-29951)
      }
      if (valid) a.out[(int64_t)b * a.q_stride + ((int64_t)kvh * G + g) * HD + d] = o;
    }
  } else if (pw >= 0) {
    for (int bt = 0; bt < n_batches; ++bt) {
      const int buf = bt & 1;
      if (bt >= 2) {
        if (buf == 0) asm volatile("bar.sync 4, %0;" ::"n"(kHandover));
        else asm volatile("bar.sync 5, %0;" ::"n"(kHandover));
      }
      cp_async_wait<VD - 1>();  // this lane's copy for batch bt has landed (only later groups may be in flight)
      const int pib = pw * PPB + v_pp, p = bt * kOaBatch + pib;  // position within the batch / in the context
      const uint4 raw = *reinterpret_cast<const uint4 *>(vring + (bt % VD) * 512 + lane * 16);
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
      const float2 v0 = __half22float2(h2[0]), v1 = __half22float2(h2[1]), v2 = __half22float2(h2[2]), v3 = __half22float2(h2[3]);
      issue_v(bt + VD);  // the slot's bytes are in registers now
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float w = p < n_pre ? s_w[g * L.cap_pad + p] : 0.0f;
        float *dst = s_prod + (buf * (kOaBatch / 4) + (pib >> 2)) * QP + (g * DPC + 8 * v_k) * 4 + (pib & 3);
        dst[0] = __fmul_rn(w, v0.x);
        dst[4] = __fmul_rn(w, v0.y);
        dst[8] = __fmul_rn(w, v1.x);
        dst[12] = __fmul_rn(w, v1.y);
        dst[16] = __fmul_rn(w, v2.x);
        dst[20] = __fmul_rn(w, v2.y);
        dst[24] = __fmul_rn(w, v3.x);
        dst[28] = __fmul_rn(w, v3.y);
      }
      __threadfence_block();  // the products before the hand-over
      if (buf == 0) asm volatile("bar.arrive 2, %0;" ::"n"(kHandover) : "memory");
      else asm volatile("bar.arrive 3, %0;" ::"n"(kHandover) : "memory");
    }
  } else if (warp < NCW) {
    const int chain = warp * 32 + lane;  // within this CTA: head g, dim dd of the CTA's slice
    const bool valid = chain < CPC;
    const int g = (valid ? chain : 0) / DPC, d = d0 + (valid ? chain : 0) % DPC;
    float o = 0.0f;
    // A unit is 16 positions (four 16-byte loads): the loads of unit u+1 are issued before the 16 dependent additions
    // of unit u.  A buffer is handed back once its last unit is in registers.
    const int n_units = (n_pre + 15) / 16;
    const uint32_t p_addr = (uint32_t)__cvta_generic_to_shared(s_prod + (valid ? chain : 0) * 4);
    auto load_unit = [&](int u, float4(&T)[4]) {
      const int bt = u >> 2, buf = bt & 1, sub = u & 3;
      if (sub == 0) {
        if (buf == 0) asm volatile("bar.sync 2, %0;" ::"n"(kHandover) : "memory");
        else asm volatile("bar.sync 3, %0;" ::"n"(kHandover) : "memory");
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(T[q].x), "=f"(T[q].y), "=f"(T[q].z), "=f"(T[q].w)
                     : "r"(p_addr + ((buf * (kOaBatch / 4) + sub * 4 + q) * QP) * 4));
      if ((sub == 3 || u == n_units - 1) && bt + 2 < n_batches) {
        if (buf == 0) asm volatile("bar.arrive 4, %0;" ::"n"(kHandover) : "memory");
        else asm volatile("bar.arrive 5, %0;" ::"n"(kHandover) : "memory");
      }
    };
    auto add_unit = [&](int u, const float4(&T)[4]) {
      const int cnt = min(16, n_pre - u * 16);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (4 * q + 0 < cnt) o = __fadd_rn(o, T[q].x);
        if (4 * q + 1 < cnt) o = __fadd_rn(o, T[q].y);
        if (4 * q + 2 < cnt) o = __fadd_rn(o, T[q].z);
        if (4 * q + 3 < cnt) o = __fadd_rn(o, T[q].w);
      }
    };
    // Main loop: two batches (eight units) per trip, written out without a branch so that it is one basic block —
    // only then are the next unit's loads scheduled under the current unit's additions (a conditional load, or a
    // barrier number chosen at run time, ends the block and the loads are waited for before the additions start).
    // It runs while the batches after the pair exist; the generic code below takes what is left.
    float4 TA[4], TB[4];
#define OA_LOAD(BUF, SUB, T)                                                                               \
  do {                                                                                                     \
    if (SUB == 0) asm volatile("bar.sync %0, %1;" ::"n"(2 + BUF), "n"(kHandover) : "memory");              \
    _Pragma("unroll") for (int q = 0; q < 4; ++q)                                                          \
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"                                            \
                     : "=f"(T[q].x), "=f"(T[q].y), "=f"(T[q].z), "=f"(T[q].w)                              \
                     : "r"(p_addr + ((BUF * (kOaBatch / 4) + SUB * 4 + q) * QP) * 4));                     \
    if (SUB == 3) asm volatile("bar.arrive %0, %1;" ::"n"(4 + BUF), "n"(kHandover) : "memory");            \
  } while (0)
#define OA_ADD(T)                                \
  do {                                           \
    _Pragma("unroll") for (int q = 0; q < 4; ++q) { \
      o = __fadd_rn(o, T[q].x);                  \
      o = __fadd_rn(o, T[q].y);                  \
      o = __fadd_rn(o, T[q].z);                  \
      o = __fadd_rn(o, T[q].w);                  \
    }                                            \
  } while (0)
    int u = 0;
    const int n_full = n_pre / kOaBatch;  // whole batches
    int main_pairs = (n_full - 2) / 2;    // pairs (2m, 2m+1) with batches 2m+2 and 2m+3 in existence, so that every
    if (n_batches < 4) main_pairs = 0;    // bar.arrive of the loop is one the producers wait for
    if (main_pairs > 0) {
      OA_LOAD(0, 0, TA);
      for (int m = 0; m < main_pairs; ++m) {
        OA_LOAD(0, 1, TB);
        OA_ADD(TA);
        OA_LOAD(0, 2, TA);
        OA_ADD(TB);
        OA_LOAD(0, 3, TB);
        OA_ADD(TA);
        OA_LOAD(1, 0, TA);
        OA_ADD(TB);
        OA_LOAD(1, 1, TB);
        OA_ADD(TA);
        OA_LOAD(1, 2, TA);
        OA_ADD(TB);
        OA_LOAD(1, 3, TB);
        OA_ADD(TA);
        OA_LOAD(0, 0, TA);
        OA_ADD(TB);
      }
      u = main_pairs * 8;  // unit u is loaded in TA, not yet added
    } else if (n_units > 0) {
      load_unit(0, TA);
    }
#undef OA_LOAD
#undef OA_ADD
    for (; u < n_units; u += 2) {
      if (u + 1 < n_units) load_unit(u + 1, TB);
      add_unit(u, TA);
      if (u + 1 < n_units) {
        if (u + 2 < n_units) load_unit(u + 2, TA);
        add_unit(u + 1, TB);
      }
    }
    if (a.fuse_rope) {
      // the row's own V, rounded through f16 as the cache holds it
      const float vl = __half2float(__float2half_rn(a.v_new[(int64_t)b * a.kv_stride + (int64_t)kvh * HD + d]));
      o = n_pos == 1 ? vl : __fadd_rn(o, __fmul_rn(s_w[g * L.cap_pad + pos], vl));
    } else if (n_pos == 1) {
      o = __half2float(vbase[d]);  // a single cached position: the context is a copy of V (src/inference.rs:29858-29951)
    }
    if (valid) a.out[(int64_t)b * a.q_stride + ((int64_t)kvh * G + g) * HD + d] = o;
  }
  cp_async_wait<0>();
  if (ph) ph[5] = global_ns();  // chains done
  // The warps with no part in the output phase park at this CTA barrier, which costs no issue slots; waiting at the
  // cluster barrier instead, they would poll and take the chain warps' issue slots (3x slower chains, measured).
  __syncthreads();
  cluster.sync();  // nobody leaves while its shared memory may still be written or read
}

template <int G, int HD, int VD>
static int32_t launch_oa_vd(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  const OaLayout L = oa_layout(G, HD, cap);
  static int configured = 0;
  if (L.total > configured) {
    CMLD_CUDA(cudaFuncSetAttribute(attn_ordered_kernel<G, HD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
    configured = L.total;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(kOaCluster, (unsigned)a.n_kv_heads, (unsigned)a.batch);
  cfg.blockDim = dim3(kOaThreads);
  cfg.dynamicSmemBytes = (size_t)L.total;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (a.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;
  attr[n_attr].val.clusterDim.x = kOaCluster;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  CMLD_CUDA(cudaLaunchKernelEx(&cfg, attn_ordered_kernel<G, HD, VD>, a, cap));
  return CMLD_OK;
}

template <int G, int HD>
static int32_t launch_oa(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  switch (oa_vdepth(cap)) {
    case 32: return launch_oa_vd<G, HD, 32>(a, cap, s);
    case 16: return launch_oa_vd<G, HD, 16>(a, cap, s);
    default: return launch_oa_vd<G, HD, 8>(a, cap, s);
  }
}

// Whether the cluster kernel takes this shape with contexts of up to `cap` positions.
bool attention_ordered_fits(int n_heads, int n_kv_heads, int head_dim, int64_t cap) {
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return false;
  const int G = n_heads / n_kv_heads;
  if (!(G == 1 || G == 2 || G == 3 || G == 4 || G == 8)) return false;
  if (!(head_dim == 64 || head_dim == 128)) return false;  // each CTA owns head_dim/8 dims: whole 16-byte pieces
  if (cap > 8192) return false;  // the exact sum takes at most 32 chunks of 256 terms
  return oa_layout(G, head_dim, cap).total <= 226 * 1024;
}

// Reference-order attention for rows whose contexts are at most `cap` positions long (a.max_pos bounds the cache rows).
int32_t launch_attention_ordered(const AttnArgs &a, int64_t cap, cudaStream_t s) {
  if (!attention_ordered_fits(a.n_heads, a.n_kv_heads, a.head_dim, cap))
    return fail(CMLD_ERR_SHAPE, "attention (reference order, cluster form): shape %d/%d x %d with %lld positions not supported", a.n_heads,
                a.n_kv_heads, a.head_dim, (long long)cap);
  const int G = a.n_heads / a.n_kv_heads;
#define OA_CASE(g, hd) \
  if (G == g && a.head_dim == hd) return launch_oa<g, hd>(a, cap, s);
  OA_CASE(1, 64) OA_CASE(2, 64) OA_CASE(3, 64) OA_CASE(4, 64) OA_CASE(8, 64)
  OA_CASE(1, 128) OA_CASE(2, 128) OA_CASE(3, 128) OA_CASE(4, 128) OA_CASE(8, 128)
#undef OA_CASE
  return fail(CMLD_ERR_SHAPE, "attention (reference order): unsupported shape");
}

}  // namespace cmld
