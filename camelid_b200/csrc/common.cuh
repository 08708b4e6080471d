// Shared internals of the sm_100a decode library: status plumbing, device layouts of the
// quantised formats, and small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/camelid_b200.h"

namespace cmld {

// ------------------------------------------------------------------ errors

void set_error(const char *fmt, ...);
int32_t fail(int32_t code, const char *fmt, ...);

#define CMLD_CUDA(expr)                                                                         \
  do {                                                                                          \
    cudaError_t err__ = (expr);                                                                 \
    if (err__ != cudaSuccess)                                                                   \
      return ::cmld::fail(err__ == cudaErrorMemoryAllocation ? CMLD_ERR_OOM : CMLD_ERR_CUDA,    \
                          "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, \
                          __LINE__);                                                            \
  } while (0)

#define CMLD_TRY(expr)               \
  do {                               \
    int32_t rc__ = (expr);           \
    if (rc__ != CMLD_OK) return rc__; \
  } while (0)

// ------------------------------------------------------------------ device layouts
//
// A quantised matrix keeps exactly its GGUF wire bytes; rows are contiguous, and within a row
// the bytes are arranged so that every field can be read as 16-byte aligned vectors:
//   Q8_0: [codes: cols x i8][scales: cols/32 x f16]                  (wire blocks are 34 B: 2-byte aligned)
//   Q4_K: the wire superblocks themselves, 144 B each = [f16 d, f16 dmin, 12 scale bytes | 128 nibble bytes]
//   Q6_K: [nsb x 208 B = ql 128 | qh 64 | 16 x i8 scales][d: nsb x f16]  (wire superblocks are 210 B)
// with the row stride rounded up to 16 bytes.  A tile of consecutive rows is therefore one
// contiguous, 16-byte aligned byte range: exactly what one bulk asynchronous copy moves.

constexpr int kWarp = 32;

__host__ __device__ inline int64_t round_up16(int64_t v) { return (v + 15) & ~int64_t(15); }

__host__ __device__ inline int64_t wire_row_bytes(int qt, int64_t cols) {
  switch (qt) {
    case CMLD_Q8_0: return cols / 32 * 34;
    case CMLD_Q4_K: return cols / 256 * 144;
    case CMLD_Q6_K: return cols / 256 * 210;
    case CMLD_Q8_0_HOST36: return cols / 32 * 36;
    case CMLD_F32: return cols * 4;
    default: return -1;
  }
}

__host__ __device__ inline int64_t dev_row_stride(int qt, int64_t cols) {
  switch (qt) {
    case CMLD_Q8_0: return round_up16(cols + cols / 32 * 2);
    case CMLD_Q4_K: return cols / 256 * 144;
    case CMLD_Q6_K: return round_up16(cols / 256 * 210);
    case CMLD_F32: return cols * 4;
    default: return -1;
  }
}

// Quantised activation row: [codes: cols x i8][scales: cols/32 x f32][bsum16: cols/16 x i16],
// stride rounded to 16 bytes.  Q8_K uses the first cols/256 scales; bsum16[j] is the sum of
// codes 16j..16j+15 (what ggml's Q8_K block carries as bsums).
__host__ __device__ inline int64_t act_scale_off(int64_t cols) { return round_up16(cols); }
__host__ __device__ inline int64_t act_bsum_off(int64_t cols) { return round_up16(cols) + round_up16(cols / 32 * 4); }
__host__ __device__ inline int64_t act_row_stride(int64_t cols) {
  return act_bsum_off(cols) + round_up16(cols / 16 * 2);
}

struct Weight {
  int32_t qt = 0;  // CMLD_Q8_0 / Q4_K / Q6_K / F32
  int64_t rows = 0, cols = 0, stride = 0;
  uint8_t *data = nullptr;  // device
  bool owned = true;
};

}  // namespace cmld

struct cmld_weight : cmld::Weight {};

namespace cmld {

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- arrival words written by other GPUs
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Waits until *flag has reached `want` (counts wrap).  Bounded twice over: by time and by polls.  When
// the bound passes, or an earlier wait of this step already gave up, records CMLD_ERR_TIMEOUT in
// *status and returns false; the caller carries on with whatever the slot holds and the host reports
// the error.
__device__ __forceinline__ bool peer_wait(const uint32_t *flag, uint32_t want, unsigned long long timeout_ns, int32_t *status) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  if (*reinterpret_cast<volatile int32_t *>(status) == 0) {
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 1; i < (1u << 26); ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
      if ((i & 255u) == 0 && global_ns() - t0 > timeout_ns) break;
    }
  }
  atomicExch(status, (int32_t)CMLD_ERR_TIMEOUT);
  return false;
}

// Q4_K 6-bit (scale, min) of group g from the 12 packed bytes held as three words
// (q4_k_scale_min, src/tensor/mod.rs:5997-6006 in the Camelid tree).
__device__ __forceinline__ void q4k_scale_min(int g, uint32_t s0, uint32_t s1, uint32_t s2, int &sc, int &m) {
  // bytes 0..3 = s0, 4..7 = s1, 8..11 = s2
  if (g < 4) {
    sc = (s0 >> (8 * g)) & 63;
    m = (s1 >> (8 * g)) & 63;
  } else {
    int k = g - 4;
    uint32_t b8 = (s2 >> (8 * k)) & 0xff;
    sc = (b8 & 0x0f) | (((s0 >> (8 * k + 6)) & 3) << 4);
    m = (b8 >> 4) | (((s1 >> (8 * k + 6)) & 3) << 4);
  }
}

// 128-bit read-only streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

#endif  // __CUDACC__

// Every kernel of the decode step asks for the same (maximum) shared-memory carve-out as the
// staged matvec: an SM whose L1/shared split has to change between two kernels drains first.
template <typename K>
inline void prefer_max_smem_carveout(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// ------------------------------------------------------------------ kernel launchers (host)

// formats.cu
int32_t launch_repack(int qt_in, const uint8_t *wire_dev, int64_t rows, int64_t cols, uint8_t *dst, cudaStream_t s);
int32_t launch_unpack_to_wire(const Weight &w, uint8_t *wire_dev, cudaStream_t s);
int32_t launch_dequant(const Weight &w, int64_t row0, int64_t nrows, float *out, cudaStream_t s);
int32_t launch_synth(const Weight &w, uint64_t seed, uint64_t stream_id, int64_t row0, float sigma, cudaStream_t s);
int32_t launch_embed_gather(const Weight &w, const int32_t *tokens_dev, int32_t batch, float *out, cudaStream_t s);

// gemv.cu
struct GemvJob {
  const uint8_t *w;
  int32_t qt;
  int64_t rows, cols, stride;
  float *y;               // [batch][y_stride]
  const float *residual;  // may be null, same layout as y
  int64_t y_stride;
};
int32_t launch_gemv(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, cudaStream_t s);

// gemv_pipe.cu: the staged kernel.  How its consumers obtain the quantised activation:
struct GemvPrologue {
  int32_t mode;            // 0: quantised rows given (act_k / act_0); 1: RMSNorm(x)*norm_w; 2: x as is; 3: SwiGLU(x, x2)
  const float *x, *x2, *norm_w;
  int64_t x_stride;        // floats between batch rows of x and x2
  float eps;
  const uint8_t *act_k, *act_0;  // mode 0: Q8_K rows / Q8_0 rows in the global activation layout
  float *norm_out;         // optional: f32 copy of the prologue's result [batch][cols]
  int32_t pair_swiglu;     // two matrices (gate, up) of equal shape and type: y of the first receives SwiGLU(gate.x, up.x)
};
// All-reduce of a tensor-parallel sublayer folded into the matvec kernels that produce and consume it,
// over peer memory (NVLink): the producing launch (one matrix: o or down) stores its partial result
// rows into a slot on EVERY rank and, when its last CTA is done, raises this rank's arrival word on
// every rank; the consuming launch's prologue waits (bounded) for all arrival words and takes the sum
// of the ranks' partials, in rank order, as its input row.  No collective kernel runs in between.
constexpr int kMaxPeers = 8;
constexpr int kPeerRows = 8;  // rows a slot holds (the staged kernel's largest batch)
struct GemvPeer {
  int32_t tx_n = 0;                    // ranks; 0 = this launch sends nothing
  float *tx_part[kMaxPeers] = {};      // on rank p: where this rank's partial rows go, [kPeerRows][hidden]
  uint32_t *tx_flag[kMaxPeers] = {};   // on rank p: this rank's arrival word for the slot
  uint32_t *tx_epoch = nullptr;        // local: arrivals sent for the slot so far
  uint32_t *tx_ticket = nullptr;       // local: CTAs of this launch that are done
  int32_t rx_n = 0;                    // ranks; 0 = the input row is read as usual
  const float *rx_part = nullptr;      // local slot: [rank][kPeerRows][hidden]
  const uint32_t *rx_flag = nullptr;   // local: arrival words [rank]
  const uint32_t *rx_epoch = nullptr;  // local: the arrival count to wait for
  float *rx_out = nullptr;             // the summed rows [batch][hidden], written by CTA 0
  unsigned long long timeout_ns = 0;   // bound of the wait
  // Optional timeline (engine option CMLD_TRACE): [0] = records taken so far, then 8 words per launch
  // written by CTA 0: start, inputs visible, peers arrived, prologue done, rows done, ticket taken, n_jobs/tx/rx tag.
  unsigned long long *trace = nullptr;
};
constexpr int kTraceRecords = 4096;
constexpr int kTraceCtas = 160, kTraceCtaRecords = 1024;  // per-CTA stamps of the staged matvec (same option)
// Stand-alone form of the receiving side: h[batch][hidden] = sum of the ranks' partials (ops.cu).
int32_t launch_peer_reduce(const GemvPeer &rx, int32_t batch, int32_t hidden, int32_t *status, bool pdl, cudaStream_t s);

// Optional side job of a staged-matvec launch: pull the KV-cache rows the attention kernel that follows will
// read into L2 (the idle lanes of the producer warp issue bulk prefetches before the kernel waits for its
// predecessor; the rows of earlier positions do not change any more).
struct KvPrefetch {
  const __half *k = nullptr, *v = nullptr;  // this layer's caches, [slot][kv_head][max_pos][head_dim]
  const int32_t *positions = nullptr, *slots = nullptr;
  int32_t n_kv_heads = 0, head_dim = 0, batch = 0;
  int64_t max_pos = 0;
};

// Returns CMLD_ERR_UNSUPPORTED, leaving the error message untouched, when the shape does not fit.
// Largest batch (<= 8) the staged kernel takes for these matrices in one launch; 0 = none.
int gemv_pipe_fit_batch(const GemvJob *jobs, int n_jobs, bool paired = false, bool norm = false);
int32_t launch_gemv_pipe(const GemvJob *jobs, int n_jobs, int32_t batch, const GemvPrologue &pro, int32_t *status,
                         cudaStream_t s, bool pdl, const GemvPeer *peer = nullptr, const KvPrefetch *pf = nullptr);

// gemv_mma.cu: 9..32 activation rows in one pass over the weights (int8 tensor-core MMA)
int64_t gemv_mma_scratch_floats(const GemvJob *jobs, int n_jobs, int32_t batch);
int32_t launch_gemv_mma(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, float *scratch, int64_t scratch_floats,
                        int32_t *status, cudaStream_t s, bool pdl, int64_t *launches);

// gemv_tc5.cu: 9..32 activation rows in one pass over the weights on the tcgen05 tensor cores, results
// bit-identical to the one-row kernels (reference order of f32 operations in the epilogue)
int64_t gemv_tc5_pack_bytes(int64_t cols);
bool gemv_tc5_fits(const GemvJob *jobs, int n_jobs, int32_t batch);
int32_t launch_gemv_tc5(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, uint8_t *pack, int64_t pack_bytes,
                        int32_t *status, cudaStream_t s, int64_t *launches);

int64_t gemv_mma_expert_scratch_floats(const GemvJob *jobs, int n_jobs, int nt, int n_experts, int n_pass);
int32_t launch_gemv_mma_experts(const GemvJob *jobs, int n_jobs, const uint8_t *act, int nt, int n_experts, int n_pass,
                                const int32_t *counts, int first_expert, int expert_step, int cap, int count_mul, float *scratch,
                                int64_t scratch_floats, int32_t *status, cudaStream_t s, bool pdl, int64_t *launches);

// ops.cu
struct NormQuantArgs {
  const float *x;       // [batch][cols]
  const float *x2;      // second operand for SwiGLU (u), else null
  const float *weight;  // RMSNorm weight or null (no norm)
  float eps;
  int64_t cols;
  int32_t batch;
  float *out;           // f32 result or null
  uint8_t *act;         // quantised result or null
  int32_t act_q8_0, act_q8_k;  // which formats to emit; both allowed: Q8_K at act, Q8_0 at act2
  uint8_t *act2;
  int32_t pdl;                 // launch with programmatic stream serialisation
  int32_t exact;               // RMSNorm: add the squares one after another like the CPU (slow)
};
int32_t launch_norm_quant(const NormQuantArgs &a, cudaStream_t s);
int32_t launch_exact_sum_selftest(const float *terms, int32_t n, float *out, cudaStream_t s);
// key_out != null: a vocabulary shard — the final stage writes the packed (value, idx_offset + index)
// key per row instead of the token, and leaves the feedback to launch_argmax_finish.
int32_t launch_argmax(const float *x, int64_t n, int32_t batch, float *part_val, int32_t *part_idx,
                      uint32_t *ticket, int32_t *out_idx, int32_t *next_tokens, int32_t *positions,
                      int32_t *history, cudaStream_t s, unsigned long long *key_out = nullptr, int32_t idx_offset = 0);
int argmax_blocks();

struct RopeKvArgs {
  float *q;        // [batch][n_heads*hd], rotated in place
  const float *k;  // [batch][n_kv*hd]
  const float *v;
  const float *cos_tab, *sin_tab;  // [rows][rope_dim/2]
  int32_t index_by_position;       // 1: row = positions[b]; 0: row = b
  const int32_t *positions;        // [batch]
  const int32_t *slots;            // [batch] KV slot per row
  __half *k_cache, *v_cache;       // this layer: [slot][kv_head][max_pos][hd]
  int32_t n_heads, n_kv_heads, head_dim, rope_dim, split_half, batch;
  int64_t max_pos;
  int64_t q_stride, kv_stride;     // floats between batch rows of q and of k/v
};
int32_t launch_rope_kv(const RopeKvArgs &a, cudaStream_t s);

// attn.cu
struct AttnArgs {
  const float *q;  // [batch][n_heads*hd]
  const __half *k_cache, *v_cache;
  const int32_t *positions, *slots;  // n_pos = positions[b] + 1
  int32_t n_heads, n_kv_heads, head_dim, batch, n_splits;
  int64_t max_pos;
  float scale;
  float *part;  // [batch][n_heads][n_splits][hd + 2]
  uint32_t *tickets;  // [batch][n_kv_heads], zero between launches
  float *out;   // [batch][n_heads*hd]
  int64_t q_stride;
  // Optional fusion of RoPE and the KV-cache write (fuse_rope != 0): q is rotated on the fly, and
  // the CTA whose range holds the row's own position rotates k_new, rounds k_new / v_new to f16
  // and stores them in the cache before using them.
  int32_t fuse_rope, rope_dim, split_half, index_by_position;
  const float *k_new, *v_new;      // [batch][n_kv_heads*hd]
  int64_t kv_stride;
  const float *cos_tab, *sin_tab;  // [rows][rope_dim/2]
  int32_t pdl;                     // launch with programmatic stream serialisation
  int32_t cluster;                 // ranges as the CTAs of a thread-block cluster, merged through distributed shared memory
  unsigned long long *phase_ns;    // optional (reference-order cluster kernel): %globaltimer of CTA 0 at the end of each phase
  // Tree verification (plain reference-order kernel only): cache rows tree_base.. hold the nodes of a draft tree in
  // breadth-first order; row b attends to every position below tree_base and to node j only if bit j of its mask
  // is set (its ancestors and itself).  Null = ordinary causal attention.
  const uint32_t *tree_mask = nullptr;  // [batch][tree_words]
  int32_t tree_base = 0, tree_words = 0;
};
int32_t launch_attention(const AttnArgs &a, cudaStream_t s);
// attn_ordered.cu: the reference-order cluster kernel (contexts of at most `cap` positions)
bool attention_ordered_fits(int n_heads, int n_kv_heads, int head_dim, int64_t cap);
int32_t launch_attention_ordered(const AttnArgs &a, int64_t cap, cudaStream_t s);

// attn_rows.cu: the reference-order attention for steps of several rows (one CTA per (row, KV head))
bool attention_rows_fits(int n_heads, int n_kv_heads, int head_dim, int64_t cap);
int32_t launch_attention_rows(const AttnArgs &a, int64_t cap, cudaStream_t s);

// comm.cu: NCCL collectives of the sharded engine
int32_t comm_unique_id(uint8_t *out128);
int32_t comm_init(void **comm_out, const uint8_t *id128, int rank, int world);
void comm_destroy(void *comm);
int32_t comm_wait_stream(void **comm, cudaStream_t s, int64_t limit_ms, void (*before_abort)(void *), void *ctx);
int32_t comm_allreduce_sum_f32(void *comm, float *buf, int64_t count, cudaStream_t s);
int32_t comm_allreduce_max_u64(void *comm, unsigned long long *buf, int64_t count, cudaStream_t s);
int32_t comm_allgather_f32(void *comm, const float *send, float *recv, int64_t count_per_rank, cudaStream_t s);

// kv_q8.cu: KV cache as Q8_0 blocks (CMLD_FLAG_KV_Q8_0)
int64_t kv_q8_layer_bytes(int64_t seqs, int n_kv, int64_t max_pos, int hd);
int32_t launch_rope_kv_q8(const RopeKvArgs &a, uint8_t *kq, uint8_t *vq, cudaStream_t s);
int32_t launch_attention_q8(const AttnArgs &a, const uint8_t *kq, const uint8_t *vq, cudaStream_t s);
int32_t launch_kv_q8_convert(uint8_t *cache, float *rows, int n_kv, int64_t max_pos, int64_t n_pos, int hd, bool to_cache, cudaStream_t s);

// sample.cu: temperature / min-p sampling over a resident logits row
int32_t launch_sample_gumbel(const float *logits, int32_t n, float inv_temp, uint64_t seed, uint32_t *out_dev, cudaStream_t s);
int32_t launch_sample_gumbel_filtered(const float *logits, int32_t n, float temperature, float min_p, uint64_t seed, uint32_t *out_dev,
                                      cudaStream_t s);
int32_t launch_min_p_mask(const float *logits, int32_t n, float min_p, int32_t *mask_dev, cudaStream_t s);
int32_t launch_sample_uniforms(uint64_t seed, int32_t n, float *out_dev, cudaStream_t s);

// ops.cu: helpers of the sharded step
int32_t launch_residual_add(float *h, const float *delta, int64_t n, bool pdl, cudaStream_t s);
int32_t launch_argmax_finish(const unsigned long long *keys, int32_t batch, int32_t *out_idx, int32_t *next_tokens,
                             int32_t *positions, int32_t *history, uint32_t *ticket_base, cudaStream_t s);
int32_t launch_gather_permute(const float *gathered, float *out, int32_t ranks, int32_t batch, int64_t per_rank, cudaStream_t s);

// exact.cu: reference-order kernels (q already rotated, KV already appended for the attention)
int32_t launch_gemv_exact(const GemvJob &J, const uint8_t *act, int32_t batch, cudaStream_t s);
int32_t launch_attention_exact(const AttnArgs &a, cudaStream_t s);

}  // namespace cmld
