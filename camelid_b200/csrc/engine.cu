// The resident decode engine behind the C ABI: owns weights, KV cache and scratch on one
// B200 and runs the per-token layer stack.  Host-side mirror of Camelid's
// `CudaResidentDecode` (src/cuda_resident.rs:15093 in the Camelid tree): same call surface,
// same argument meaning, errors as status codes instead of Result<_, String>.
#include <cmath>
#include <string>
#include <map>
#include <tuple>
#include <vector>

#include "common.cuh"

namespace cmld {

// ------------------------------------------------------------------ errors

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int32_t fail(int32_t code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

const char *last_error() { return g_err; }

// ------------------------------------------------------------------ weights

int32_t weight_alloc(Weight &w, int32_t qt, int64_t rows, int64_t cols) {
  const int qd = qt == CMLD_Q8_0_HOST36 ? CMLD_Q8_0 : qt;
  if (qd != CMLD_Q8_0 && qd != CMLD_Q4_K && qd != CMLD_Q6_K && qd != CMLD_F32)
    return fail(CMLD_ERR_UNSUPPORTED, "tensor type %d is not one of F32/Q8_0/Q4_K/Q6_K", qt);
  if (rows <= 0 || cols <= 0) return fail(CMLD_ERR_SHAPE, "empty tensor %lld x %lld", (long long)rows, (long long)cols);
  const int blk = qd == CMLD_F32 ? 1 : (qd == CMLD_Q8_0 ? 32 : 256);
  if (cols % blk != 0)
    return fail(CMLD_ERR_SHAPE, "row length %lld is not a multiple of the %d-value block of type %d", (long long)cols, blk, qd);
  w.qt = qd;
  w.rows = rows;
  w.cols = cols;
  w.stride = dev_row_stride(qd, cols);
  w.owned = true;
  CMLD_CUDA(cudaMalloc(&w.data, (size_t)(rows * w.stride)));
  return CMLD_OK;
}

void weight_free(Weight &w) {
  if (w.data && w.owned) cudaFree(w.data);
  w.data = nullptr;
}

// Upload GGUF wire bytes (host or device memory) and re-lay them out.
int32_t weight_upload(Weight &w, int32_t qt, int64_t rows, int64_t cols, const void *wire, uint64_t nbytes, cudaStream_t s) {
  if (!wire) return fail(CMLD_ERR_INVALID, "tensor data is null");
  const int64_t need = wire_row_bytes(qt, cols) * rows;
  if (need < 0) return fail(CMLD_ERR_UNSUPPORTED, "tensor type %d is not one of F32/Q8_0/Q4_K/Q6_K", qt);
  if ((int64_t)nbytes != need)
    return fail(CMLD_ERR_SHAPE, "tensor of type %d and shape %lld x %lld needs %lld bytes, got %llu", qt, (long long)rows,
                (long long)cols, (long long)need, (unsigned long long)nbytes);
  weight_free(w);
  CMLD_TRY(weight_alloc(w, qt, rows, cols));
  if (w.qt == CMLD_F32) {
    CMLD_CUDA(cudaMemcpyAsync(w.data, wire, (size_t)need, cudaMemcpyDefault, s));
    CMLD_CUDA(cudaStreamSynchronize(s));
    return CMLD_OK;
  }
  // Stage in slabs so a 128256 x 4096 table does not need a second full-size buffer.
  const int64_t wrb = wire_row_bytes(qt, cols);
  const int64_t slab_rows = std::max<int64_t>(1, std::min<int64_t>(rows, (int64_t)(256ll << 20) / wrb));
  uint8_t *stage = nullptr;
  CMLD_CUDA(cudaMalloc(&stage, (size_t)(slab_rows * wrb)));
  int32_t rc = CMLD_OK;
  for (int64_t r0 = 0; r0 < rows && rc == CMLD_OK; r0 += slab_rows) {
    const int64_t nr = std::min(slab_rows, rows - r0);
    cudaError_t ce = cudaMemcpyAsync(stage, static_cast<const uint8_t *>(wire) + r0 * wrb, (size_t)(nr * wrb), cudaMemcpyDefault, s);
    if (ce != cudaSuccess) {
      rc = fail(CMLD_ERR_CUDA, "weight upload copy failed: %s", cudaGetErrorString(ce));
      break;
    }
    rc = launch_repack(qt, stage, nr, cols, w.data + r0 * w.stride, s);
    if (rc == CMLD_OK && cudaStreamSynchronize(s) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "weight re-layout failed");
  }
  cudaFree(stage);
  return rc;
}

// ------------------------------------------------------------------ engine

struct LayerW {
  Weight proj[7];  // q k v o gate up down
  float *attn_norm = nullptr, *ffn_norm = nullptr;
  bool dense_set = false;
  // Mixtral
  float *router = nullptr;
  Weight exps[3];  // gate, up, down slabs: rows = n_experts * rows_per_expert
  bool moe_set = false;
};

}  // namespace cmld

using namespace cmld;

struct cmld_engine {
  cmld_config cfg{};   // dimensions of THIS rank: n_heads, n_kv_heads and ffn_dim are the tensor-parallel shares
  cmld_config full{};  // the model's dimensions as given to cmld_engine_create
  int32_t tp = 1, ep = 1, shard_rank = 0;
  int32_t vocab_local = 0;  // rows of the output matrix held here
  void *comm = nullptr;     // NCCL communicator of a sharded engine
  unsigned long long *am_keys = nullptr;  // packed (value, index) per row for the sharded argmax
  float *logits_gather = nullptr, *logits_full = nullptr;
  // Peer-memory link of a tensor-parallel group: one region per rank, mapped into every rank.
  //   parts: [2 slots][rank][kPeerRows][hidden] f32, then arrival words [2 slots][rank] u32
  struct PeerLink {
    bool ready = false;
    uint8_t *region[kMaxPeers] = {};  // [shard_rank] is this rank's own allocation
    uint32_t *local = nullptr;        // epochs[2], tickets[2]
    unsigned long long timeout_ns = 0;
  } peer;
  float *mma_scratch = nullptr;  // per-chunk partial sums of the batched tensor-core matvec
  uint8_t *kq8 = nullptr, *vq8 = nullptr;  // CMLD_FLAG_KV_Q8_0: the KV cache as Q8_0 blocks, [layer][slot][kv_head][max_pos][hd/32] x 34 B
  int64_t kv_q8_bytes = 0;                 // bytes of one layer of one side
  uint32_t *tree_mask = nullptr;  // [kTreeMaxNodes] ancestor masks of a draft tree (one word: at most 32 nodes)
  std::vector<float> rope_freq;  // per-pair angular frequency of the engine-owned RoPE table (rope_pair_frequency)
  uint8_t *tc5_pack = nullptr;   // packed activation records of the tcgen05 batched matvec
  int64_t tc5_pack_bytes = 0;
  int64_t mma_scratch_floats = 0;
  unsigned long long *trace = nullptr;  // matvec timeline (environment CMLD_TRACE=<file>), dumped at destroy
  unsigned long long *attn_phases = nullptr;  // with CMLD_TRACE: the last attention launch's phase clocks (8 words)
  std::string trace_path;
  std::map<int32_t, bool> peer_fit;   // rows -> every matvec of a step fits the staged kernel in one pass
  int device = 0;
  cudaStream_t stream = nullptr;
  int32_t max_rows = 0;  // scratch rows (sequences per step)
  int32_t n_splits = 1, sm_count = 148;
  int32_t q_width = 0, kv_width = 0;
  std::vector<LayerW> layers;
  Weight output, token_embd;
  float *final_norm = nullptr;
  bool has_output = false, has_embd = false;
  __half *kcache = nullptr, *vcache = nullptr;
  int64_t kv_layer_elems = 0;  // halfs per layer per side
  float *cos_all = nullptr, *sin_all = nullptr, *cos_step = nullptr, *sin_step = nullptr;
  float *h = nullptr, *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *gate = nullptr,
        *up = nullptr, *logits = nullptr, *taps = nullptr;
  uint8_t *act_k = nullptr, *act_0 = nullptr;  // Q8_K and Q8_0 operand buffers (widest row)
  float *attn_part = nullptr;
  uint32_t *attn_tickets = nullptr;
  float *am_val = nullptr;
  int32_t *am_idx = nullptr;
  uint32_t *am_ticket = nullptr;  // [2*max_rows]: tickets, then history lengths
  int32_t *out_idx = nullptr, *d_tokens = nullptr, *d_positions = nullptr, *d_slots = nullptr, *d_history = nullptr;
  int64_t history_cap = 0;
  int32_t *moe_sel_idx = nullptr, *moe_counts = nullptr, *moe_lists = nullptr;
  float *moe_sel_w = nullptr, *moe_g = nullptr, *moe_u = nullptr, *moe_act = nullptr, *moe_down = nullptr;
  // tensor-core expert path: three Q8_K rows per assignment, `moe_cap` rows per local expert
  int32_t *moe_pos = nullptr;
  int32_t moe_cap = 0, moe_pass_rows = 0;
  uint8_t *moe_act3_h = nullptr, *moe_act3_f = nullptr;
  float *moe_g3 = nullptr, *moe_u3 = nullptr, *moe_d3 = nullptr, *moe_scratch = nullptr;
  int64_t moe_scratch_floats = 0;
  int32_t *d_status = nullptr;  // set by a kernel whose bounded wait gave up
  int64_t filled = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = 0.0f;
  int64_t last_launches = 0, launches = 0;
  std::vector<void *> allocs;
  // CUDA graphs of whole steps, keyed by (rows, option bits, score-scale bits).  A key's first
  // step runs as plain launches (it also sets kernel attributes); its second is captured.
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int64_t launches = 0;
    int uses = 0;
  };
  std::map<std::tuple<int32_t, uint32_t, uint32_t>, StepGraph> graphs;
  bool graphs_off = false;
};

namespace cmld {

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
    if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

#define CMLD_ENGINE_ENTER(e)                                              \
  if (!(e)) return fail(CMLD_ERR_INVALID, "engine handle is null");       \
  DeviceGuard guard__((e)->device);                                       \
  if (!guard__.ok) return fail(CMLD_ERR_CUDA, "cannot select CUDA device %d", (e)->device)

template <typename T>
static int32_t dev_alloc(cmld_engine *e, T **p, int64_t count, bool zero = true) {
  void *raw = nullptr;
  const size_t bytes = (size_t)std::max<int64_t>(count, 1) * sizeof(T);
  CMLD_CUDA(cudaMalloc(&raw, bytes));
  e->allocs.push_back(raw);
  if (zero) CMLD_CUDA(cudaMemsetAsync(raw, 0, bytes, e->stream));
  *p = static_cast<T *>(raw);
  return CMLD_OK;
}

// cos/sin of position * frequency for every position and pair, by the host libm, onto the device.
static int32_t upload_rope_tables(cmld_engine *e) {
  const cmld_config &c = e->cfg;
  const int half = c.rope_dim / 2;
  std::vector<float> ct((size_t)c.max_pos * half), st((size_t)c.max_pos * half);
  for (int64_t p = 0; p < c.max_pos; ++p)
    for (int i = 0; i < half; ++i) {
      const float ang = (float)p * e->rope_freq[i];
      st[(size_t)p * half + i] = sinf(ang);
      ct[(size_t)p * half + i] = cosf(ang);
    }
  CMLD_CUDA(cudaMemcpyAsync(e->cos_all, ct.data(), ct.size() * 4, cudaMemcpyHostToDevice, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->sin_all, st.data(), st.size() * 4, cudaMemcpyHostToDevice, e->stream));
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  return CMLD_OK;
}

static int32_t validate_config(const cmld_config &c) {
  if (c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.hidden <= 0 || c.ffn_dim <= 0 ||
      c.max_pos <= 0 || c.vocab <= 0)
    return fail(CMLD_ERR_SHAPE, "engine dimensions must be positive");
  // resident_decode_eligible (src/inference.rs:3503-3529 in the Camelid tree)
  if (c.hidden % 32 || c.ffn_dim % 32 || (c.n_heads * c.head_dim) % 32)
    return fail(CMLD_ERR_SHAPE, "hidden, ffn_dim and n_heads*head_dim must be multiples of 32");
  if (c.n_heads % c.n_kv_heads) return fail(CMLD_ERR_SHAPE, "n_heads must be a multiple of n_kv_heads");
  if (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128)
    return fail(CMLD_ERR_SHAPE, "head_dim %d not in {32,64,128}", c.head_dim);
  const int g = c.n_heads / c.n_kv_heads;
  if (!(g == 1 || g == 2 || g == 3 || g == 4 || g == 8))
    return fail(CMLD_ERR_SHAPE, "%d query heads per kv head not supported", g);
  if (c.rope_dim <= 0 || c.rope_dim > c.head_dim || c.rope_dim % 2)
    return fail(CMLD_ERR_SHAPE, "rope_dim %d must be even and within head_dim", c.rope_dim);
  if (c.n_experts < 0 || (c.n_experts > 0 && (c.n_experts_used <= 0 || c.n_experts_used > c.n_experts)))
    return fail(CMLD_ERR_SHAPE, "bad expert counts %d/%d", c.n_experts_used, c.n_experts);
  if (c.max_pos > (1 << 24)) return fail(CMLD_ERR_SHAPE, "max_pos too large");
  return CMLD_OK;
}

static int32_t engine_init(cmld_engine *e) {
  const cmld_config &c = e->cfg;
  CMLD_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
  CMLD_CUDA(cudaEventCreate(&e->ev0));
  CMLD_CUDA(cudaEventCreate(&e->ev1));
  const int seqs = std::max(1, c.max_seqs);
  e->max_rows = std::max(seqs, 32);  // a prompt is ingested 32 rows at a time (one tensor-core pass over the weights)
  e->q_width = c.n_heads * c.head_dim;
  e->kv_width = c.n_kv_heads * c.head_dim;
  e->layers.resize(c.n_layers);
  // KV cache: [layer][slot][kv_head][max_pos][head_dim] f16, K and V
  e->kv_layer_elems = (int64_t)seqs * c.n_kv_heads * c.max_pos * c.head_dim;
  if (c.flags & CMLD_FLAG_KV_Q8_0) {
    // the cache as Q8_0 blocks (src/tensor/kv_quant.rs): 34 bytes per 32 values instead of 64
    if (c.head_dim % 32) return fail(CMLD_ERR_SHAPE, "Q8_0 KV cache: head_dim %d is not a multiple of 32", c.head_dim);
    e->kv_q8_bytes = kv_q8_layer_bytes(seqs, c.n_kv_heads, c.max_pos, c.head_dim);
    CMLD_TRY(dev_alloc(e, &e->kq8, e->kv_q8_bytes * c.n_layers));
    CMLD_TRY(dev_alloc(e, &e->vq8, e->kv_q8_bytes * c.n_layers));
    e->kv_layer_elems = 0;
    CMLD_TRY(dev_alloc(e, &e->kcache, 8));
    CMLD_TRY(dev_alloc(e, &e->vcache, 8));
  } else {
    CMLD_TRY(dev_alloc(e, &e->kcache, e->kv_layer_elems * c.n_layers));
    CMLD_TRY(dev_alloc(e, &e->vcache, e->kv_layer_elems * c.n_layers));
  }
  // RoPE tables for every position, computed with the host libm exactly as the reference's
  // resident_decode_rope_tables does per token (src/inference/rope.rs:600-655).  The default per-pair
  // frequency is freq_base^(-2i/rope_dim); cmld_engine_set_rope_frequencies replaces it (rope_freqs.weight,
  // linear / llama3 scaling: rope_pair_frequency, src/inference/rope.rs:532-560).
  const int half = c.rope_dim / 2;
  {
    const float base = c.rope_theta > 0.0f ? c.rope_theta : 10000.0f;
    e->rope_freq.resize(half);
    for (int i = 0; i < half; ++i) e->rope_freq[i] = powf(base, -((float)i * 2.0f) / (float)c.rope_dim);
    CMLD_TRY(dev_alloc(e, &e->cos_all, (int64_t)c.max_pos * half, false));
    CMLD_TRY(dev_alloc(e, &e->sin_all, (int64_t)c.max_pos * half, false));
    CMLD_TRY(upload_rope_tables(e));
  }
  const int64_t R = e->max_rows;
  CMLD_TRY(dev_alloc(e, &e->cos_step, R * half));
  CMLD_TRY(dev_alloc(e, &e->sin_step, R * half));
  CMLD_TRY(dev_alloc(e, &e->h, R * c.hidden));
  CMLD_TRY(dev_alloc(e, &e->normed, R * c.hidden));
  CMLD_TRY(dev_alloc(e, &e->q, R * e->q_width));
  CMLD_TRY(dev_alloc(e, &e->k, R * e->kv_width));
  CMLD_TRY(dev_alloc(e, &e->v, R * e->kv_width));
  CMLD_TRY(dev_alloc(e, &e->attn, R * e->q_width));
  CMLD_TRY(dev_alloc(e, &e->gate, R * c.ffn_dim));
  CMLD_TRY(dev_alloc(e, &e->up, R * c.ffn_dim));
  CMLD_TRY(dev_alloc(e, &e->logits, R * (int64_t)e->vocab_local));
  CMLD_TRY(dev_alloc(e, &e->am_keys, R));
  if (e->tp > 1) {
    CMLD_TRY(dev_alloc(e, &e->logits_gather, R * (int64_t)c.vocab));
    CMLD_TRY(dev_alloc(e, &e->logits_full, R * (int64_t)c.vocab));
  }
  CMLD_TRY(dev_alloc(e, &e->taps, (int64_t)c.n_layers * R * c.hidden));
  const int64_t widest = std::max<int64_t>(std::max(c.hidden, c.ffn_dim), e->q_width);
  CMLD_TRY(dev_alloc(e, &e->act_k, R * act_row_stride(widest)));
  CMLD_TRY(dev_alloc(e, &e->act_0, R * act_row_stride(widest)));
  // flash-decoding splits: enough CTAs to cover the SMs twice at batch 1
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device);
  e->sm_count = sms;
  e->n_splits = std::max(1, std::min<int>(64, (2 * sms + c.n_kv_heads - 1) / c.n_kv_heads));
  e->n_splits = (int)std::min<int64_t>(e->n_splits, std::max<int64_t>(1, c.max_pos / 32));
  CMLD_TRY(dev_alloc(e, &e->attn_part, R * c.n_heads * e->n_splits * (c.head_dim + 2)));
  CMLD_TRY(dev_alloc(e, &e->attn_tickets, R * c.n_kv_heads));
  CMLD_TRY(dev_alloc(e, &e->am_val, R * argmax_blocks()));
  CMLD_TRY(dev_alloc(e, &e->am_idx, R * argmax_blocks()));
  CMLD_TRY(dev_alloc(e, &e->am_ticket, 2 * R));
  CMLD_TRY(dev_alloc(e, &e->out_idx, R));
  CMLD_TRY(dev_alloc(e, &e->d_tokens, R));
  CMLD_TRY(dev_alloc(e, &e->d_positions, R));
  CMLD_TRY(dev_alloc(e, &e->d_slots, R));
  if (c.n_experts > 0) {
    const int64_t na = R * c.n_experts_used;
    CMLD_TRY(dev_alloc(e, &e->moe_sel_idx, na));
    CMLD_TRY(dev_alloc(e, &e->moe_sel_w, na));
    CMLD_TRY(dev_alloc(e, &e->moe_counts, c.n_experts));
    CMLD_TRY(dev_alloc(e, &e->moe_lists, (int64_t)c.n_experts * na));
    CMLD_TRY(dev_alloc(e, &e->moe_g, na * c.ffn_dim));
    CMLD_TRY(dev_alloc(e, &e->moe_u, na * c.ffn_dim));
    CMLD_TRY(dev_alloc(e, &e->moe_act, na * c.ffn_dim));
    CMLD_TRY(dev_alloc(e, &e->moe_down, na * c.hidden));
    CMLD_TRY(dev_alloc(e, &e->moe_pos, na));
    if (c.hidden % 256 == 0 && c.ffn_dim % 256 == 0 && (c.flags & CMLD_FLAG_TENSOR_BATCH) && !(c.flags & (CMLD_FLAG_EXACT_ORDER | CMLD_FLAG_DIRECT_GEMV))) {
      const int64_t n_local = c.n_experts / std::max(1, c.ep_size);
      e->moe_cap = (int32_t)(3 * na);  // every assignment could land on one expert
      const int64_t rows = n_local * e->moe_cap;
      CMLD_TRY(dev_alloc(e, &e->moe_act3_h, rows * act_row_stride(c.hidden)));
      CMLD_TRY(dev_alloc(e, &e->moe_act3_f, rows * act_row_stride(c.ffn_dim)));
      CMLD_TRY(dev_alloc(e, &e->moe_g3, rows * c.ffn_dim, false));
      CMLD_TRY(dev_alloc(e, &e->moe_u3, rows * c.ffn_dim, false));
      CMLD_TRY(dev_alloc(e, &e->moe_d3, rows * c.hidden, false));
      // per-chunk partial sums of the expert matvecs: (rows in flight + one pass of padding) per local expert
      auto chunks = [](int64_t cols) { return (cols / 256 + 3) / 4; };
      const int64_t per_row = std::max(chunks(c.hidden) * 2 * (int64_t)c.ffn_dim, chunks(c.ffn_dim) * (int64_t)c.hidden);
      e->moe_scratch_floats = n_local * per_row * (e->moe_cap + 32);
      CMLD_TRY(dev_alloc(e, &e->moe_scratch, e->moe_scratch_floats, false));
    }
  }
  {
    // the batched matvec cuts the columns into 1024-wide chunks and sums the chunks afterwards
    auto chunks = [](int64_t cols) { return (cols / 256 + 3) / 4; };
    int64_t need = 0;
    need = std::max(need, chunks(c.hidden) * (e->q_width + 2 * (int64_t)e->kv_width));
    need = std::max(need, chunks(e->q_width) * c.hidden);
    need = std::max(need, chunks(c.hidden) * 2 * (int64_t)c.ffn_dim);
    need = std::max(need, chunks(c.ffn_dim) * c.hidden);
    need = std::max(need, chunks(c.hidden) * (int64_t)e->vocab_local);
    e->mma_scratch_floats = need * 32;
    CMLD_TRY(dev_alloc(e, &e->mma_scratch, e->mma_scratch_floats, false));
  }
  {
    const int64_t widest = std::max<int64_t>(std::max<int64_t>(c.hidden, c.ffn_dim), e->q_width);
    e->tc5_pack_bytes = gemv_tc5_pack_bytes((widest + 255) / 256 * 256);
    CMLD_TRY(dev_alloc(e, &e->tc5_pack, e->tc5_pack_bytes, false));
  }
  if (const char *tp = getenv("CMLD_TRACE")) {
    e->trace_path = std::string(tp) + "." + std::to_string(e->shard_rank);
    CMLD_TRY(dev_alloc(e, &e->trace, 1 + 8 * (int64_t)kTraceRecords + (int64_t)kTraceCtas * (1 + 4 * (int64_t)kTraceCtaRecords)));
    CMLD_TRY(dev_alloc(e, &e->attn_phases, 8));
  }
  e->history_cap = 4096;
  CMLD_TRY(dev_alloc(e, &e->d_history, e->history_cap * R));
  CMLD_TRY(dev_alloc(e, &e->d_status, 1));
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  return CMLD_OK;
}

static void peer_link_close(cmld_engine *e) {
  cmld_engine::PeerLink &L = e->peer;
  L.ready = false;
  for (int p = 0; p < kMaxPeers; ++p) {
    if (!L.region[p]) continue;
    if (p == e->shard_rank) cudaFree(L.region[p]);
    else cudaIpcCloseMemHandle(L.region[p]);
    L.region[p] = nullptr;
  }
  cudaGetLastError();
}

// Weights changed: graphs captured so far hold the old matrices' addresses.
static void drop_graphs(cmld_engine *e) {
  cudaStreamSynchronize(e->stream);
  for (auto &kv : e->graphs)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  e->graphs.clear();
  e->peer_fit.clear();
}

static void dump_trace(cmld_engine *e) {
  if (e->attn_phases) {
    unsigned long long h[8] = {0};
    if (cudaMemcpy(h, e->attn_phases, 64, cudaMemcpyDeviceToHost) == cudaSuccess && h[5])
      fprintf(stderr, "last attention launch, phases (us): scores %.2f, maxima %.2f, weights %.2f, sums %.2f, scaling %.2f, chains %.2f\n",
              (h[1] - h[0]) * 1e-3, (h[2] - h[1]) * 1e-3, (h[3] - h[2]) * 1e-3, (h[4] - h[3]) * 1e-3, (h[6] - h[4]) * 1e-3, (h[5] - h[6]) * 1e-3);
  }
  if (!e->trace || e->trace_path.empty()) return;
  std::vector<unsigned long long> host(1 + 8 * (size_t)kTraceRecords);
  if (cudaMemcpy(host.data(), e->trace, host.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
  FILE *f = fopen(e->trace_path.c_str(), "w");
  if (!f) return;
  const size_t n = std::min<size_t>(host[0], kTraceRecords);
  fprintf(f, "start_ns,visible,arrived,prologue,rows,ticket,jobs,tx,rx,cols\n");
  for (size_t i = 0; i < n; ++i) {
    const unsigned long long *r = host.data() + 1 + i * 8;
    fprintf(f, "%llu,%lld,%lld,%lld,%lld,%lld,%llu,%llu,%llu,%llu,%lld\n", r[0], (long long)(r[1] - r[0]), (long long)(r[2] - r[0]),
            (long long)(r[3] - r[0]), (long long)(r[4] - r[0]), r[5] ? (long long)(r[5] - r[0]) : -1, r[6] & 0xff, (r[6] >> 8) & 0xff,
            (r[6] >> 16) & 0xff, r[6] >> 32, r[7] ? (long long)(r[7] - r[0]) : -1);
  }
  fclose(f);
  // per-CTA stamps: one line per (CTA, launch) of the last kTraceCtaRecords launches, absolute nanoseconds
  const size_t per = 1 + 4 * (size_t)kTraceCtaRecords;
  std::vector<unsigned long long> cta((size_t)kTraceCtas * per);
  if (cudaMemcpy(cta.data(), e->trace + 1 + 8 * (size_t)kTraceRecords, cta.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
  f = fopen((e->trace_path + ".cta").c_str(), "w");
  if (!f) return;
  fprintf(f, "cta,launch,start_ns,visible_ns,prologue_ns,rows_ns\n");
  for (int b = 0; b < kTraceCtas; ++b) {
    const unsigned long long cnt = cta[b * per];
    const unsigned long long lo = cnt > (unsigned long long)kTraceCtaRecords ? cnt - kTraceCtaRecords : 0;
    for (unsigned long long k = lo; k < cnt; ++k) {
      const unsigned long long *r = cta.data() + b * per + 1 + 4 * (k % kTraceCtaRecords);
      fprintf(f, "%d,%llu,%llu,%llu,%llu,%llu\n", b, k, r[0], r[1], r[2], r[3]);
    }
  }
  fclose(f);
}

static void engine_free(cmld_engine *e) {
  dump_trace(e);
  // Graphs first, communicator second: NCCL counts the graphs that captured its collectives and its
  // teardown waits until the last of them is gone.
  for (auto &kv : e->graphs)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  e->graphs.clear();
  comm_destroy(e->comm);
  e->comm = nullptr;
  peer_link_close(e);

  for (auto &L : e->layers) {
    for (auto &w : L.proj) weight_free(w);
    for (auto &w : L.exps) weight_free(w);
    cudaFree(L.attn_norm);
    cudaFree(L.ffn_norm);
    cudaFree(L.router);
  }
  weight_free(e->output);
  weight_free(e->token_embd);
  cudaFree(e->final_norm);
  for (void *p : e->allocs) cudaFree(p);
  if (e->ev0) cudaEventDestroy(e->ev0);
  if (e->ev1) cudaEventDestroy(e->ev1);
  if (e->stream) cudaStreamDestroy(e->stream);
}

static int32_t upload_f32(float **dst, const float *src, int64_t n, cudaStream_t s) {
  if (!src) return fail(CMLD_ERR_INVALID, "norm weights are null");
  if (!*dst) CMLD_CUDA(cudaMalloc(dst, (size_t)n * 4));
  CMLD_CUDA(cudaMemcpyAsync(*dst, src, (size_t)n * 4, cudaMemcpyDefault, s));
  CMLD_CUDA(cudaStreamSynchronize(s));
  return CMLD_OK;
}

// Which operand formats a group of matrices reading the same activation needs.
static void act_kinds(const Weight *const *ws, int n, bool &need_0, bool &need_k) {
  need_0 = need_k = false;
  for (int i = 0; i < n; ++i) {
    if (ws[i]->qt == CMLD_Q8_0) need_0 = true;
    else need_k = true;
  }
}

struct Proj {
  const Weight *w;
  float *y;
  const float *residual;
  int64_t y_stride;
};

// Matvecs that share one activation row, direct-load kernel: one launch per operand format.
static int32_t run_gemv_group(cmld_engine *e, const Proj *p, int n, int32_t batch) {
  for (int pass = 0; pass < 2; ++pass) {
    GemvJob jobs[4];
    int nj = 0;
    for (int i = 0; i < n; ++i) {
      const bool is0 = p[i].w->qt == CMLD_Q8_0;
      if (is0 != (pass == 0)) continue;
      jobs[nj++] = GemvJob{p[i].w->data, p[i].w->qt, p[i].w->rows, p[i].w->cols, p[i].w->stride, p[i].y, p[i].residual, p[i].y_stride};
    }
    if (nj == 0) continue;
    CMLD_TRY(launch_gemv(jobs, nj, pass == 0 ? e->act_0 : e->act_k, batch, e->stream));
    e->launches += (batch + 7) / 8;
  }
  return CMLD_OK;
}

static int32_t run_norm_quant(cmld_engine *e, const float *x, const float *x2, const float *weight, int64_t cols,
                              int32_t batch, float *out, bool need_0, bool need_k) {
  NormQuantArgs a{};
  a.x = x;
  a.x2 = x2;
  a.weight = weight;
  a.eps = e->cfg.eps;
  a.cols = cols;
  a.batch = batch;
  a.out = out;
  a.act_q8_0 = need_0;
  a.act_q8_k = need_k;
  a.act = need_k ? e->act_k : e->act_0;
  a.act2 = e->act_0;
  a.pdl = !(e->cfg.flags & CMLD_FLAG_NO_PDL);
  a.exact = (e->cfg.flags & CMLD_FLAG_EXACT_ORDER) != 0;
  CMLD_TRY(launch_norm_quant(a, e->stream));
  e->launches += 1;
  return CMLD_OK;
}

// One sublayer's matvecs: y_i = W_i . quantise(f(x)) (+ residual), f = RMSNorm / identity / SwiGLU.
// Fast path: the staged kernel with f and the quantiser fused into its prologue (batch in passes
// of 8 columns).  Shapes it does not take fall back to quantise-kernel + direct-load kernel.
// Prologue in the matvec CTAs only for the smallest batches: every CTA repeats it, so its cost grows with
// the rows while a separate kernel does it once.
constexpr int kFusedPrologueMaxBatch = 2;

// Rows from which a step's matvecs run on the int8 mma.sync kernel.  That kernel adds a row's terms in a
// different order from the CPU path, so it is opt-in (CMLD_FLAG_TENSOR_BATCH); by default every step
// goes through the staged kernel, in passes of up to 8 rows.
static int mma_min_rows(const cmld_engine *e) { return (e->cfg.flags & CMLD_FLAG_TENSOR_BATCH) ? 5 : (1 << 30); }
// Steps of this many rows or more (and prompt chunks) take the tcgen05 batched matvec: one pass over the weights
// for up to 32 rows, the same bits as the one-row kernels.  Up to 8 rows the staged kernel's single pass is faster.
static int tc5_min_rows(const cmld_engine *e) {
  return (e->cfg.flags & (CMLD_FLAG_EXACT_ORDER | CMLD_FLAG_DIRECT_GEMV | CMLD_FLAG_TENSOR_BATCH)) ? (1 << 30) : 9;
}

static int32_t gemv_fused(cmld_engine *e, const Proj *p, int n, int32_t batch, int mode, const float *x, const float *x2,
                          const float *norm_w, int64_t cols, const GemvPeer *peer = nullptr, bool pair_swiglu = false,
                          const KvPrefetch *pf = nullptr) {
  bool n0, nk;
  const Weight *ws[4];
  for (int i = 0; i < n; ++i) ws[i] = p[i].w;
  act_kinds(ws, n, n0, nk);
  const bool fused = !(e->cfg.flags & CMLD_FLAG_SPLIT_PROLOGUE) && (batch <= kFusedPrologueMaxBatch || peer != nullptr);
  const bool pdl = !(e->cfg.flags & CMLD_FLAG_NO_PDL);
  if (e->cfg.flags & CMLD_FLAG_EXACT_ORDER) {
    // reference order: quantise once (sequential mean square), then one ordered matvec per matrix
    CMLD_TRY(run_norm_quant(e, x, mode == 3 ? x2 : nullptr, mode == 1 ? norm_w : nullptr, cols, batch, nullptr, n0, nk));
    for (int i = 0; i < n; ++i) {
      const GemvJob j{p[i].w->data, p[i].w->qt, p[i].w->rows, p[i].w->cols, p[i].w->stride, p[i].y, p[i].residual, p[i].y_stride};
      CMLD_TRY(launch_gemv_exact(j, p[i].w->qt == CMLD_Q8_0 ? e->act_0 : e->act_k, batch, e->stream));
      e->launches += 1;
    }
    return CMLD_OK;
  }
  if (batch >= tc5_min_rows(e) && n <= 3 && !peer && !pair_swiglu && !(n0 && nk)) {
    GemvJob jobs[3];
    for (int i = 0; i < n; ++i)
      jobs[i] = GemvJob{p[i].w->data, p[i].w->qt, p[i].w->rows, p[i].w->cols, p[i].w->stride, p[i].y, p[i].residual, p[i].y_stride};
    if (gemv_tc5_fits(jobs, n, std::min(batch, 32)) && gemv_tc5_pack_bytes(cols) <= e->tc5_pack_bytes) {
      CMLD_TRY(run_norm_quant(e, x, mode == 3 ? x2 : nullptr, mode == 1 ? norm_w : nullptr, cols, batch, nullptr, n0, nk));
      for (int b0 = 0; b0 < batch; b0 += 32) {
        const int nb = std::min(32, batch - b0);
        for (int i = 0; i < n; ++i) {
          jobs[i].y = p[i].y + (int64_t)b0 * p[i].y_stride;
          jobs[i].residual = p[i].residual ? p[i].residual + (int64_t)b0 * p[i].y_stride : nullptr;
        }
        const uint8_t *act = (n0 ? e->act_0 : e->act_k) + (int64_t)b0 * act_row_stride(cols);
        CMLD_TRY(launch_gemv_tc5(jobs, n, act, nb, e->tc5_pack, e->tc5_pack_bytes, e->d_status, e->stream, &e->launches));
      }
      return CMLD_OK;
    }
  }
  if (!(e->cfg.flags & CMLD_FLAG_DIRECT_GEMV) && n <= 3 && batch > mma_min_rows(e) - 1 && !peer && !pair_swiglu && !(n0 && nk)) {
    // more rows than the dp4a kernel takes in one pass: one pass over the weights on the tensor cores
    GemvJob jobs[3];
    for (int i = 0; i < n; ++i)
      jobs[i] = GemvJob{p[i].w->data, p[i].w->qt, p[i].w->rows, p[i].w->cols, p[i].w->stride, p[i].y, p[i].residual, p[i].y_stride};
    const int64_t need = gemv_mma_scratch_floats(jobs, n, std::min(batch, 32));
    if (need >= 0 && need <= e->mma_scratch_floats) {
      CMLD_TRY(run_norm_quant(e, x, mode == 3 ? x2 : nullptr, mode == 1 ? norm_w : nullptr, cols, batch, nullptr, n0, nk));
      for (int b0 = 0; b0 < batch; b0 += 32) {
        const int nb = std::min(32, batch - b0);
        for (int i = 0; i < n; ++i) {
          jobs[i].y = p[i].y + (int64_t)b0 * p[i].y_stride;
          jobs[i].residual = p[i].residual ? p[i].residual + (int64_t)b0 * p[i].y_stride : nullptr;
        }
        const uint8_t *act = (n0 ? e->act_0 : e->act_k) + (int64_t)b0 * act_row_stride(cols);
        CMLD_TRY(launch_gemv_mma(jobs, n, act, nb, e->mma_scratch, e->mma_scratch_floats, e->d_status, e->stream, pdl, &e->launches));
      }
      return CMLD_OK;
    }
  }
  if (!(e->cfg.flags & CMLD_FLAG_DIRECT_GEMV) && n <= 3) {
    GemvJob jobs[3];
    for (int i = 0; i < n; ++i)
      jobs[i] = GemvJob{p[i].w->data, p[i].w->qt, p[i].w->rows, p[i].w->cols, p[i].w->stride, p[i].y, p[i].residual, p[i].y_stride};
    const int fit = gemv_pipe_fit_batch(jobs, n, pair_swiglu, fused && mode == 1);  // columns per pass: the same for every batch size, so
    if (fit > 0) {                                // a row's result does not depend on who shares its step
      // Activation preparation.  Default: each matvec CTA computes norm / SwiGLU / quantisation itself in
      // its prologue (repeated on every SM, but no extra launch on the critical path); with
      // CMLD_FLAG_SPLIT_PROLOGUE one small multi-CTA kernel writes the quantised rows once and the
      // matvec CTAs copy them.
      if (!fused) CMLD_TRY(run_norm_quant(e, x, mode == 3 ? x2 : nullptr, mode == 1 ? norm_w : nullptr, cols, batch, nullptr, n0, nk));
      for (int b0 = 0; b0 < batch; b0 += fit) {
        const int nb = std::min(fit, batch - b0);
        for (int i = 0; i < n; ++i) {
          jobs[i].y = p[i].y + (int64_t)b0 * p[i].y_stride;
          jobs[i].residual = p[i].residual ? p[i].residual + (int64_t)b0 * p[i].y_stride : nullptr;
        }
        GemvPrologue pro{};
        pro.pair_swiglu = pair_swiglu ? 1 : 0;
        if (fused) {
          pro.mode = mode;
          pro.x = x + (int64_t)b0 * cols;
          pro.x2 = x2 ? x2 + (int64_t)b0 * cols : nullptr;
          pro.norm_w = norm_w;
          pro.x_stride = cols;
          pro.eps = e->cfg.eps;
        } else {
          pro.mode = 0;
          pro.act_k = e->act_k + (int64_t)b0 * act_row_stride(cols);
          pro.act_0 = e->act_0 + (int64_t)b0 * act_row_stride(cols);
        }
        if (peer && (b0 != 0 || nb != batch)) return fail(CMLD_ERR_STATE, "peer-memory matvec split into passes");
        GemvPeer traced;
        if (e->trace) {
          if (peer) traced = *peer;
          traced.trace = e->trace;
        }
        CMLD_TRY(launch_gemv_pipe(jobs, n, nb, pro, e->d_status, e->stream, pdl, e->trace ? &traced : peer, b0 == 0 ? pf : nullptr));
        e->launches += 1;
      }
      return CMLD_OK;
    }
  }
  if (peer || pair_swiglu) return fail(CMLD_ERR_STATE, "matvec with a fused sum or SwiGLU does not fit the staged kernel");
  CMLD_TRY(run_norm_quant(e, x, mode == 3 ? x2 : nullptr, mode == 1 ? norm_w : nullptr, cols, batch, nullptr, n0, nk));
  return run_gemv_group(e, p, n, batch);
}

struct StepOpts {
  int32_t batch = 1;
  bool from_tokens = false;    // gather embeddings of d_tokens, else h holds them
  bool rope_by_position = true;  // index the engine's all-position table, else cos_step/sin_step rows
  float scale = 0.0f;
  bool logits = true;
  bool argmax = true;
  bool feed_back = false;  // argmax writes next token / position / history
  bool taps = false;
  int32_t layer_begin = 0, layer_end = -1;  // layers to run; -1 = through the last
  bool attn_cluster = false;  // short contexts, few rows: attention ranges as a thread-block cluster (host-side choice)
  int32_t attn_cap = 0;       // bound on the context length of every row of this step (a bucket: 1024, 2048, 4096, 8192), 0 = unknown
  const uint32_t *tree_mask = nullptr;  // tree verification: per-row ancestor masks (device), nodes at cache rows tree_base..
  int32_t tree_base = 0, tree_words = 0;
  bool shared_slots = false;  // several rows of this step belong to one sequence (prefill, verify): row b
                              // reads K/V that rows < b write, so the KV append must be a kernel of its own
};

// moe.cu
int32_t moe_route(const float *normed, const float *router, int hidden, int n_exp, int k, int batch, int32_t *sel_idx,
                  float *sel_w, int32_t *counts, int32_t *lists, cudaStream_t s, int32_t *pos);
int32_t moe_quant3(const float *x, const float *x2, int mode, int cols, int k, int n_assign, int n_local, int first_expert,
                   int expert_step, int cap, const int32_t *counts, const int32_t *lists, uint8_t *act, cudaStream_t s);
int32_t moe_combine3(float *h, const float *y3, const float *sel_w, const int32_t *sel_idx, const int32_t *pos, int hidden, int k,
                     int batch, int first_expert, int expert_step, int cap, bool add_residual, cudaStream_t s);
int32_t moe_expert_gemv(const Weight &slab, int64_t rows_per_expert, int n_local_experts, int first_expert, int expert_step,
                        const float *x, int64_t x_stride, int x_div, float *y, const int32_t *counts, const int32_t *lists,
                        int n_assign, cudaStream_t s);
int32_t moe_expert_gemv_ordered(const Weight &slab, int64_t rows_per_expert, int n_local_experts, int first_expert, int expert_step,
                                const float *x, int64_t x_stride, int x_div, float *y, const int32_t *counts, const int32_t *lists,
                                int n_assign, cudaStream_t s, const Weight *slab2 = nullptr, float *y2 = nullptr);
int32_t moe_combine(float *h, const float *down, const float *sel_w, const int32_t *sel_idx, int hidden, int k, int batch,
                    int first_expert, int expert_step, bool add_residual, cudaStream_t s);

// Sum of the ranks' partial sublayer outputs, in place.  Rank 0's partial carries the residual.
static int32_t reduce_hidden(cmld_engine *e, int32_t B) {
  if (!e->comm) return CMLD_OK;
  CMLD_TRY(comm_allreduce_sum_f32(e->comm, e->h, (int64_t)B * e->cfg.hidden, e->stream));
  e->launches += 1;
  return CMLD_OK;
}

static int ep_size(const cmld_engine *e) { return std::max(1, e->cfg.ep_size); }

// The expert matvecs on the tensor cores (three Q8_K rows per assignment).  Returns CMLD_ERR_UNSUPPORTED, having
// launched nothing, when the shapes or the scratch do not allow it.
static int32_t moe_ffn_step_mma(cmld_engine *e, LayerW &L, int32_t B) {
  const cmld_config &c = e->cfg;
  if (!e->moe_act3_h || L.exps[0].qt != L.exps[1].qt) return CMLD_ERR_UNSUPPORTED;
  const int k = c.n_experts_used, na = B * k;
  const int n_local = c.n_experts / ep_size(e), first = ep_size(e) > 1 ? c.ep_rank : 0, step = ep_size(e);
  const bool pdl = !(c.flags & CMLD_FLAG_NO_PDL);
  // rows per pass: enough for the expected load of an expert (3 rows per assignment), at most 32
  const int expect = 3 * ((na + c.n_experts - 1) / c.n_experts);
  const int nt = std::max(1, std::min(4, (expect * 3 / 2 + 7) / 8));
  const int n_pass = (3 * na + nt * 8 - 1) / (nt * 8);
  GemvJob gu[2] = {{L.exps[0].data, L.exps[0].qt, c.ffn_dim, c.hidden, L.exps[0].stride, e->moe_g3, nullptr, c.ffn_dim},
                   {L.exps[1].data, L.exps[1].qt, c.ffn_dim, c.hidden, L.exps[1].stride, e->moe_u3, nullptr, c.ffn_dim}};
  GemvJob dn[1] = {{L.exps[2].data, L.exps[2].qt, c.hidden, c.ffn_dim, L.exps[2].stride, e->moe_d3, nullptr, c.hidden}};
  const int64_t need_gu = gemv_mma_expert_scratch_floats(gu, 2, nt, n_local, n_pass), need_dn = gemv_mma_expert_scratch_floats(dn, 1, nt, n_local, n_pass);
  if (need_gu < 0 || need_dn < 0 || std::max(need_gu, need_dn) > e->moe_scratch_floats) return CMLD_ERR_UNSUPPORTED;
  CMLD_TRY(moe_route(e->normed, L.router, c.hidden, c.n_experts, k, B, e->moe_sel_idx, e->moe_sel_w, e->moe_counts,
                     e->moe_lists, e->stream, e->moe_pos));
  CMLD_TRY(moe_quant3(e->normed, nullptr, 0, c.hidden, k, na, n_local, first, step, e->moe_cap, e->moe_counts, e->moe_lists,
                      e->moe_act3_h, e->stream));
  e->launches += 3;
  CMLD_TRY(launch_gemv_mma_experts(gu, 2, e->moe_act3_h, nt, n_local, n_pass, e->moe_counts, first, step, e->moe_cap, 3,
                                   e->moe_scratch, e->moe_scratch_floats, e->d_status, e->stream, pdl, &e->launches));
  CMLD_TRY(moe_quant3(e->moe_g3, e->moe_u3, 1, c.ffn_dim, k, na, n_local, first, step, e->moe_cap, e->moe_counts, e->moe_lists,
                      e->moe_act3_f, e->stream));
  CMLD_TRY(launch_gemv_mma_experts(dn, 1, e->moe_act3_f, nt, n_local, n_pass, e->moe_counts, first, step, e->moe_cap, 3,
                                   e->moe_scratch, e->moe_scratch_floats, e->d_status, e->stream, pdl, &e->launches));
  CMLD_TRY(moe_combine3(e->h, e->moe_d3, e->moe_sel_w, e->moe_sel_idx, e->moe_pos, c.hidden, k, B, first, step, e->moe_cap,
                        e->ep == 1 || e->shard_rank == 0, e->stream));
  e->launches += 2;
  if (e->ep > 1) CMLD_TRY(reduce_hidden(e, B));
  return CMLD_OK;
}

// Mixtral FFN on e->normed (f32): route, expert gate/up, SwiGLU, expert down, weighted sum.
static int32_t moe_ffn_step(cmld_engine *e, LayerW &L, int32_t B) {
  const cmld_config &c = e->cfg;
  // Default: the expert matvecs in the CPU path's order (f32 activation x dequantised weight, one accumulator).
  // CMLD_FLAG_TENSOR_BATCH opts into the int8 tensor-core form (three residual Q8_K rows per activation), which
  // reads the weights once for all rows but adds in another order.
  const bool fast = (c.flags & CMLD_FLAG_TENSOR_BATCH) != 0;
  if (fast) {
    const int32_t rc = moe_ffn_step_mma(e, L, B);
    if (rc != CMLD_ERR_UNSUPPORTED) return rc;
  }
  const int k = c.n_experts_used, na = B * k;
  const int n_local = c.n_experts / ep_size(e), first = ep_size(e) > 1 ? c.ep_rank : 0, step = ep_size(e);
  CMLD_TRY(moe_route(e->normed, L.router, c.hidden, c.n_experts, k, B, e->moe_sel_idx, e->moe_sel_w, e->moe_counts,
                     e->moe_lists, e->stream, e->moe_pos));
  const bool pair = !fast && L.exps[0].qt == L.exps[1].qt && L.exps[0].stride == L.exps[1].stride;
  if (pair) {
    // gate and up in one launch: the rows of the few active experts are too few to fill the machine on their own
    CMLD_TRY(moe_expert_gemv_ordered(L.exps[0], c.ffn_dim, n_local, first, step, e->normed, c.hidden, k, e->moe_g, e->moe_counts,
                                     e->moe_lists, na, e->stream, &L.exps[1], e->moe_u));
  } else if (fast) {
    CMLD_TRY(moe_expert_gemv(L.exps[0], c.ffn_dim, n_local, first, step, e->normed, c.hidden, k, e->moe_g, e->moe_counts, e->moe_lists, na, e->stream));
    CMLD_TRY(moe_expert_gemv(L.exps[1], c.ffn_dim, n_local, first, step, e->normed, c.hidden, k, e->moe_u, e->moe_counts, e->moe_lists, na, e->stream));
  } else {
    CMLD_TRY(moe_expert_gemv_ordered(L.exps[0], c.ffn_dim, n_local, first, step, e->normed, c.hidden, k, e->moe_g, e->moe_counts, e->moe_lists, na, e->stream));
    CMLD_TRY(moe_expert_gemv_ordered(L.exps[1], c.ffn_dim, n_local, first, step, e->normed, c.hidden, k, e->moe_u, e->moe_counts, e->moe_lists, na, e->stream));
  }
  NormQuantArgs a{};
  a.x = e->moe_g;
  a.x2 = e->moe_u;
  a.cols = c.ffn_dim;
  a.batch = na;
  a.out = e->moe_act;
  CMLD_TRY(launch_norm_quant(a, e->stream));
  if (fast) CMLD_TRY(moe_expert_gemv(L.exps[2], c.hidden, n_local, first, step, e->moe_act, c.ffn_dim, 1, e->moe_down, e->moe_counts, e->moe_lists, na, e->stream));
  else CMLD_TRY(moe_expert_gemv_ordered(L.exps[2], c.hidden, n_local, first, step, e->moe_act, c.ffn_dim, 1, e->moe_down, e->moe_counts, e->moe_lists, na, e->stream));
  CMLD_TRY(moe_combine(e->h, e->moe_down, e->moe_sel_w, e->moe_sel_idx, c.hidden, k, B, first, step,
                       e->ep == 1 || e->shard_rank == 0, e->stream));
  e->launches += pair ? 6 : 7;
  if (e->ep > 1) CMLD_TRY(reduce_hidden(e, B));
  return CMLD_OK;
}

// [rows][vocab] logits of a vocabulary-sharded engine, assembled on every rank in e->logits_full.
static int32_t gather_logits(cmld_engine *e, int32_t B) {
  CMLD_TRY(comm_allgather_f32(e->comm, e->logits, e->logits_gather, (int64_t)B * e->vocab_local, e->stream));
  CMLD_TRY(launch_gather_permute(e->logits_gather, e->logits_full, e->tp, B, e->vocab_local, e->stream));
  return CMLD_OK;
}

// ---- peer-memory link (tensor-parallel sublayer sums inside the matvec kernels)

static size_t peer_parts_bytes(const cmld_engine *e) { return (size_t)2 * e->tp * kPeerRows * e->cfg.hidden * 4; }
static float *peer_part(const cmld_engine *e, int on_rank, int slot, int src_rank) {
  return reinterpret_cast<float *>(e->peer.region[on_rank]) + ((int64_t)slot * e->tp + src_rank) * kPeerRows * e->cfg.hidden;
}
static uint32_t *peer_flag(const cmld_engine *e, int on_rank, int slot, int src_rank) {
  return reinterpret_cast<uint32_t *>(e->peer.region[on_rank] + peer_parts_bytes(e)) + slot * kMaxPeers + src_rank;
}
static void peer_tx(const cmld_engine *e, int slot, GemvPeer &g) {
  g.tx_n = e->tp;
  for (int p = 0; p < e->tp; ++p) {
    g.tx_part[p] = peer_part(e, p, slot, e->shard_rank);
    g.tx_flag[p] = peer_flag(e, p, slot, e->shard_rank);
  }
  g.tx_epoch = e->peer.local + slot;
  g.tx_ticket = e->peer.local + 2 + slot;
}
static void peer_rx(const cmld_engine *e, int slot, GemvPeer &g) {
  g.rx_n = e->tp;
  g.rx_part = peer_part(e, e->shard_rank, slot, 0);
  g.rx_flag = peer_flag(e, e->shard_rank, slot, 0);
  g.rx_epoch = e->peer.local + slot;
  g.rx_out = e->h;
  g.timeout_ns = e->peer.timeout_ns;
}

// Whether a step of B rows can fold its sublayer sums into the matvec kernels: every matvec of the
// step must go through the staged kernel in a single pass.
static bool peer_step_ok(cmld_engine *e, int32_t B, bool taps) {
  if (!e->peer.ready || e->tp <= 1 || taps || B > kPeerRows || B > kFusedPrologueMaxBatch) return false;
  if (e->cfg.flags & (CMLD_FLAG_EXACT_ORDER | CMLD_FLAG_SPLIT_PROLOGUE | CMLD_FLAG_DIRECT_GEMV | CMLD_FLAG_NCCL_ONLY)) return false;
  auto it = e->peer_fit.find(B);
  if (it != e->peer_fit.end()) return it->second;
  bool ok = e->cfg.hidden % 256 == 0 && e->cfg.hidden <= 8192;
  auto fits = [&](std::initializer_list<const Weight *> ws, bool norm = false) {
    GemvJob jobs[3];
    int n = 0;
    for (const Weight *w : ws) {
      if (!w->data) return false;
      jobs[n++] = GemvJob{w->data, w->qt, w->rows, w->cols, w->stride, nullptr, nullptr, w->rows};
    }
    return gemv_pipe_fit_batch(jobs, n, false, norm) >= B;
  };
  for (const LayerW &L : e->layers) {
    if (!ok) break;
    ok = L.dense_set && !L.moe_set && fits({&L.proj[0], &L.proj[1], &L.proj[2]}, true) && fits({&L.proj[3]}) &&
         fits({&L.proj[4], &L.proj[5]}, true) && fits({&L.proj[6]});
  }
  if (ok && e->has_output) ok = fits({&e->output}, true);
  e->peer_fit[B] = ok;
  return ok;
}

static int32_t engine_step(cmld_engine *e, const StepOpts &o) {
  const cmld_config &c = e->cfg;
  const int32_t B = o.batch;
  const bool sharded = e->tp > 1 || e->ep > 1;
  const bool use_peer = peer_step_ok(e, B, o.taps);
  int pending = -1;  // slot whose partial rows are the not-yet-summed residual stream
  auto take_pending = [&](GemvPeer &g) {
    if (pending >= 0) peer_rx(e, pending, g);
    pending = -1;
  };
  if (sharded && !e->comm)
    return fail(CMLD_ERR_STATE, "this sharded engine has no communicator (cmld_engine_comm_init not called, or aborted after a peer stopped answering)");
  const bool lead = e->shard_rank == 0;  // the rank whose partial sums carry the residual
  if (B < 1 || B > e->max_rows) return fail(CMLD_ERR_INVALID, "step of %d rows exceeds the engine's %d", B, e->max_rows);
  if (o.from_tokens) {
    if (!e->has_embd) return fail(CMLD_ERR_STATE, "token embedding table not set");
    CMLD_TRY(launch_embed_gather(e->token_embd, e->d_tokens, B, e->h, e->stream));
    e->launches += 1;
  }
  const int32_t l_end = o.layer_end < 0 ? c.n_layers : o.layer_end;
  for (int32_t li = o.layer_begin; li < l_end; ++li) {
    LayerW &L = e->layers[li];
    {
      // The three projections share a launch; the matrices of the type whose tiles take longest (Q6_K, then Q8_0)
      // go first, so that a CTA's last round of tiles is made of the quick ones.
      const Proj qkv[3] = {{&L.proj[0], e->q, nullptr, e->q_width},
                           {&L.proj[1], e->k, nullptr, e->kv_width},
                           {&L.proj[2], e->v, nullptr, e->kv_width}};
      auto tile_cost = [](const Weight *w) { return w->qt == CMLD_Q6_K ? 0 : (w->qt == CMLD_Q8_0 ? 1 : 2); };
      int order[3] = {0, 1, 2};
      std::stable_sort(order, order + 3, [&](int x, int y) { return tile_cost(qkv[x].w) < tile_cost(qkv[y].w); });
      const Proj p[3] = {qkv[order[0]], qkv[order[1]], qkv[order[2]]};
      GemvPeer g{};
      take_pending(g);
      // the attention that follows reads this layer's KV rows: have them pulled into L2 meanwhile (every row but
      // the step's own, which the attention kernel appends itself, is final)
      KvPrefetch pf{};
      if (!o.shared_slots && !e->kq8) {
        pf.k = e->kcache + (int64_t)li * e->kv_layer_elems;
        pf.v = e->vcache + (int64_t)li * e->kv_layer_elems;
        pf.positions = e->d_positions;
        pf.slots = e->d_slots;
        pf.n_kv_heads = c.n_kv_heads;
        pf.head_dim = c.head_dim;
        pf.batch = B;
        pf.max_pos = c.max_pos;
      }
      CMLD_TRY(gemv_fused(e, p, 3, B, 1, e->h, nullptr, L.attn_norm, c.hidden, use_peer ? &g : nullptr, false, pf.k ? &pf : nullptr));
    }
    {
      // Attention.  Default: the reference-order cluster kernel (the CPU path's bits); contexts or shapes it
      // does not take, and CMLD_FLAG_EXACT_ORDER, use the plain reference-order kernel; CMLD_FLAG_FAST_ORDER
      // opts into the split-range (flash-decoding) kernel, whose sums are trees.
      if (e->kq8) {
        // Q8_0 KV cache: append (RoPE + block quantisation) and attention over the blocks, in the CPU lane's order
        RopeKvArgs r{};
        r.q = e->q;
        r.k = e->k;
        r.v = e->v;
        r.cos_tab = o.rope_by_position ? e->cos_all : e->cos_step;
        r.sin_tab = o.rope_by_position ? e->sin_all : e->sin_step;
        r.index_by_position = o.rope_by_position;
        r.positions = e->d_positions;
        r.slots = e->d_slots;
        r.n_heads = c.n_heads;
        r.n_kv_heads = c.n_kv_heads;
        r.head_dim = c.head_dim;
        r.rope_dim = c.rope_dim;
        r.split_half = c.split_half_pairing;
        r.batch = B;
        r.max_pos = c.max_pos;
        r.q_stride = e->q_width;
        r.kv_stride = e->kv_width;
        uint8_t *kq = e->kq8 + (int64_t)li * e->kv_q8_bytes, *vq = e->vq8 + (int64_t)li * e->kv_q8_bytes;
        CMLD_TRY(launch_rope_kv_q8(r, kq, vq, e->stream));
        AttnArgs a{};
        a.q = e->q;
        a.positions = e->d_positions;
        a.slots = e->d_slots;
        a.n_heads = c.n_heads;
        a.n_kv_heads = c.n_kv_heads;
        a.head_dim = c.head_dim;
        a.batch = B;
        a.max_pos = c.max_pos;
        a.scale = o.scale;
        a.out = e->attn;
        a.q_stride = e->q_width;
        a.tree_mask = o.tree_mask;
        CMLD_TRY(launch_attention_q8(a, kq, vq, e->stream));
        e->launches += 2;
      } else {
      const bool fast = (c.flags & CMLD_FLAG_FAST_ORDER) && !(c.flags & CMLD_FLAG_EXACT_ORDER) && !o.tree_mask;
      // steps of three rows and more: one CTA per (row, KV head) instead of a cluster of eight (same bits)
      const bool rows = !fast && !(c.flags & CMLD_FLAG_EXACT_ORDER) && B >= 3 && o.attn_cap > 0 && !o.tree_mask &&
                        attention_rows_fits(c.n_heads, c.n_kv_heads, c.head_dim, o.attn_cap);
      const bool ordered = !rows && !fast && !(c.flags & CMLD_FLAG_EXACT_ORDER) && o.attn_cap > 0 && !o.tree_mask &&
                           attention_ordered_fits(c.n_heads, c.n_kv_heads, c.head_dim, o.attn_cap);
      const bool fuse = !o.shared_slots && (fast || ordered);
      if (!fuse) {
        RopeKvArgs r{};
        r.q = e->q;
        r.k = e->k;
        r.v = e->v;
        r.cos_tab = o.rope_by_position ? e->cos_all : e->cos_step;
        r.sin_tab = o.rope_by_position ? e->sin_all : e->sin_step;
        r.index_by_position = o.rope_by_position;
        r.positions = e->d_positions;
        r.slots = e->d_slots;
        r.k_cache = e->kcache + (int64_t)li * e->kv_layer_elems;
        r.v_cache = e->vcache + (int64_t)li * e->kv_layer_elems;
        r.n_heads = c.n_heads;
        r.n_kv_heads = c.n_kv_heads;
        r.head_dim = c.head_dim;
        r.rope_dim = c.rope_dim;
        r.split_half = c.split_half_pairing;
        r.batch = B;
        r.max_pos = c.max_pos;
        r.q_stride = e->q_width;
        r.kv_stride = e->kv_width;
        CMLD_TRY(launch_rope_kv(r, e->stream));
        e->launches += 1;
      }
      AttnArgs a{};
      a.q = e->q;
      a.k_cache = e->kcache + (int64_t)li * e->kv_layer_elems;
      a.v_cache = e->vcache + (int64_t)li * e->kv_layer_elems;
      a.positions = e->d_positions;
      a.slots = e->d_slots;
      a.n_heads = c.n_heads;
      a.n_kv_heads = c.n_kv_heads;
      a.head_dim = c.head_dim;
      a.batch = B;
      // enough CTAs to fill the machine about twice, and no more: with many rows each (row, kv head) pair
      // needs few ranges, and a range that is too short is all fixed cost
      a.n_splits = std::max(1, std::min(e->n_splits, (2 * e->sm_count + B * c.n_kv_heads - 1) / (B * c.n_kv_heads)));
      a.max_pos = c.max_pos;
      a.scale = o.scale;
      a.part = e->attn_part;
      a.tickets = e->attn_tickets;
      a.out = e->attn;
      a.q_stride = e->q_width;
      a.fuse_rope = fuse ? 1 : 0;  // RoPE(q), RoPE(k) and the f16 KV append inside the attention kernel
      a.rope_dim = c.rope_dim;
      a.split_half = c.split_half_pairing;
      a.index_by_position = o.rope_by_position;
      a.k_new = e->k;
      a.v_new = e->v;
      a.kv_stride = e->kv_width;
      a.cos_tab = o.rope_by_position ? e->cos_all : e->cos_step;
      a.sin_tab = o.rope_by_position ? e->sin_all : e->sin_step;
      a.pdl = !(c.flags & CMLD_FLAG_NO_PDL);
      a.cluster = o.attn_cluster && fast ? 1 : 0;
      a.phase_ns = e->attn_phases;
      a.tree_mask = o.tree_mask;
      a.tree_base = o.tree_base;
      a.tree_words = o.tree_words;
      if (rows) CMLD_TRY(launch_attention_rows(a, o.attn_cap, e->stream));
      else if (ordered) CMLD_TRY(launch_attention_ordered(a, o.attn_cap, e->stream));
      else if (fast) CMLD_TRY(launch_attention(a, e->stream));
      else CMLD_TRY(launch_attention_exact(a, e->stream));
      e->launches += 1;
      }
    }
    {
      const Proj p[1] = {{&L.proj[3], e->h, (e->tp == 1 || lead) ? e->h : nullptr, c.hidden}};
      if (use_peer) {
        GemvPeer g{};
        peer_tx(e, 0, g);
        CMLD_TRY(gemv_fused(e, p, 1, B, 2, e->attn, nullptr, nullptr, e->q_width, &g));
        pending = 0;
      } else {
        CMLD_TRY(gemv_fused(e, p, 1, B, 2, e->attn, nullptr, nullptr, e->q_width));
        if (e->tp > 1) CMLD_TRY(reduce_hidden(e, B));
      }
    }
    if (L.moe_set) {
      CMLD_TRY(run_norm_quant(e, e->h, nullptr, L.ffn_norm, c.hidden, B, e->normed, false, false));
      CMLD_TRY(moe_ffn_step(e, L, B));
    } else {
      const Proj p[2] = {{&L.proj[4], e->gate, nullptr, c.ffn_dim}, {&L.proj[5], e->up, nullptr, c.ffn_dim}};
      GemvPeer g{};
      take_pending(g);
      // gate and up of equal type: the staged kernel pairs their tiles and writes SwiGLU(gate, up) itself,
      // so the down projection's operand is a plain quantisation of one vector
      bool pair = !(c.flags & (CMLD_FLAG_EXACT_ORDER | CMLD_FLAG_DIRECT_GEMV)) && L.proj[4].qt == L.proj[5].qt && B < mma_min_rows(e) && B < tc5_min_rows(e);
      if (pair) {
        const GemvJob pj[2] = {{L.proj[4].data, L.proj[4].qt, L.proj[4].rows, L.proj[4].cols, L.proj[4].stride, nullptr, nullptr, 0},
                               {L.proj[5].data, L.proj[5].qt, L.proj[5].rows, L.proj[5].cols, L.proj[5].stride, nullptr, nullptr, 0}};
        pair = gemv_pipe_fit_batch(pj, 2, true, true) >= 1;
      }
      CMLD_TRY(gemv_fused(e, p, 2, B, 1, e->h, nullptr, L.ffn_norm, c.hidden, use_peer ? &g : nullptr, pair));
      const Proj pd[1] = {{&L.proj[6], e->h, (e->tp == 1 || lead) ? e->h : nullptr, c.hidden}};
      const int dmode = pair ? 2 : 3;  // operand: the SwiGLU vector already in e->gate, or SwiGLU(gate, up) to be formed
      if (use_peer) {
        GemvPeer gd{};
        peer_tx(e, 1, gd);
        CMLD_TRY(gemv_fused(e, pd, 1, B, dmode, e->gate, pair ? nullptr : e->up, nullptr, c.ffn_dim, &gd));
        pending = 1;
      } else {
        CMLD_TRY(gemv_fused(e, pd, 1, B, dmode, e->gate, pair ? nullptr : e->up, nullptr, c.ffn_dim));
        if (e->tp > 1) CMLD_TRY(reduce_hidden(e, B));
      }
    }
    if (o.taps) {
      CMLD_CUDA(cudaMemcpyAsync(e->taps + (int64_t)li * e->max_rows * c.hidden, e->h, (size_t)B * c.hidden * 4,
                                cudaMemcpyDeviceToDevice, e->stream));
    }
  }
  if (o.logits) {
    if (!e->has_output) return fail(CMLD_ERR_STATE, "output weights not set");
    const Proj p[1] = {{&e->output, e->logits, nullptr, e->vocab_local}};
    GemvPeer g{};
    take_pending(g);
    CMLD_TRY(gemv_fused(e, p, 1, B, 1, e->h, nullptr, e->final_norm, c.hidden, use_peer ? &g : nullptr));
    if (o.argmax && e->tp == 1) {
      CMLD_TRY(launch_argmax(e->logits, c.vocab, B, e->am_val, e->am_idx, e->am_ticket, e->out_idx,
                             o.feed_back ? e->d_tokens : nullptr, e->d_positions, e->d_history, e->stream));
      e->launches += 1;
    } else if (o.argmax) {
      // vocabulary shard: local best as a packed key, max over the ranks, then the feedback
      CMLD_TRY(launch_argmax(e->logits, e->vocab_local, B, e->am_val, e->am_idx, e->am_ticket, e->out_idx, nullptr,
                             e->d_positions, e->d_history, e->stream, e->am_keys, e->shard_rank * e->vocab_local));
      CMLD_TRY(comm_allreduce_max_u64(e->comm, e->am_keys, B, e->stream));
      CMLD_TRY(launch_argmax_finish(e->am_keys, B, e->out_idx, o.feed_back ? e->d_tokens : nullptr, e->d_positions,
                                    e->d_history, e->am_ticket, e->stream));
      e->launches += 3;
    }
  }
  if (pending >= 0) {  // the step ends on a sublayer: sum its partial rows into h
    GemvPeer g{};
    take_pending(g);
    CMLD_TRY(launch_peer_reduce(g, B, c.hidden, e->d_status, !(c.flags & CMLD_FLAG_NO_PDL), e->stream));
    e->launches += 1;
  }
  return CMLD_OK;
}

// A step through a CUDA graph when possible: one graph launch replaces ~200 kernel launches, and
// the programmatic-dependent-launch edges between the matvec kernels are kept inside the graph.
static int32_t run_step(cmld_engine *e, const StepOpts &o) {
  if ((e->cfg.flags & CMLD_FLAG_NO_GRAPH) || e->graphs_off || o.tree_mask) return engine_step(e, o);
  uint32_t bits = (o.from_tokens ? 1u : 0u) | (o.rope_by_position ? 2u : 0u) | (o.logits ? 4u : 0u) | (o.argmax ? 8u : 0u) |
                  (o.feed_back ? 16u : 0u) | (o.taps ? 32u : 0u) | (o.shared_slots ? 64u : 0u) | (o.attn_cluster ? 128u : 0u) | ((uint32_t)(o.layer_begin & 0xfff) << 8) | ((uint32_t)((o.layer_end + 1) & 0xfff) << 20);
  uint32_t scale_bits;
  memcpy(&scale_bits, &o.scale, 4);
  auto &g = e->graphs[std::make_tuple(o.batch | (o.attn_cap << 8), bits, scale_bits)];
  if (g.exec) {
    CMLD_CUDA(cudaGraphLaunch(g.exec, e->stream));
    e->launches += g.launches;
    return CMLD_OK;
  }
  if (g.uses++ == 0) return engine_step(e, o);
  const int64_t before = e->launches;
  if (cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    e->graphs_off = true;
    return engine_step(e, o);
  }
  const int32_t rc = engine_step(e, o);
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
  const int64_t n = e->launches - before;
  e->launches = before;
  if (rc == CMLD_OK && ce == cudaSuccess && graph && cudaGraphInstantiate(&g.exec, graph, 0) == cudaSuccess) {
    cudaGraphDestroy(graph);
    g.launches = n;
    CMLD_CUDA(cudaGraphLaunch(g.exec, e->stream));
    e->launches += n;
    return CMLD_OK;
  }
  // capture or instantiation failed: nothing ran; keep to plain launches from now on
  if (graph) cudaGraphDestroy(graph);
  cudaGetLastError();
  g.exec = nullptr;
  e->graphs_off = true;
  if (rc != CMLD_OK) return rc;
  return engine_step(e, o);
}

static int32_t require_weights(const cmld_engine *e, bool need_output) {
  for (size_t i = 0; i < e->layers.size(); ++i) {
    const LayerW &L = e->layers[i];
    if (!L.dense_set) return fail(CMLD_ERR_STATE, "layer %zu has no weights", i);
    if (e->cfg.n_experts > 0 && !L.moe_set) return fail(CMLD_ERR_STATE, "layer %zu has no expert weights", i);
  }
  if (need_output && !e->has_output) return fail(CMLD_ERR_STATE, "output weights not set");
  return CMLD_OK;
}

// Attention ranges as a thread-block cluster: worth it while a range (1/8 of the context) is short and the rows
// are few; beyond that the 37-way split through global memory, or no split at all for many rows, is better.
// The rule does not depend on the row count up to 8 rows, so that a step of <= 8 rows keeps giving the bits of
// the same rows stepped one by one (as long as all of them are on one side of the context threshold).
static bool use_attn_cluster(int32_t rows, int64_t max_position) { return rows <= 8 && max_position < 2048; }

// Bound on the context length handed to the reference-order attention kernel: the smallest of a few buckets
// that holds every row's context (a step graph is kept per bucket), 0 beyond the largest.
static int32_t attn_cap_for(int64_t max_position) {
  for (int32_t cap : {1024, 2048, 4096, 8192})
    if (max_position < cap) return cap;
  return 0;
}

// Rows of one step: tokens (or none), positions and KV slots to the device.
static int32_t stage_rows(cmld_engine *e, int32_t n, const int32_t *tokens, const int32_t *positions, const int32_t *slots) {
  if (tokens) CMLD_CUDA(cudaMemcpyAsync(e->d_tokens, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->d_positions, positions, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->d_slots, slots, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
  return CMLD_OK;
}

// Sharded engines wait for their device work here, with a bound, BEFORE any device-to-host copy: a
// copy into pageable host memory blocks the calling thread until the stream has drained, and a
// collective whose peer went away never drains by itself.  No-op for an unsharded engine.
static int32_t settle(cmld_engine *e) {
  if (!e->comm) return CMLD_OK;
  static const int64_t limit_ms = [] {
    const char *v = getenv("CMLD_COMM_TIMEOUT_MS");
    const long long n = v ? atoll(v) : 0;
    return (int64_t)(n > 0 ? n : 120000);
  }();
  return comm_wait_stream(&e->comm, e->stream, limit_ms, [](void *ctx) {
    // once the aborted collective has let the stream drain: release the graphs that captured the
    // communicator's collectives, or NCCL's teardown would wait for them for ever
    cmld_engine *eng = static_cast<cmld_engine *>(ctx);
    for (auto &kv : eng->graphs)
      if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    eng->graphs.clear();
  }, e);
}

static int32_t finish(cmld_engine *e, const char *what) {
  CMLD_TRY(settle(e));
  int32_t st = 0;
  cudaError_t ce = cudaMemcpyAsync(&st, e->d_status, 4, cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail(CMLD_ERR_CUDA, "%s: %s", what, cudaGetErrorString(ce));
  if (st != 0) {
    cudaMemsetAsync(e->d_status, 0, 4, e->stream);
    return fail(st, "%s: a bounded device-side wait gave up (status %d); results of this call are invalid", what, st);
  }
  return CMLD_OK;
}

// One sequence-0 row fed by an embedding vector: the forward_token family.
static int32_t forward_embedding_rows(cmld_engine *e, const float *embeddings, const float *cosv, const float *sinv,
                                      int64_t position0, int32_t n_rows, float scale, bool logits, bool argmax, bool taps,
                                      int32_t layer_begin = 0, int32_t layer_end = -1) {
  const cmld_config &c = e->cfg;
  if (!embeddings || !cosv || !sinv) return fail(CMLD_ERR_INVALID, "embedding / cos / sin pointer is null");
  if (position0 < 0 || position0 + n_rows > c.max_pos)
    return fail(CMLD_ERR_STATE, "positions %lld..%lld exceed max_pos %d", (long long)position0,
                (long long)(position0 + n_rows - 1), c.max_pos);
  CMLD_TRY(require_weights(e, logits));
  const int half = c.rope_dim / 2;
  CMLD_CUDA(cudaMemcpyAsync(e->h, embeddings, (size_t)n_rows * c.hidden * 4, cudaMemcpyDefault, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->cos_step, cosv, (size_t)n_rows * half * 4, cudaMemcpyDefault, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->sin_step, sinv, (size_t)n_rows * half * 4, cudaMemcpyDefault, e->stream));
  std::vector<int32_t> pos(n_rows), slots(n_rows, 0);
  for (int i = 0; i < n_rows; ++i) pos[i] = (int32_t)(position0 + i);
  CMLD_TRY(stage_rows(e, n_rows, nullptr, pos.data(), slots.data()));
  StepOpts o;
  o.batch = n_rows;
  o.shared_slots = n_rows > 1;
  o.from_tokens = false;
  o.rope_by_position = false;
  o.scale = scale;
  o.logits = logits;
  o.argmax = argmax;
  o.taps = taps;
  o.layer_begin = layer_begin;
  o.layer_end = layer_end;
  o.attn_cluster = use_attn_cluster(n_rows, position0 + n_rows - 1);
  o.attn_cap = attn_cap_for(position0 + n_rows - 1);
  return run_step(e, o);
}

}  // namespace cmld

// ====================================================================== C ABI

extern "C" {

const char *cmld_last_error(void) { return cmld::last_error(); }
const char *cmld_version(void) { return "camelid_b200 0.1 (sm_100a)"; }

int32_t cmld_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int32_t cmld_set_device(int32_t device) {
  CMLD_CUDA(cudaSetDevice(device));
  return CMLD_OK;
}

int32_t cmld_malloc(void **dev_ptr, uint64_t nbytes) {
  if (!dev_ptr) return fail(CMLD_ERR_INVALID, "null out pointer");
  CMLD_CUDA(cudaMalloc(dev_ptr, (size_t)std::max<uint64_t>(nbytes, 1)));
  return CMLD_OK;
}
int32_t cmld_free(void *dev_ptr) {
  if (dev_ptr) CMLD_CUDA(cudaFree(dev_ptr));
  return CMLD_OK;
}
int32_t cmld_memcpy_h2d(void *dst_dev, const void *src_host, uint64_t nbytes) {
  CMLD_CUDA(cudaMemcpy(dst_dev, src_host, (size_t)nbytes, cudaMemcpyHostToDevice));
  return CMLD_OK;
}
int32_t cmld_memcpy_d2h(void *dst_host, const void *src_dev, uint64_t nbytes) {
  CMLD_CUDA(cudaMemcpy(dst_host, src_dev, (size_t)nbytes, cudaMemcpyDeviceToHost));
  return CMLD_OK;
}
int32_t cmld_memset(void *dst_dev, int32_t value, uint64_t nbytes) {
  CMLD_CUDA(cudaMemset(dst_dev, value, (size_t)nbytes));
  return CMLD_OK;
}
int32_t cmld_device_synchronize(void) {
  CMLD_CUDA(cudaDeviceSynchronize());
  return CMLD_OK;
}
int32_t cmld_mem_info(uint64_t *free_bytes, uint64_t *total_bytes) {
  size_t f = 0, t = 0;
  CMLD_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = f;
  if (total_bytes) *total_bytes = t;
  return CMLD_OK;
}

// The dimensions one rank of a tensor-parallel group holds.  Heads split by kv group, so that a query
// head and its kv head stay on one rank; o and down split by columns on 256-value boundaries (a whole
// K-quant superblock); the vocabulary splits by rows.
static int32_t shard_config(const cmld_config &full, cmld_config &local, int32_t &tp, int32_t &ep, int32_t &rank) {
  local = full;
  tp = std::max(1, full.tp_size);
  ep = std::max(1, full.ep_size);
  rank = 0;
  if (tp > 1 && ep > 1) return fail(CMLD_ERR_UNSUPPORTED, "tensor and expert parallelism cannot be combined");
  if (tp > 1) {
    if (full.n_experts > 0) return fail(CMLD_ERR_UNSUPPORTED, "a Mixtral-shaped model shards by experts (ep_size), not tp_size");
    if (full.tp_rank < 0 || full.tp_rank >= tp) return fail(CMLD_ERR_INVALID, "tp_rank %d outside 0..%d", full.tp_rank, tp - 1);
    if (full.n_kv_heads % tp || full.vocab % tp || full.ffn_dim % (tp * 256) ||
        ((full.n_heads / tp) * full.head_dim) % 256)
      return fail(CMLD_ERR_SHAPE, "tp_size %d does not divide kv heads %d / vocab %d, or leaves ffn %d / attention width %d "
                  "shares that are not multiples of 256", tp, full.n_kv_heads, full.vocab, full.ffn_dim, full.n_heads * full.head_dim);
    local.n_heads = full.n_heads / tp;
    local.n_kv_heads = full.n_kv_heads / tp;
    local.ffn_dim = full.ffn_dim / tp;
    rank = full.tp_rank;
  }
  if (ep > 1) {
    if (full.n_experts <= 0 || full.n_experts % ep) return fail(CMLD_ERR_SHAPE, "ep_size %d does not divide %d experts", ep, full.n_experts);
    if (full.ep_rank < 0 || full.ep_rank >= ep) return fail(CMLD_ERR_INVALID, "ep_rank %d outside 0..%d", full.ep_rank, ep - 1);
    rank = full.ep_rank;
  }
  return CMLD_OK;
}

int32_t cmld_engine_create(const cmld_config *cfg_in, cmld_engine **out) {
  if (!cfg_in || !out) return fail(CMLD_ERR_INVALID, "config or out pointer is null");
  *out = nullptr;
  CMLD_TRY(validate_config(*cfg_in));
  cmld_config local{};
  int32_t tp = 1, ep = 1, shard_rank = 0;
  CMLD_TRY(shard_config(*cfg_in, local, tp, ep, shard_rank));
  CMLD_TRY(validate_config(local));
  const cmld_config *cfg = &local;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    return fail(CMLD_ERR_CUDA, "no CUDA device: this engine has no CPU path");
  }
  int dev = cfg->device;
  if (dev < 0) CMLD_CUDA(cudaGetDevice(&dev));
  if (dev >= ndev) return fail(CMLD_ERR_INVALID, "device %d out of range (%d present)", dev, ndev);
  cudaDeviceProp prop{};
  CMLD_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) return fail(CMLD_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
  // capacity check (the reference sizes VRAM in build_resident_cuda_engine, src/inference.rs:16455-16720)
  const int seqs = std::max(1, cfg->max_seqs);
  const double kv_bytes = 2.0 * 2.0 * cfg->n_layers * seqs * (double)cfg->n_kv_heads * cfg->max_pos * cfg->head_dim;
  DeviceGuard guard(dev);
  if (!guard.ok) return fail(CMLD_ERR_CUDA, "cannot select CUDA device %d", dev);
  size_t free_b = 0, total_b = 0;
  CMLD_CUDA(cudaMemGetInfo(&free_b, &total_b));
  if (kv_bytes > 0.95 * (double)free_b)
    return fail(CMLD_ERR_OOM, "KV cache of %.1f GiB does not fit in %.1f GiB free", kv_bytes / (1 << 30), (double)free_b / (1 << 30));
  cmld_engine *e = new cmld_engine();
  e->cfg = local;
  e->full = *cfg_in;
  e->tp = tp;
  e->ep = ep;
  e->shard_rank = shard_rank;
  e->vocab_local = local.vocab / tp;
  e->device = dev;
  int32_t rc = engine_init(e);
  if (rc != CMLD_OK) {
    engine_free(e);
    delete e;
    return rc;
  }
  *out = e;
  return CMLD_OK;
}

int32_t cmld_engine_destroy(cmld_engine *e) {
  if (!e) return CMLD_OK;
  DeviceGuard guard(e->device);
  cudaStreamSynchronize(e->stream);
  engine_free(e);
  delete e;
  return CMLD_OK;
}

// Maps every rank's slot region into this process (CUDA IPC over NVLink peer access).  Collective.
// When any rank cannot map any other (no peer access, ranks sharing a process, IPC unavailable) all
// ranks agree to keep the NCCL path; that is not an error.
static int32_t peer_link_open(cmld_engine *e) {
  cmld_engine::PeerLink &L = e->peer;
  const int me = e->shard_rank, n = e->tp;
  if (n > kMaxPeers) return CMLD_OK;
  const size_t bytes = peer_parts_bytes(e) + 2 * kMaxPeers * sizeof(uint32_t);
  void *own = nullptr;
  CMLD_CUDA(cudaMalloc(&own, bytes));
  L.region[me] = static_cast<uint8_t *>(own);
  CMLD_CUDA(cudaMemsetAsync(own, 0, bytes, e->stream));
  CMLD_TRY(dev_alloc(e, &L.local, 4));
  // exchange the IPC handles through the communicator (64 bytes per rank)
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t mine{};
  bool ok = cudaIpcGetMemHandle(&mine, own) == cudaSuccess;
  if (!ok) cudaGetLastError();
  float *send = nullptr, *recv = nullptr;
  CMLD_TRY(dev_alloc(e, &send, 16));
  CMLD_TRY(dev_alloc(e, &recv, 16 * n));
  CMLD_CUDA(cudaMemcpyAsync(send, &mine, 64, cudaMemcpyHostToDevice, e->stream));
  CMLD_TRY(comm_allgather_f32(e->comm, send, recv, 16, e->stream));
  std::vector<cudaIpcMemHandle_t> all(n);
  CMLD_CUDA(cudaMemcpyAsync(all.data(), recv, (size_t)64 * n, cudaMemcpyDeviceToHost, e->stream));
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  for (int p = 0; p < n && ok; ++p) {
    if (p == me) continue;
    void *ptr = nullptr;
    if (cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
    } else {
      L.region[p] = static_cast<uint8_t *>(ptr);
    }
  }
  // agree: one rank that failed sends everybody to the NCCL path
  const unsigned long long bad = ok ? 0ull : 1ull;
  CMLD_CUDA(cudaMemcpyAsync(e->am_keys, &bad, 8, cudaMemcpyHostToDevice, e->stream));
  CMLD_TRY(comm_allreduce_max_u64(e->comm, e->am_keys, 1, e->stream));
  unsigned long long any_bad = 1;
  CMLD_CUDA(cudaMemcpyAsync(&any_bad, e->am_keys, 8, cudaMemcpyDeviceToHost, e->stream));
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  if (any_bad) {
    peer_link_close(e);
    return CMLD_OK;
  }
  const char *v = getenv("CMLD_COMM_TIMEOUT_MS");
  const long long ms = v ? atoll(v) : 0;
  L.timeout_ns = (unsigned long long)(ms > 0 ? ms : 20000) * 1000000ull;
  L.ready = true;
  return CMLD_OK;
}

int32_t cmld_comm_unique_id(uint8_t out[128]) {
  if (!out) return fail(CMLD_ERR_INVALID, "null out pointer");
  return comm_unique_id(out);
}

int32_t cmld_engine_comm_init(cmld_engine *e, const uint8_t id[128], int32_t rank, int32_t world) {
  CMLD_ENGINE_ENTER(e);
  if (!id) return fail(CMLD_ERR_INVALID, "null communicator id");
  const int32_t want = e->tp > 1 ? e->tp : e->ep;
  if (want <= 1) return fail(CMLD_ERR_STATE, "this engine is not sharded (tp_size and ep_size are 1)");
  if (world != want || rank != e->shard_rank)
    return fail(CMLD_ERR_INVALID, "communicator rank %d of %d does not match the engine's shard %d of %d", rank, world, e->shard_rank, want);
  if (e->comm) return fail(CMLD_ERR_STATE, "communicator already set");
  CMLD_TRY(comm_init(&e->comm, id, rank, world));
  // one small all-reduce now, so that the connections to the peers are made inside this collective
  // call and not inside the first step
  CMLD_CUDA(cudaMemsetAsync(e->am_keys, 0, 8, e->stream));
  CMLD_TRY(comm_allreduce_max_u64(e->comm, e->am_keys, 1, e->stream));
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  if (e->tp > 1 && !(e->cfg.flags & CMLD_FLAG_NCCL_ONLY)) CMLD_TRY(peer_link_open(e));
  return CMLD_OK;
}

int32_t cmld_engine_set_layer(cmld_engine *e, int32_t layer, const cmld_tensor projs[7], const float *attn_norm,
                              const float *ffn_norm) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  const cmld_config &c = e->cfg;
  if (layer < 0 || layer >= c.n_layers) return fail(CMLD_ERR_INVALID, "set_layer: layer %d out of range", layer);
  if (!projs) return fail(CMLD_ERR_INVALID, "set_layer: projections are null");
  LayerW &L = e->layers[layer];
  const int64_t shapes[7][2] = {{e->q_width, c.hidden},  {e->kv_width, c.hidden}, {e->kv_width, c.hidden}, {c.hidden, e->q_width},
                                {c.ffn_dim, c.hidden},   {c.ffn_dim, c.hidden},   {c.hidden, c.ffn_dim}};
  static const char *names[7] = {"q", "k", "v", "o", "gate", "up", "down"};
  for (int i = 0; i < 7; ++i) {
    if (i >= 4 && c.n_experts > 0 && !projs[i].data) continue;  // MoE layer: dense FFN absent
    int32_t rc = weight_upload(L.proj[i], projs[i].qtype, shapes[i][0], shapes[i][1], projs[i].data, projs[i].nbytes, e->stream);
    if (rc != CMLD_OK) {
      std::string msg = cmld_last_error();
      return fail(rc, "set_layer(%d).%s: %s", layer, names[i], msg.c_str());
    }
    if (L.proj[i].qt == CMLD_F32) return fail(CMLD_ERR_UNSUPPORTED, "set_layer(%d).%s: f32 projections are not supported", layer, names[i]);
  }
  CMLD_TRY(upload_f32(&L.attn_norm, attn_norm, c.hidden, e->stream));
  CMLD_TRY(upload_f32(&L.ffn_norm, ffn_norm, c.hidden, e->stream));
  L.dense_set = true;
  return CMLD_OK;
}

int32_t cmld_engine_set_layer_moe(cmld_engine *e, int32_t layer, const float *router, const cmld_tensor *gate_exps,
                                  const cmld_tensor *up_exps, const cmld_tensor *down_exps) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  const cmld_config &c = e->cfg;
  if (c.n_experts <= 0) return fail(CMLD_ERR_STATE, "set_layer_moe: engine was created without experts");
  if (layer < 0 || layer >= c.n_layers) return fail(CMLD_ERR_INVALID, "set_layer_moe: layer %d out of range", layer);
  if (!router || !gate_exps || !up_exps || !down_exps) return fail(CMLD_ERR_INVALID, "set_layer_moe: null tensor");
  if (c.n_experts % ep_size(e)) return fail(CMLD_ERR_SHAPE, "n_experts %d not divisible by ep_size %d", c.n_experts, ep_size(e));
  if (c.hidden % 256 || c.ffn_dim % 256) return fail(CMLD_ERR_SHAPE, "expert matrices need hidden and ffn_dim to be multiples of 256");
  LayerW &L = e->layers[layer];
  const int64_t n_local = c.n_experts / ep_size(e);
  const cmld_tensor *ts[3] = {gate_exps, up_exps, down_exps};
  const int64_t shapes[3][2] = {{n_local * c.ffn_dim, c.hidden}, {n_local * c.ffn_dim, c.hidden}, {n_local * c.hidden, c.ffn_dim}};
  for (int i = 0; i < 3; ++i) {
    if (ts[i]->qtype != CMLD_Q4_K && ts[i]->qtype != CMLD_Q6_K)
      return fail(CMLD_ERR_UNSUPPORTED, "set_layer_moe: expert tensors must be Q4_K or Q6_K (got type %d)", ts[i]->qtype);
    CMLD_TRY(weight_upload(L.exps[i], ts[i]->qtype, shapes[i][0], shapes[i][1], ts[i]->data, ts[i]->nbytes, e->stream));
  }
  CMLD_TRY(upload_f32(&L.router, router, (int64_t)c.n_experts * c.hidden, e->stream));
  L.moe_set = true;
  return CMLD_OK;
}

int32_t cmld_engine_set_output(cmld_engine *e, const float *final_norm, const cmld_tensor *output) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  if (!output) return fail(CMLD_ERR_INVALID, "set_output: tensor is null");
  CMLD_TRY(weight_upload(e->output, output->qtype, e->vocab_local, e->cfg.hidden, output->data, output->nbytes, e->stream));
  if (e->output.qt == CMLD_F32) return fail(CMLD_ERR_UNSUPPORTED, "set_output: f32 output weights are not supported");
  CMLD_TRY(upload_f32(&e->final_norm, final_norm, e->cfg.hidden, e->stream));
  e->has_output = true;
  return CMLD_OK;
}

int32_t cmld_engine_set_token_embd(cmld_engine *e, const cmld_tensor *t) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  if (!t) return fail(CMLD_ERR_INVALID, "set_token_embd: tensor is null");
  CMLD_TRY(weight_upload(e->token_embd, t->qtype, e->cfg.vocab, e->cfg.hidden, t->data, t->nbytes, e->stream));
  e->has_embd = true;
  return CMLD_OK;
}

static int32_t adopt(Weight &dst, cmld_weight *src, int64_t rows, int64_t cols, const char *what, bool allow_f32 = false) {
  if (src->rows != rows || src->cols != cols)
    return fail(CMLD_ERR_SHAPE, "%s: weight is %lld x %lld, expected %lld x %lld", what, (long long)src->rows, (long long)src->cols,
                (long long)rows, (long long)cols);
  if (src->qt == CMLD_F32 && !allow_f32) return fail(CMLD_ERR_UNSUPPORTED, "%s: f32 weights are not supported here", what);
  {
    // the matrix must live on the engine's GPU: a kernel reading another GPU's memory without peer
    // access would fault
    cudaPointerAttributes pa{};
    int cur = -1;
    if (cudaPointerGetAttributes(&pa, src->data) != cudaSuccess || cudaGetDevice(&cur) != cudaSuccess) {
      cudaGetLastError();
      return fail(CMLD_ERR_CUDA, "%s: cannot query where the weight lives", what);
    }
    if (pa.type != cudaMemoryTypeDevice || pa.device != cur)
      return fail(CMLD_ERR_INVALID, "%s: weight lives on device %d, the engine on device %d (cmld_set_device before making weights)",
                  what, pa.device, cur);
  }
  weight_free(dst);
  dst = *src;
  src->data = nullptr;
  delete src;
  return CMLD_OK;
}

int32_t cmld_engine_adopt_layer(cmld_engine *e, int32_t layer, cmld_weight *const projs[7], const float *attn_norm,
                                const float *ffn_norm) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  const cmld_config &c = e->cfg;
  if (layer < 0 || layer >= c.n_layers) return fail(CMLD_ERR_INVALID, "adopt_layer: layer %d out of range", layer);
  if (!projs) return fail(CMLD_ERR_INVALID, "adopt_layer: projections are null");
  LayerW &L = e->layers[layer];
  const int64_t shapes[7][2] = {{e->q_width, c.hidden},  {e->kv_width, c.hidden}, {e->kv_width, c.hidden}, {c.hidden, e->q_width},
                                {c.ffn_dim, c.hidden},   {c.ffn_dim, c.hidden},   {c.hidden, c.ffn_dim}};
  for (int i = 0; i < 7; ++i)  // validate everything before consuming anything
    if (projs[i] && (projs[i]->rows != shapes[i][0] || projs[i]->cols != shapes[i][1] || projs[i]->qt == CMLD_F32))
      return fail(CMLD_ERR_SHAPE, "adopt_layer(%d): projection %d has the wrong shape or type", layer, i);
  for (int i = 0; i < 7; ++i)
    if (projs[i]) CMLD_TRY(adopt(L.proj[i], projs[i], shapes[i][0], shapes[i][1], "adopt_layer"));
  CMLD_TRY(upload_f32(&L.attn_norm, attn_norm, c.hidden, e->stream));
  CMLD_TRY(upload_f32(&L.ffn_norm, ffn_norm, c.hidden, e->stream));
  L.dense_set = true;
  return CMLD_OK;
}

int32_t cmld_engine_adopt_layer_moe(cmld_engine *e, int32_t layer, cmld_weight *router_f32, cmld_weight *gate_exps,
                                    cmld_weight *up_exps, cmld_weight *down_exps) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  const cmld_config &c = e->cfg;
  if (c.n_experts <= 0) return fail(CMLD_ERR_STATE, "adopt_layer_moe: engine was created without experts");
  if (layer < 0 || layer >= c.n_layers) return fail(CMLD_ERR_INVALID, "adopt_layer_moe: layer %d out of range", layer);
  if (!router_f32 || !gate_exps || !up_exps || !down_exps) return fail(CMLD_ERR_INVALID, "adopt_layer_moe: null weight");
  if (c.n_experts % ep_size(e)) return fail(CMLD_ERR_SHAPE, "n_experts %d not divisible by ep_size %d", c.n_experts, ep_size(e));
  const int64_t n_local = c.n_experts / ep_size(e);
  LayerW &L = e->layers[layer];
  cmld_weight *ts[3] = {gate_exps, up_exps, down_exps};
  const int64_t shapes[3][2] = {{n_local * c.ffn_dim, c.hidden}, {n_local * c.ffn_dim, c.hidden}, {n_local * c.hidden, c.ffn_dim}};
  if (router_f32->qt != CMLD_F32 || router_f32->rows != c.n_experts || router_f32->cols != c.hidden)
    return fail(CMLD_ERR_SHAPE, "adopt_layer_moe: router must be f32 [n_experts][hidden]");
  for (int i = 0; i < 3; ++i)
    if (ts[i]->rows != shapes[i][0] || ts[i]->cols != shapes[i][1] || (ts[i]->qt != CMLD_Q4_K && ts[i]->qt != CMLD_Q6_K))
      return fail(CMLD_ERR_SHAPE, "adopt_layer_moe: expert tensor %d has the wrong shape or type", i);
  for (int i = 0; i < 3; ++i) CMLD_TRY(adopt(L.exps[i], ts[i], shapes[i][0], shapes[i][1], "adopt_layer_moe"));
  cudaFree(L.router);
  L.router = reinterpret_cast<float *>(router_f32->data);
  router_f32->data = nullptr;
  delete router_f32;
  L.moe_set = true;
  return CMLD_OK;
}

int32_t cmld_engine_adopt_output(cmld_engine *e, const float *final_norm, cmld_weight *output) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  if (!output) return fail(CMLD_ERR_INVALID, "adopt_output: weight is null");
  CMLD_TRY(adopt(e->output, output, e->vocab_local, e->cfg.hidden, "adopt_output"));
  CMLD_TRY(upload_f32(&e->final_norm, final_norm, e->cfg.hidden, e->stream));
  e->has_output = true;
  return CMLD_OK;
}

int32_t cmld_engine_adopt_token_embd(cmld_engine *e, cmld_weight *token_embd) {
  CMLD_ENGINE_ENTER(e);
  drop_graphs(e);
  if (!token_embd) return fail(CMLD_ERR_INVALID, "adopt_token_embd: weight is null");
  CMLD_TRY(adopt(e->token_embd, token_embd, e->cfg.vocab, e->cfg.hidden, "adopt_token_embd", true));
  e->has_embd = true;
  return CMLD_OK;
}

int32_t cmld_engine_weights_ready(const cmld_engine *e) {
  if (!e) return 0;
  for (const auto &L : e->layers)
    if (!L.dense_set || (e->cfg.n_experts > 0 && !L.moe_set)) return 0;
  return e->has_output ? 1 : 0;
}
int64_t cmld_engine_filled(const cmld_engine *e) { return e ? e->filled : 0; }
int32_t cmld_engine_set_filled(cmld_engine *e, int64_t filled) {
  if (!e) return fail(CMLD_ERR_INVALID, "engine handle is null");
  if (filled < 0 || filled > e->cfg.max_pos) return fail(CMLD_ERR_INVALID, "filled %lld out of range", (long long)filled);
  e->filled = filled;
  return CMLD_OK;
}
int64_t cmld_engine_max_pos(const cmld_engine *e) { return e ? e->cfg.max_pos : 0; }
int32_t cmld_engine_n_layers(const cmld_engine *e) { return e ? e->cfg.n_layers : 0; }

int32_t cmld_engine_set_rope_frequencies(cmld_engine *e, const float *freq, int32_t n) {
  if (!e || !freq) return fail(CMLD_ERR_INVALID, "null argument");
  if (n != e->cfg.rope_dim / 2) return fail(CMLD_ERR_INVALID, "%d frequencies given, the engine rotates %d pairs", n, e->cfg.rope_dim / 2);
  for (int i = 0; i < n; ++i)
    if (!(freq[i] >= 0.0f) || !std::isfinite(freq[i])) return fail(CMLD_ERR_INVALID, "frequency %d is not a finite non-negative number", i);
  DeviceGuard guard(e->device);
  CMLD_CUDA(cudaStreamSynchronize(e->stream));
  e->rope_freq.assign(freq, freq + n);
  return upload_rope_tables(e);
}

int32_t cmld_engine_rope_row(const cmld_engine *e, int64_t position, float *cos_out, float *sin_out) {
  if (!e || !cos_out || !sin_out) return fail(CMLD_ERR_INVALID, "null argument");
  if (position < 0 || position >= e->cfg.max_pos) return fail(CMLD_ERR_INVALID, "position %lld out of range", (long long)position);
  const int half = e->cfg.rope_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float ang = (float)position * e->rope_freq[i];
    sin_out[i] = sinf(ang);
    cos_out[i] = cosf(ang);
  }
  return CMLD_OK;
}

int32_t cmld_engine_forward_token(cmld_engine *e, const float *embedding, const float *cosv, const float *sinv,
                                  int64_t position, float scale, int32_t compute_logits, uint32_t *token_out) {
  CMLD_ENGINE_ENTER(e);
  if (compute_logits && !token_out) return fail(CMLD_ERR_INVALID, "token_out is null");
  CMLD_TRY(forward_embedding_rows(e, embedding, cosv, sinv, position, 1, scale, compute_logits != 0, compute_logits != 0, false));
  int32_t tok = 0;
  CMLD_TRY(settle(e));
  if (compute_logits) CMLD_CUDA(cudaMemcpyAsync(&tok, e->out_idx, 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "forward_token"));
  if (compute_logits) *token_out = (uint32_t)tok;
  return CMLD_OK;
}

// forward_token_sample / forward_token_sample_min_p (src/cuda_resident.rs:20163, :20197): the full forward, then the
// draw over the resident logits.  min_p <= 0 selects the unfiltered draw (inv_temp = 1 / temperature).  With the
// filter, *token_out = 0xffffffff means "sample this row on the CPU": logits_out (if given) then holds the row.
int32_t cmld_engine_forward_token_sample(cmld_engine *e, const float *embedding, const float *cosv, const float *sinv,
                                         int64_t position, float scale, float temperature, float min_p, uint64_t seed,
                                         uint32_t *token_out, float *logits_out) {
  CMLD_ENGINE_ENTER(e);
  if (!token_out) return fail(CMLD_ERR_INVALID, "token_out is null");
  if (!(temperature > 0.0f) || !std::isfinite(temperature)) return fail(CMLD_ERR_INVALID, "temperature must be a finite positive number");
  if (min_p > 0.0f && !(min_p <= 1.0f)) return fail(CMLD_ERR_INVALID, "min_p must lie in (0, 1]");
  if (e->tp > 1) return fail(CMLD_ERR_UNSUPPORTED, "sampling on a tensor-parallel engine is not supported");
  CMLD_TRY(forward_embedding_rows(e, embedding, cosv, sinv, position, 1, scale, true, false, false));
  uint32_t *d_tok = reinterpret_cast<uint32_t *>(e->out_idx);
  if (min_p > 0.0f) CMLD_TRY(launch_sample_gumbel_filtered(e->logits, e->cfg.vocab, temperature, min_p, seed, d_tok, e->stream));
  else CMLD_TRY(launch_sample_gumbel(e->logits, e->cfg.vocab, 1.0f / temperature, seed, d_tok, e->stream));
  e->launches += 1;
  uint32_t tok = 0;
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(&tok, d_tok, 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "forward_token_sample"));
  *token_out = tok;
  if (tok == 0xffffffffu && logits_out) {
    CMLD_CUDA(cudaMemcpyAsync(logits_out, e->logits, (size_t)e->cfg.vocab * 4, cudaMemcpyDeviceToHost, e->stream));
    CMLD_TRY(finish(e, "forward_token_sample"));
  }
  return CMLD_OK;
}

int32_t cmld_engine_forward_token_logits(cmld_engine *e, const float *embedding, const float *cosv, const float *sinv,
                                         int64_t position, float scale, float *logits_out) {
  CMLD_ENGINE_ENTER(e);
  if (!logits_out) return fail(CMLD_ERR_INVALID, "logits_out is null");
  CMLD_TRY(forward_embedding_rows(e, embedding, cosv, sinv, position, 1, scale, true, false, false));
  if (e->tp > 1) CMLD_TRY(gather_logits(e, 1));
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(logits_out, e->tp > 1 ? e->logits_full : e->logits, (size_t)e->cfg.vocab * 4, cudaMemcpyDeviceToHost, e->stream));
  return finish(e, "forward_token_logits");
}

int32_t cmld_engine_forward_token_hidden(cmld_engine *e, const float *embedding, const float *cosv, const float *sinv,
                                         int64_t position, float scale, float *hidden_out, float *layer_taps) {
  CMLD_ENGINE_ENTER(e);
  if (!hidden_out) return fail(CMLD_ERR_INVALID, "hidden_out is null");
  CMLD_TRY(forward_embedding_rows(e, embedding, cosv, sinv, position, 1, scale, false, false, layer_taps != nullptr));
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(hidden_out, e->h, (size_t)e->cfg.hidden * 4, cudaMemcpyDeviceToHost, e->stream));
  if (layer_taps)
    CMLD_CUDA(cudaMemcpy2DAsync(layer_taps, (size_t)e->cfg.hidden * 4, e->taps, (size_t)e->max_rows * e->cfg.hidden * 4,
                                (size_t)e->cfg.hidden * 4, e->cfg.n_layers, cudaMemcpyDeviceToHost, e->stream));
  return finish(e, "forward_token_hidden");
}

int32_t cmld_engine_forward_layer(cmld_engine *e, int32_t layer, const float *hidden_in, const float *cosv, const float *sinv,
                                  int64_t position, float scale, float *hidden_out) {
  CMLD_ENGINE_ENTER(e);
  if (!hidden_out) return fail(CMLD_ERR_INVALID, "hidden_out is null");
  if (layer < 0 || layer >= e->cfg.n_layers) return fail(CMLD_ERR_INVALID, "layer %d out of range", layer);
  CMLD_TRY(forward_embedding_rows(e, hidden_in, cosv, sinv, position, 1, scale, false, false, false, layer, layer + 1));
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(hidden_out, e->h, (size_t)e->cfg.hidden * 4, cudaMemcpyDeviceToHost, e->stream));
  return finish(e, "forward_layer");
}

int32_t cmld_engine_prefill_from(cmld_engine *e, const float *embeddings, const float *cos_all, const float *sin_all,
                                 int64_t n, float scale, int64_t start) {
  CMLD_ENGINE_ENTER(e);
  if (n < 0 || start < 0 || start > n) return fail(CMLD_ERR_INVALID, "prefill: start=%lld exceeds n=%lld", (long long)start, (long long)n);
  const int half = e->cfg.rope_dim / 2;
  // up to 8 rows go through the row kernel (bit-identical to serial calls); longer prompts 32 rows at a time
  const int chunk = (n - start > 8 && !(e->cfg.flags & CMLD_FLAG_EXACT_ORDER)) ? 32 : 8;
  for (int64_t i = start; i < n; i += chunk) {
    const int rows = (int)std::min<int64_t>(chunk, n - i);
    CMLD_TRY(forward_embedding_rows(e, embeddings + i * e->cfg.hidden, cos_all + i * half, sin_all + i * half, i, rows, scale,
                                    false, false, false));
  }
  return finish(e, "prefill");
}

int32_t cmld_engine_verify_batch(cmld_engine *e, const float *embeddings, const float *cos_all, const float *sin_all,
                                 int64_t base_position, int32_t k, float scale, uint32_t *tokens_out) {
  CMLD_ENGINE_ENTER(e);
  if (k < 1 || k > e->max_rows) return fail(CMLD_ERR_INVALID, "verify_batch: k=%d out of 1..=%d", k, e->max_rows);
  if (!tokens_out) return fail(CMLD_ERR_INVALID, "tokens_out is null");
  CMLD_TRY(forward_embedding_rows(e, embeddings, cos_all, sin_all, base_position, k, scale, true, true, false));
  std::vector<int32_t> toks(k);
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(toks.data(), e->out_idx, (size_t)k * 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "verify_batch"));
  for (int i = 0; i < k; ++i) tokens_out[i] = (uint32_t)toks[i];
  return CMLD_OK;
}


// verify_tree (src/cuda_resident.rs:22944): the N nodes of a draft tree (breadth-first order) in one batched pass.
// Node i writes its K/V to cache row node_kvslot[i] (= base + i), is rotated by its own cos/sin row (position base +
// depth) and attends to the committed prefix below base plus the nodes its ancestor mask names; tokens_out[i] is the
// greedy token after node i along its path.  The sums run over exactly the rows a linear decode of that path would
// see, in the same order, so the prediction is the linear decode's.
int32_t cmld_engine_verify_tree(cmld_engine *e, const float *embeddings, const float *cos_all, const float *sin_all,
                                const int32_t *node_kvslot, const uint32_t *ancestor_bits, int32_t words, int64_t base_position,
                                int32_t n, float scale, uint32_t *tokens_out) {
  CMLD_ENGINE_ENTER(e);
  const cmld_config &c = e->cfg;
  if (n < 1 || n > CMLD_TREE_MAX_NODES) return fail(CMLD_ERR_INVALID, "verify_tree: n=%d out of 1..=%d", n, CMLD_TREE_MAX_NODES);
  if (!embeddings || !cos_all || !sin_all || !node_kvslot || !ancestor_bits || !tokens_out) return fail(CMLD_ERR_INVALID, "verify_tree: null argument");
  if (words != 1) return fail(CMLD_ERR_INVALID, "verify_tree: %d mask words per node, 1 expected for at most %d nodes", words, CMLD_TREE_MAX_NODES);
  if (base_position < 0 || base_position + n > c.max_pos) return fail(CMLD_ERR_STATE, "verify_tree: rows %lld..%lld exceed max_pos %d", (long long)base_position, (long long)(base_position + n - 1), c.max_pos);
  if (e->tp > 1 || e->ep > 1) return fail(CMLD_ERR_UNSUPPORTED, "verify_tree: sharded engines are not supported");
  if (e->kq8) return fail(CMLD_ERR_UNSUPPORTED, "verify_tree: not supported over a Q8_0 KV cache");
  std::vector<uint32_t> masks(n);
  std::vector<int32_t> pos(n), slots(n, 0);
  for (int i = 0; i < n; ++i) {
    if (node_kvslot[i] != base_position + i) return fail(CMLD_ERR_INVALID, "verify_tree: node %d has cache row %d, base + index = %lld expected", i, node_kvslot[i], (long long)(base_position + i));
    if (ancestor_bits[i] >> (i + 1)) return fail(CMLD_ERR_INVALID, "verify_tree: node %d names a later node as its ancestor", i);
    masks[i] = ancestor_bits[i] | (1u << i);  // a node sees itself
    pos[i] = (int32_t)(base_position + i);
  }
  CMLD_TRY(require_weights(e, true));
  if (!e->tree_mask) CMLD_TRY(dev_alloc(e, &e->tree_mask, CMLD_TREE_MAX_NODES));
  const int half = c.rope_dim / 2;
  CMLD_CUDA(cudaMemcpyAsync(e->h, embeddings, (size_t)n * c.hidden * 4, cudaMemcpyDefault, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->cos_step, cos_all, (size_t)n * half * 4, cudaMemcpyDefault, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->sin_step, sin_all, (size_t)n * half * 4, cudaMemcpyDefault, e->stream));
  CMLD_CUDA(cudaMemcpyAsync(e->tree_mask, masks.data(), (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
  CMLD_TRY(stage_rows(e, n, nullptr, pos.data(), slots.data()));
  StepOpts o;
  o.batch = n;
  o.shared_slots = true;  // every node's K/V row is appended before any node attends
  o.from_tokens = false;
  o.rope_by_position = false;
  o.scale = scale;
  o.logits = true;
  o.argmax = true;
  o.tree_mask = e->tree_mask;
  o.tree_base = (int32_t)base_position;
  o.tree_words = 1;
  CMLD_TRY(run_step(e, o));
  std::vector<int32_t> toks(n);
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(toks.data(), e->out_idx, (size_t)n * 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "verify_tree"));
  for (int i = 0; i < n; ++i) tokens_out[i] = (uint32_t)toks[i];
  return CMLD_OK;
}

__global__ void kv_compact_kernel(__half *kc, __half *vc, int64_t layer_elems, int n_layers, int n_kv, int64_t max_pos, int hd, int64_t src,
                                  int64_t dst) {
  const int64_t total = (int64_t)n_layers * n_kv * hd;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t li = i / ((int64_t)n_kv * hd), rem = i % ((int64_t)n_kv * hd), kh = rem / hd, d = rem % hd;
    const int64_t row = li * layer_elems + kh * max_pos * hd;
    kc[row + dst * hd + d] = kc[row + src * hd + d];
    vc[row + dst * hd + d] = vc[row + src * hd + d];
  }
}

// compact_tree_kv_path (src/cuda_resident.rs:23071): the accepted path's K/V rows, at cache rows base + path[r], move
// to the contiguous rows base + r (front to back; path[r] >= r, so a source is never overwritten before it is read).
int32_t cmld_engine_compact_tree_kv_path(cmld_engine *e, const int32_t *path, int32_t len, int64_t base_position) {
  CMLD_ENGINE_ENTER(e);
  const cmld_config &c = e->cfg;
  if (!path || len < 0 || len > CMLD_TREE_MAX_NODES) return fail(CMLD_ERR_INVALID, "compact_tree_kv_path: bad path");
  if (e->kq8) return fail(CMLD_ERR_UNSUPPORTED, "compact_tree_kv_path: not supported over a Q8_0 KV cache");
  for (int r = 0; r < len; ++r) {
    if (path[r] < r || path[r] >= CMLD_TREE_MAX_NODES || (r > 0 && path[r] <= path[r - 1])) return fail(CMLD_ERR_INVALID, "compact_tree_kv_path: path is not an increasing sequence of node indices");
    if (base_position + path[r] >= c.max_pos) return fail(CMLD_ERR_STATE, "compact_tree_kv_path: row beyond max_pos");
  }
  for (int r = 0; r < len; ++r) {
    if (path[r] == r) continue;
    kv_compact_kernel<<<64, 256, 0, e->stream>>>(e->kcache, e->vcache, e->kv_layer_elems, c.n_layers, c.n_kv_heads, c.max_pos, c.head_dim,
                                                 base_position + path[r], base_position + r);
    CMLD_CUDA(cudaGetLastError());
  }
  return finish(e, "compact_tree_kv_path");
}

// KV import/export, slot 0: f32 [kv_head][n_positions][head_dim] <-> f16 cache rows.
__global__ void kv_convert_kernel(__half *cache, float *host_layout, int n_kv, int64_t max_pos, int64_t n_pos, int hd,
                                  bool to_cache) {
  const int64_t total = (int64_t)n_kv * n_pos * hd;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t kh = i / (n_pos * hd), rem = i % (n_pos * hd);
    const int64_t ci = kh * max_pos * hd + rem;
    if (to_cache) cache[ci] = __float2half_rn(host_layout[i]);
    else host_layout[i] = __half2float(cache[ci]);
  }
}

static int32_t kv_transfer(cmld_engine *e, int32_t layer, float *ck, float *cv, int64_t n_pos, bool to_cache) {
  const cmld_config &c = e->cfg;
  if (layer < 0 || layer >= c.n_layers) return fail(CMLD_ERR_INVALID, "layer %d out of range", layer);
  if (n_pos < 0 || n_pos > c.max_pos) return fail(CMLD_ERR_INVALID, "n_positions %lld out of range", (long long)n_pos);
  if (n_pos == 0) return CMLD_OK;
  if (!ck || !cv) return fail(CMLD_ERR_INVALID, "KV buffer is null");
  const int64_t n = (int64_t)c.n_kv_heads * n_pos * c.head_dim;
  float *tmp = nullptr;
  CMLD_CUDA(cudaMalloc(&tmp, (size_t)n * 4));
  int32_t rc = CMLD_OK;
  for (int side = 0; side < 2 && rc == CMLD_OK; ++side) {
    float *hostp = side == 0 ? ck : cv;
    if (e->kq8) {
      // Q8_0 cache: rows are quantised block by block on the way in and dequantised (code * d) on the way out
      uint8_t *qc = (side == 0 ? e->kq8 : e->vq8) + (int64_t)layer * e->kv_q8_bytes;
      if (to_cache && cudaMemcpyAsync(tmp, hostp, (size_t)n * 4, cudaMemcpyDefault, e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV upload failed");
      if (rc == CMLD_OK) rc = launch_kv_q8_convert(qc, tmp, c.n_kv_heads, c.max_pos, n_pos, c.head_dim, to_cache, e->stream);
      if (rc == CMLD_OK && !to_cache && cudaMemcpyAsync(hostp, tmp, (size_t)n * 4, cudaMemcpyDefault, e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV download failed");
      if (rc == CMLD_OK && cudaStreamSynchronize(e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV transfer failed");
      continue;
    }
    __half *cache = (side == 0 ? e->kcache : e->vcache) + (int64_t)layer * e->kv_layer_elems;
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 255) / 256, 4096);
    if (to_cache) {
      if (cudaMemcpyAsync(tmp, hostp, (size_t)n * 4, cudaMemcpyDefault, e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV upload failed");
      kv_convert_kernel<<<blocks, 256, 0, e->stream>>>(cache, tmp, c.n_kv_heads, c.max_pos, n_pos, c.head_dim, true);
    } else {
      kv_convert_kernel<<<blocks, 256, 0, e->stream>>>(cache, tmp, c.n_kv_heads, c.max_pos, n_pos, c.head_dim, false);
      if (cudaMemcpyAsync(hostp, tmp, (size_t)n * 4, cudaMemcpyDefault, e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV download failed");
    }
    if (rc == CMLD_OK && cudaStreamSynchronize(e->stream) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "KV transfer failed");
  }
  cudaFree(tmp);
  return rc;
}

int32_t cmld_engine_seed_layer(cmld_engine *e, int32_t layer, const float *ck, const float *cv, int64_t n_positions) {
  CMLD_ENGINE_ENTER(e);
  return kv_transfer(e, layer, const_cast<float *>(ck), const_cast<float *>(cv), n_positions, true);
}

int32_t cmld_engine_read_kv_layer(cmld_engine *e, int32_t layer, int64_t n_positions, float *ck_out, float *cv_out) {
  CMLD_ENGINE_ENTER(e);
  return kv_transfer(e, layer, ck_out, cv_out, n_positions, false);
}

// ---------------------------------------------------------------- token-id driven calls

static int32_t check_rows(cmld_engine *e, int32_t n, const int32_t *seqs, const int32_t *tokens, const int64_t *positions,
                          int64_t extra_steps, std::vector<int32_t> &pos32) {
  const cmld_config &c = e->cfg;
  if (n < 1 || n > e->max_rows) return fail(CMLD_ERR_INVALID, "%d rows exceed the engine's %d", n, e->max_rows);
  if (!seqs || !tokens || !positions) return fail(CMLD_ERR_INVALID, "seqs / tokens / positions pointer is null");
  pos32.resize(n);
  const int slots = std::max(1, c.max_seqs);
  for (int i = 0; i < n; ++i) {
    if (seqs[i] < 0 || seqs[i] >= slots) return fail(CMLD_ERR_INVALID, "sequence slot %d out of range (max_seqs %d)", seqs[i], slots);
    if (tokens[i] < 0 || tokens[i] >= c.vocab) return fail(CMLD_ERR_INVALID, "token id %d out of range", tokens[i]);
    if (positions[i] < 0 || positions[i] + extra_steps > c.max_pos)
      return fail(CMLD_ERR_STATE, "position %lld (+%lld steps) exceeds max_pos %d", (long long)positions[i], (long long)extra_steps, c.max_pos);
    pos32[i] = (int32_t)positions[i];
  }
  return CMLD_OK;
}

static bool has_shared_slots(const int32_t *seqs, int n) {
  for (int i = 0; i < n; ++i)
    for (int j = i + 1; j < n; ++j)
      if (seqs[i] == seqs[j]) return true;
  return false;
}

int32_t cmld_engine_step_batch(cmld_engine *e, int32_t n_seqs, const int32_t *seqs, const int32_t *tokens_in,
                               const int64_t *positions, uint32_t *tokens_out, float *logits_out, float *hidden_out) {
  CMLD_ENGINE_ENTER(e);
  std::vector<int32_t> pos32;
  CMLD_TRY(check_rows(e, n_seqs, seqs, tokens_in, positions, 1, pos32));
  CMLD_TRY(require_weights(e, true));
  CMLD_TRY(stage_rows(e, n_seqs, tokens_in, pos32.data(), seqs));
  e->launches = 0;
  CMLD_CUDA(cudaEventRecord(e->ev0, e->stream));
  StepOpts o;
  o.batch = n_seqs;
  o.shared_slots = has_shared_slots(seqs, n_seqs);
  o.from_tokens = true;
  o.scale = 1.0f / sqrtf((float)e->cfg.head_dim);
  {
    int64_t mx = 0;
    for (int i = 0; i < n_seqs; ++i) mx = std::max<int64_t>(mx, positions[i]);
    o.attn_cluster = use_attn_cluster(n_seqs, mx);
    o.attn_cap = attn_cap_for(mx);
  }
  CMLD_TRY(run_step(e, o));
  CMLD_CUDA(cudaEventRecord(e->ev1, e->stream));
  std::vector<int32_t> toks(n_seqs);
  if (logits_out && e->tp > 1) CMLD_TRY(gather_logits(e, n_seqs));
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(toks.data(), e->out_idx, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, e->stream));
  if (logits_out) CMLD_CUDA(cudaMemcpyAsync(logits_out, e->tp > 1 ? e->logits_full : e->logits, (size_t)n_seqs * e->cfg.vocab * 4, cudaMemcpyDeviceToHost, e->stream));
  if (hidden_out) CMLD_CUDA(cudaMemcpyAsync(hidden_out, e->h, (size_t)n_seqs * e->cfg.hidden * 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "step_batch"));
  cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
  e->last_launches = e->launches;
  if (tokens_out)
    for (int i = 0; i < n_seqs; ++i) tokens_out[i] = (uint32_t)toks[i];
  return CMLD_OK;
}

int32_t cmld_engine_prefill_tokens(cmld_engine *e, int32_t seq, const int32_t *tokens, int64_t n, int64_t start_pos,
                                   uint32_t *next_token_out) {
  CMLD_ENGINE_ENTER(e);
  if (n < 1 || !tokens) return fail(CMLD_ERR_INVALID, "prefill_tokens: no tokens");
  CMLD_TRY(require_weights(e, true));
  const int chunk = (n > 8 && !(e->cfg.flags & CMLD_FLAG_EXACT_ORDER)) ? 32 : 8;
  e->launches = 0;
  CMLD_CUDA(cudaEventRecord(e->ev0, e->stream));
  int last_rows = 0;
  for (int64_t i = 0; i < n; i += chunk) {
    const int rows = (int)std::min<int64_t>(chunk, n - i);
    std::vector<int32_t> seqs(rows, seq), pos32;
    std::vector<int64_t> pos(rows);
    for (int r = 0; r < rows; ++r) pos[r] = start_pos + i + r;
    CMLD_TRY(check_rows(e, rows, seqs.data(), tokens + i, pos.data(), 1, pos32));
    CMLD_TRY(stage_rows(e, rows, tokens + i, pos32.data(), seqs.data()));
    StepOpts o;
    o.batch = rows;
    o.shared_slots = rows > 1;
    o.from_tokens = true;
    o.scale = 1.0f / sqrtf((float)e->cfg.head_dim);
    o.logits = o.argmax = (i + chunk >= n);
    o.attn_cluster = use_attn_cluster(rows, start_pos + i + rows - 1);
    o.attn_cap = attn_cap_for(start_pos + i + rows - 1);
    CMLD_TRY(run_step(e, o));
    last_rows = rows;
  }
  CMLD_CUDA(cudaEventRecord(e->ev1, e->stream));
  int32_t tok = 0;
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(&tok, e->out_idx + (last_rows - 1), 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "prefill_tokens"));
  cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
  e->last_launches = e->launches;
  if (next_token_out) *next_token_out = (uint32_t)tok;
  return CMLD_OK;
}

int32_t cmld_engine_decode_greedy(cmld_engine *e, int32_t n_seqs, const int32_t *seqs, const int32_t *tokens_in,
                                  const int64_t *positions, int32_t n_steps, uint32_t *tokens_out) {
  CMLD_ENGINE_ENTER(e);
  if (n_steps < 1 || n_steps > e->history_cap) return fail(CMLD_ERR_INVALID, "decode_greedy: n_steps %d out of 1..=%lld", n_steps, (long long)e->history_cap);
  if (!tokens_out) return fail(CMLD_ERR_INVALID, "tokens_out is null");
  std::vector<int32_t> pos32;
  CMLD_TRY(check_rows(e, n_seqs, seqs, tokens_in, positions, n_steps, pos32));
  CMLD_TRY(require_weights(e, true));
  CMLD_TRY(stage_rows(e, n_seqs, tokens_in, pos32.data(), seqs));
  CMLD_CUDA(cudaMemsetAsync(e->am_ticket, 0, (size_t)2 * e->max_rows * 4, e->stream));
  e->launches = 0;
  CMLD_CUDA(cudaEventRecord(e->ev0, e->stream));
  StepOpts o;
  o.batch = n_seqs;
  o.shared_slots = has_shared_slots(seqs, n_seqs);
  o.from_tokens = true;
  o.scale = 1.0f / sqrtf((float)e->cfg.head_dim);
  o.feed_back = true;
  int64_t max_start = 0;
  for (int i = 0; i < n_seqs; ++i) max_start = std::max<int64_t>(max_start, positions[i]);
  for (int s = 0; s < n_steps; ++s) {
    o.attn_cluster = use_attn_cluster(n_seqs, max_start + s);
    o.attn_cap = attn_cap_for(max_start + s);
    CMLD_TRY(run_step(e, o));
  }
  CMLD_CUDA(cudaEventRecord(e->ev1, e->stream));
  std::vector<int32_t> hist((size_t)n_steps * n_seqs);
  CMLD_TRY(settle(e));
  CMLD_CUDA(cudaMemcpyAsync(hist.data(), e->d_history, hist.size() * 4, cudaMemcpyDeviceToHost, e->stream));
  CMLD_TRY(finish(e, "decode_greedy"));
  cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
  e->last_launches = e->launches;
  for (size_t i = 0; i < hist.size(); ++i) tokens_out[i] = (uint32_t)hist[i];
  return CMLD_OK;
}

int32_t cmld_engine_last_timing(const cmld_engine *e, float *ms_out, int64_t *launches_out) {
  if (!e) return fail(CMLD_ERR_INVALID, "engine handle is null");
  if (ms_out) *ms_out = e->last_ms;
  if (launches_out) *launches_out = e->last_launches;
  return CMLD_OK;
}

}  // extern "C"
