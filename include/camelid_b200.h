/*
 * camelid_b200.h — C ABI of the B200 (sm_100a) decode engine.
 *
 * The engine replaces Camelid's resident CUDA decode lane.  In Camelid that lane is a
 * Rust type, `cuda_resident::CudaResidentDecode` (src/cuda_resident.rs:15093), driven by
 * `build_resident_cuda_engine` (src/inference.rs:16352) and
 * `try_resident_decode_forward_cuda` (src/inference.rs:4945).  Every `cmld_engine_*`
 * entry point below names the method it stands in for; argument order and meaning follow
 * that method.  Calls on one engine must be serialised by the caller (Camelid holds its
 * engine inside a process-global Mutex, src/inference.rs:5087-5090).
 *
 * Conventions: every call returns a cmld_status (0 = OK); cmld_last_error() gives the
 * calling thread's last message; nothing throws across this boundary; host pointers are
 * borrowed for the duration of the call only; there is no CPU fallback — a call either
 * runs on the GPU or returns an error.
 */
#ifndef CAMELID_B200_H
#define CAMELID_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CMLD_API __attribute__((visibility("default")))

typedef enum {
  CMLD_OK = 0,
  CMLD_ERR_INVALID = 1,     /* null pointer, bad handle, argument out of range */
  CMLD_ERR_SHAPE = 2,       /* dimensions the kernels do not accept */
  CMLD_ERR_UNSUPPORTED = 3, /* quantisation type or feature outside Q8_0/Q4_K/Q6_K */
  CMLD_ERR_OOM = 4,
  CMLD_ERR_CUDA = 5,
  CMLD_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up */
  CMLD_ERR_STATE = 7        /* weights not set, position beyond max_pos, ... */
} cmld_status;

/* GGUF tensor type ids (src/gguf/reader.rs:94-128); ProjQuant in src/cuda_resident.rs:14846. */
typedef enum {
  CMLD_F32 = 0,
  CMLD_Q8_0 = 8,          /* 34-byte wire blocks: f16 d + 32 x i8 */
  CMLD_Q4_K = 12,         /* 144-byte superblocks */
  CMLD_Q6_K = 14,         /* 210-byte superblocks */
  CMLD_Q8_0_HOST36 = 108  /* Camelid's host block {f32 scale; i8[32]} (src/tensor/mod.rs:105-118),
                             what q8_0_raw_bytes hands to set_layer (src/inference.rs:16387) */
} cmld_qtype;

/* Activation quantisation formats (src/inference.rs:22510-22528 and :23121-23152). */
typedef enum { CMLD_ACT_Q8_0 = 1, CMLD_ACT_Q8_K = 2 } cmld_act_kind;

typedef struct {
  const void *data; /* host or device memory */
  uint64_t nbytes;
  int32_t qtype;    /* cmld_qtype */
  int32_t reserved;
} cmld_tensor;

/* Arguments of CudaResidentDecode::new (src/cuda_resident.rs:15718-15731) plus what the
 * on-device token loop, batching and sharding need. */
typedef struct {
  int32_t n_layers, n_heads, n_kv_heads, head_dim, hidden, ffn_dim, rope_dim, max_pos, vocab;
  float eps;
  int32_t split_half_pairing;
  float rope_theta;        /* base of the engine-owned all-position RoPE table */
  int32_t max_seqs;        /* independent sequences (KV slots); 0 means 1 */
  int32_t n_experts;       /* 0 = dense FFN */
  int32_t n_experts_used;
  int32_t tp_rank, tp_size; /* tensor-parallel shard of a dense model; tp_size 0/1 = unsharded */
  int32_t ep_rank, ep_size; /* expert-parallel shard of a MoE model */
  int32_t device;           /* CUDA ordinal; -1 = current device */
  int32_t flags;            /* CMLD_FLAG_* */
} cmld_config;

#define CMLD_FLAG_NO_GRAPH 1u     /* launch kernels directly instead of replaying a CUDA graph */
#define CMLD_FLAG_DIRECT_GEMV 2u  /* use the generic matvec kernel everywhere (no staged kernel) */
#define CMLD_FLAG_NO_PDL 4u       /* no programmatic dependent launch between kernels */
#define CMLD_FLAG_EXACT_ORDER 16u   /* the plain reference-order kernels (one lane walks each sum): the same bits as the default path, slowly; a cross-check */
#define CMLD_FLAG_SPLIT_PROLOGUE 8u /* norm/SwiGLU/quantise in a small kernel of its own instead of the matvec prologue (always so for steps of more than 2 rows) */
#define CMLD_FLAG_FAST_ORDER 128u  /* attention by the split-range (flash-decoding) kernel, whose sums are trees: faster at long contexts, no longer the CPU path's bits */
#define CMLD_FLAG_TENSOR_BATCH 64u   /* steps of 5..32 rows and prompt ingestion on the int8 mma.sync matvec (one pass over the weights; its row sums are trees, so no longer the CPU path's bits) */
#define CMLD_FLAG_KV_Q8_0 256u     /* KV cache as Q8_0 blocks (new_with_kv_quant, src/cuda_resident.rs:15748; src/tensor/kv_quant.rs): 34 bytes per 32 values; the arithmetic of the CPU lane's scalar path */
#define CMLD_FLAG_NCCL_ONLY 32u     /* sharded engines: every sublayer sum as an NCCL all-reduce (no peer-memory path in the matvec kernels) */

typedef struct cmld_engine cmld_engine;
typedef struct cmld_weight cmld_weight;

CMLD_API const char *cmld_last_error(void);
CMLD_API const char *cmld_version(void);
CMLD_API int32_t cmld_device_count(void);
/* Selects the calling thread's CUDA device: cmld_malloc, cmld_weight_create/synth/shard and the
 * operator-level calls work on it.  Engine calls select their own engine's device themselves. */
CMLD_API int32_t cmld_set_device(int32_t device);

/* ---- device memory helpers (so a host without its own CUDA binding can stage buffers) ---- */
CMLD_API int32_t cmld_malloc(void **dev_ptr, uint64_t nbytes);
CMLD_API int32_t cmld_free(void *dev_ptr);
CMLD_API int32_t cmld_memcpy_h2d(void *dst_dev, const void *src_host, uint64_t nbytes);
CMLD_API int32_t cmld_memcpy_d2h(void *dst_host, const void *src_dev, uint64_t nbytes);
CMLD_API int32_t cmld_memset(void *dst_dev, int32_t value, uint64_t nbytes);
CMLD_API int32_t cmld_device_synchronize(void);
CMLD_API int32_t cmld_mem_info(uint64_t *free_bytes, uint64_t *total_bytes);

/* ---- engine lifetime: CudaResidentDecode::new_with_kv_quant (src/cuda_resident.rs:15748) ---- */
CMLD_API int32_t cmld_engine_create(const cmld_config *cfg, cmld_engine **out);
CMLD_API int32_t cmld_engine_destroy(cmld_engine *e);

/* Sharded engines (no reference counterpart: Camelid's only multi-device mode is a two-stage TCP
 * pipeline, src/distributed.rs).  One process per GPU.  With cfg.tp_size = N > 1 (dense models) the
 * engine holds n_heads/N query heads with their kv heads, ffn_dim/N FFN rows and vocab/N output
 * rows: set_layer / adopt_layer then take q,k,v,gate,up as that rank's ROW block, o and down as its
 * COLUMN block (multiples of 256), set_output its vocabulary rows; the embedding table, norms and
 * all host-visible vectors (embeddings, hidden, logits, tokens) keep the model's full sizes.  With
 * cfg.ep_size = N > 1 (Mixtral shapes) the expert slabs hold experts ep_rank, ep_rank+N, ....
 * seed_layer / read_kv_layer see only the rank's kv heads.  Every rank must make the same calls in
 * the same order: each step all-reduces over NCCL (NVLink / NVSwitch).
 * cmld_comm_unique_id: made once on rank 0 and sent to the others by the caller (any channel).
 * cmld_engine_comm_init: collective over the N ranks; required before the first step.
 * A rank whose peers stop answering does not wait for ever: a call that is still waiting for its
 * device work after the limit (CMLD_COMM_TIMEOUT_MS in the environment, default 120000) aborts the
 * communicator and returns CMLD_ERR_TIMEOUT; the engine then refuses further sharded steps. */
CMLD_API int32_t cmld_comm_unique_id(uint8_t out[128]);
CMLD_API int32_t cmld_engine_comm_init(cmld_engine *e, const uint8_t id[128], int32_t rank, int32_t world);

/* set_layer_located (src/cuda_resident.rs:16133): projs = q,k,v,o,gate,up,down as GGUF wire
 * bytes (Q4_K/Q6_K/Q8_0) or 36-byte host blocks (CMLD_Q8_0_HOST36).  Layers may be set in
 * any order.  For a MoE layer pass gate/up/down with data == NULL and call
 * cmld_engine_set_layer_moe as well. */
CMLD_API int32_t cmld_engine_set_layer(cmld_engine *e, int32_t layer, const cmld_tensor projs[7],
                                       const float *attn_norm, const float *ffn_norm);
/* Mixtral FFN (CPU path: mixtral_moe_ffn, src/inference.rs:14142): router f32
 * [n_experts][hidden]; each expert tensor holds n_experts consecutive [rows][cols] slabs. */
CMLD_API int32_t cmld_engine_set_layer_moe(cmld_engine *e, int32_t layer, const float *router,
                                           const cmld_tensor *gate_exps, const cmld_tensor *up_exps,
                                           const cmld_tensor *down_exps);
/* set_output (src/cuda_resident.rs:16361). */
CMLD_API int32_t cmld_engine_set_output(cmld_engine *e, const float *final_norm, const cmld_tensor *output);
/* set_device_decode_tables (src/cuda_resident.rs:19671): keeps the embedding table on the
 * device so a greedy step needs only the previous token id. */
CMLD_API int32_t cmld_engine_set_token_embd(cmld_engine *e, const cmld_tensor *token_embd);

/* The same three calls for matrices that already live on the device as cmld_weight handles
 * (made by cmld_weight_create or cmld_weight_synth, declared below).  The engine takes the
 * handles over: on success they are consumed and must not be used or destroyed by the caller.
 * A NULL entry leaves that slot as it is. */
CMLD_API int32_t cmld_engine_adopt_layer(cmld_engine *e, int32_t layer, struct cmld_weight *const projs[7],
                                         const float *attn_norm, const float *ffn_norm);
CMLD_API int32_t cmld_engine_adopt_layer_moe(cmld_engine *e, int32_t layer, struct cmld_weight *router_f32,
                                             struct cmld_weight *gate_exps, struct cmld_weight *up_exps,
                                             struct cmld_weight *down_exps);
CMLD_API int32_t cmld_engine_adopt_output(cmld_engine *e, const float *final_norm, struct cmld_weight *output);
CMLD_API int32_t cmld_engine_adopt_token_embd(cmld_engine *e, struct cmld_weight *token_embd);

/* weights_ready / filled / set_filled / max_pos / n_layers (src/cuda_resident.rs:16988-17342). */
CMLD_API int32_t cmld_engine_weights_ready(const cmld_engine *e);
CMLD_API int64_t cmld_engine_filled(const cmld_engine *e);
CMLD_API int32_t cmld_engine_set_filled(cmld_engine *e, int64_t filled);
CMLD_API int64_t cmld_engine_max_pos(const cmld_engine *e);
CMLD_API int32_t cmld_engine_n_layers(const cmld_engine *e);

/* Replaces the per-pair angular frequencies of the engine-owned RoPE table (n = rope_dim / 2) and
 * recomputes the table for every position: what rope_pair_frequency yields for the model at hand
 * (src/inference/rope.rs:532-560: freq_base^(-2i/rope_dim), divided by rope_freqs.weight[i], then
 * linear / llama3 scaling).  The default after cmld_engine_create is the unscaled form.  Not to be
 * called while a step is in flight. */
CMLD_API int32_t cmld_engine_set_rope_frequencies(cmld_engine *e, const float *freq, int32_t n);

/* The RoPE row of one position, cos_out/sin_out[rope_dim/2], as the engine's own all-position
 * table holds it: theta_i = powf(rope_theta, -2i/rope_dim), sinf/cosf of position*theta_i with the
 * host libm — what resident_decode_rope_tables computes per token (src/inference/rope.rs:600-655).
 * Host-side helper; touches no device memory. */
CMLD_API int32_t cmld_engine_rope_row(const cmld_engine *e, int64_t position, float *cos_out, float *sin_out);

/* forward_token (src/cuda_resident.rs:19548): embedding[hidden], cos/sin[rope_dim/2], the
 * position to write, the score scale; *token_out receives the argmax id when
 * compute_logits != 0. */
CMLD_API int32_t cmld_engine_forward_token(cmld_engine *e, const float *embedding, const float *cosv,
                                           const float *sinv, int64_t position, float scale,
                                           int32_t compute_logits, uint32_t *token_out);
/* forward_token_sample / forward_token_sample_min_p (src/cuda_resident.rs:20163, :20197): the full forward, then a
 * temperature draw over the resident logits by the Gumbel-max trick, the per-token uniforms a splitmix64 hash of
 * (seed, index) (src/cuda_resident/sampling.cuh).  min_p <= 0: unfiltered draw at inv_temp = 1 / temperature.
 * min_p in (0, 1]: min-p filtering precedes temperature; *token_out = 0xffffffff then means the filter could
 * not be decided on the device (a probability ratio within 64 ulp of the cutoff, or a non-finite logit) and the
 * caller samples on the CPU from logits_out[vocab], which is filled in that case if not NULL. */
CMLD_API int32_t cmld_engine_forward_token_sample(cmld_engine *e, const float *embedding, const float *cosv, const float *sinv,
                                                  int64_t position, float scale, float temperature, float min_p, uint64_t seed,
                                                  uint32_t *token_out, float *logits_out);

/* forward_token_logits (src/cuda_resident.rs:20024): logits_out[vocab]. */
CMLD_API int32_t cmld_engine_forward_token_logits(cmld_engine *e, const float *embedding, const float *cosv,
                                                  const float *sinv, int64_t position, float scale,
                                                  float *logits_out);
/* forward_token_hidden (src/cuda_resident.rs:19648): hidden_out[hidden], the residual stream
 * before the final norm.  layer_taps, if not NULL, receives [n_layers][hidden]: the residual
 * stream after each layer (for per-layer parity checks). */
CMLD_API int32_t cmld_engine_forward_token_hidden(cmld_engine *e, const float *embedding, const float *cosv,
                                                  const float *sinv, int64_t position, float scale,
                                                  float *hidden_out, float *layer_taps);
/* One layer only (no counterpart in the reference; for per-layer parity checks): runs layer
 * `layer` on hidden_in[hidden] — the residual stream entering that layer — at `position`, writes
 * that layer's KV row, and returns the residual stream leaving it in hidden_out[hidden]. */
CMLD_API int32_t cmld_engine_forward_layer(cmld_engine *e, int32_t layer, const float *hidden_in, const float *cosv,
                                           const float *sinv, int64_t position, float scale, float *hidden_out);
/* prefill / prefill_from (src/cuda_resident.rs:20266-20316): n positions of one sequence,
 * embeddings[n][hidden], cos_all/sin_all[n][rope_dim/2]; positions [0,start) are kept. */
CMLD_API int32_t cmld_engine_prefill_from(cmld_engine *e, const float *embeddings, const float *cos_all,
                                          const float *sin_all, int64_t n, float scale, int64_t start);
/* verify_batch (src/cuda_resident.rs:20325): k consecutive positions of one sequence in one
 * pass; tokens_out[k] = greedy id at each position. */
CMLD_API int32_t cmld_engine_verify_batch(cmld_engine *e, const float *embeddings, const float *cos_all,
                                          const float *sin_all, int64_t base_position, int32_t k, float scale,
                                          uint32_t *tokens_out);
/* verify_tree (src/cuda_resident.rs:22944): runs the n nodes of a draft tree (breadth-first order,
 * n <= CMLD_TREE_MAX_NODES = TREE_MAX_NODES of src/inference/spec_tree.rs:27) through the model in one
 * batched pass.  embeddings[n][hidden]; cos_all/sin_all[n][rope_dim/2] are the nodes' own RoPE rows
 * (position base + depth); node_kvslot[i] must be base_position + i; ancestor_bits[n][words] is the
 * causal tree mask (bit j of node i = node j is an ancestor of i; words = 1).  tokens_out[i] = the
 * greedy token after node i along its path: what a linear decode of that path yields.  The nodes'
 * K/V rows stay at base_position + i; cmld_engine_compact_tree_kv_path then moves the accepted
 * path's rows to base_position + rank (compact_tree_kv_path, :23071). */
#define CMLD_TREE_MAX_NODES 16
CMLD_API int32_t cmld_engine_verify_tree(cmld_engine *e, const float *embeddings, const float *cos_all, const float *sin_all,
                                         const int32_t *node_kvslot, const uint32_t *ancestor_bits, int32_t words,
                                         int64_t base_position, int32_t n, float scale, uint32_t *tokens_out);
CMLD_API int32_t cmld_engine_compact_tree_kv_path(cmld_engine *e, const int32_t *path, int32_t len, int64_t base_position);

/* seed_layer / read_kv_layer (src/cuda_resident.rs:17355, :17448): K and V of one layer as
 * f32 [kv_head][n_positions][head_dim] (values are f16-exact), sequence slot 0. */
CMLD_API int32_t cmld_engine_seed_layer(cmld_engine *e, int32_t layer, const float *ck, const float *cv,
                                        int64_t n_positions);
CMLD_API int32_t cmld_engine_read_kv_layer(cmld_engine *e, int32_t layer, int64_t n_positions, float *ck_out,
                                           float *cv_out);

/* ---- on-device token loop (forward_token_device, src/cuda_resident.rs:19671-19834, there
 * for one architecture only; here for all).  Needs cmld_engine_set_token_embd. ---- */

/* Feeds `n` prompt tokens of sequence slot `seq` at positions start_pos.. and returns the
 * greedy id after the last one (prompt ingestion uses the decode kernels, as the reference
 * does for K-quant models, src/inference.rs:4057-4086). */
CMLD_API int32_t cmld_engine_prefill_tokens(cmld_engine *e, int32_t seq, const int32_t *tokens, int64_t n,
                                            int64_t start_pos, uint32_t *next_token_out);
/* Greedy decode of `n_seqs` independent sequences for `n_steps` steps with one host
 * synchronisation at the end: step s feeds tokens_in (s = 0) or the previous argmax, at
 * positions[i] + s in KV slot seqs[i]; tokens_out[s][i] is the argmax after step s.
 * (forward_independent_paged_batch_q8, src/cuda_resident.rs:20482, generalised to every
 * quantisation type and to max_seqs rows.) */
CMLD_API int32_t cmld_engine_decode_greedy(cmld_engine *e, int32_t n_seqs, const int32_t *seqs,
                                           const int32_t *tokens_in, const int64_t *positions, int32_t n_steps,
                                           uint32_t *tokens_out);
/* One batched step that also returns logits [n_seqs][vocab] (may be NULL) and the residual
 * stream before the final norm [n_seqs][hidden] (may be NULL). */
CMLD_API int32_t cmld_engine_step_batch(cmld_engine *e, int32_t n_seqs, const int32_t *seqs,
                                        const int32_t *tokens_in, const int64_t *positions,
                                        uint32_t *tokens_out, float *logits_out, float *hidden_out);
/* Device time of the last decode_greedy / step_batch call, from CUDA events on the engine's
 * stream (milliseconds), and the number of kernel launches it made. */
CMLD_API int32_t cmld_engine_last_timing(const cmld_engine *e, float *ms_out, int64_t *launches_out);

/* ---- operator level: the kernels of the path, on device buffers (microbenchmarks and
 * kernel-level parity tests call these) ---- */

/* Device-resident quantised matrix [rows][cols].  `wire` is GGUF wire bytes in host or
 * device memory; the library re-lays each row out for 16-byte aligned streaming (same
 * bytes, permuted within the row). */
CMLD_API int32_t cmld_weight_create(int32_t qtype, int64_t rows, int64_t cols, const void *wire, uint64_t nbytes,
                                    cmld_weight **out);
/* Seeded synthetic matrix generated and quantised on the device: element (r,c) is the
 * N(0,sigma) deviate of counter (row0+r)*cols+c of stream `stream` under `seed`, quantised
 * with Camelid's quantize_block_q8_0 / quantize_block_q4_k (src/quantize.rs:98-119,
 * :152-244) or this project's Q6_K quantiser. */
CMLD_API int32_t cmld_weight_synth(int32_t qtype, uint64_t seed, uint64_t stream, int64_t row0, int64_t rows,
                                   int64_t cols, float sigma, cmld_weight **out);
/* A new matrix holding rows (first_block + j*block_step)*block_rows + [0, block_rows), j < n_blocks,
 * and columns [col0, col0+n_cols) of src (whole quantisation blocks: col0 and n_cols multiples of
 * 256 for K-quants, 32 for Q8_0).  Device-to-device; the shard a rank of a sharded engine adopts. */
CMLD_API int32_t cmld_weight_shard(const cmld_weight *src, int64_t block_rows, int64_t first_block, int64_t block_step,
                                   int64_t n_blocks, int64_t col0, int64_t n_cols, cmld_weight **out);
CMLD_API int32_t cmld_weight_destroy(cmld_weight *w);
CMLD_API int64_t cmld_weight_wire_bytes(const cmld_weight *w);
/* GGUF wire bytes back out (host buffer of cmld_weight_wire_bytes). */
CMLD_API int32_t cmld_weight_export_wire(const cmld_weight *w, void *wire_out_host);
/* Dequantise rows [row0,row0+nrows) to f32 (device buffer) — decode_q8_0_blocks,
 * Q4KBlock::dequantize, Q6KBlock::dequantize (src/tensor/mod.rs:5365-6067); bit-exact. */
CMLD_API int32_t cmld_weight_dequant(const cmld_weight *w, int64_t row0, int64_t nrows, float *out_dev);

/* Bytes of one quantised activation row of `cols` values (int8 codes + scales + sums). */
CMLD_API int64_t cmld_act_row_bytes(int64_t cols);
/* Quantise batch f32 rows x_dev[batch][cols] (quantize_q8_0_block / quantize_q8_k_blocks). */
CMLD_API int32_t cmld_act_quantize(int32_t act_kind, const float *x_dev, int64_t cols, int32_t batch, void *act_dev);
/* Codes and scales of a quantised activation back to the host (for parity checks):
 * codes_out[batch][cols] int8, scales_out[batch][cols/32 or cols/256] f32. */
CMLD_API int32_t cmld_act_export(int32_t act_kind, const void *act_dev, int64_t cols, int32_t batch,
                                 int8_t *codes_out, float *scales_out);
/* y_dev[batch][rows] = W . act (+ residual_dev[batch][rows] if not NULL): the fused
 * dequantise-and-matvec (q8_0_dot_rows, q4_k_dot_arm, q6_k_wire_row_dot:
 * src/inference.rs:26166, src/diffusion_gemma/refmath.rs:504, src/inference.rs:25535). */
CMLD_API int32_t cmld_gemv(const cmld_weight *w, const void *act_dev, int32_t batch, float *y_dev,
                           const float *residual_dev);
/* The sampling kernels as operators over a device logits row of n values (src/cuda_resident/sampling.cuh:
 * sample_gumbel, sample_gumbel_filtered, sample_min_p_mask: -1 undecided / 0 drop / 1 keep per token, and the
 * uniform generator).  Results come back to the host. */
CMLD_API int32_t cmld_sample_gumbel(const float *logits_dev, int32_t n, float inv_temp, uint64_t seed, uint32_t *token_out);
CMLD_API int32_t cmld_sample_gumbel_filtered(const float *logits_dev, int32_t n, float temperature, float min_p, uint64_t seed,
                                             uint32_t *token_out);
CMLD_API int32_t cmld_sample_min_p_mask(const float *logits_dev, int32_t n, float min_p, int32_t *mask_out);
CMLD_API int32_t cmld_sample_uniforms(uint64_t seed, int32_t n, float *out);

/* Which matvec kernel cmld_gemv / cmld_gemv_time use: bit 0 clear = the staged (bulk-copy
 * pipelined) kernel whenever it takes the shape, bit 0 set = the generic kernel only (both give
 * the CPU dot's bits); bit 1 set = cmld_gemv_time chains its launches with programmatic dependent
 * launch; bit 3 set = batches of 9..32 rows on the int8 mma.sync kernel (one pass over the weights,
 * tree sums: within tolerance, not the CPU's bits), bit 2 set = that kernel from 1 row.
 * Batches of 9 rows and more take the tcgen05 tensor-core kernel by default (one pass over the
 * weights per 32 rows, the CPU dot's bits); bit 4 set = never, bit 5 set = from 1 row.
 * Process-wide; for A/B runs. */
CMLD_API int32_t cmld_gemv_select_kernel(int32_t choice);
/* Self-test of the bounded device-side wait of the peer-memory path (no reference counterpart): waits for an
 * arrival word that nobody raises; returns CMLD_ERR_TIMEOUT after timeout_ms (1..5000) when the bound works,
 * CMLD_ERR_STATE otherwise.  One GPU; nothing faults or hangs. */
CMLD_API int32_t cmld_peer_wait_selftest(int32_t timeout_ms);
/* Self-test of the parallel evaluation of the sequential f32 sum that RMSNorm (rms_norm_into,
 * src/tensor/mod.rs:2740-2764) and the softmax of attention (src/inference.rs:30297-30466) use (no reference
 * counterpart): n non-negative f32 terms on the device, n a multiple of 256, at most 8192.  sums_host[0] = the
 * sum by the usual path; sums_host[1] = the same event list walked with every step checked and every second
 * run forced to be replayed term by term.  Both must be the one-accumulator loop's bits. */
CMLD_API int32_t cmld_exact_sum_selftest(const float *terms_dev, int32_t n, float *sums_host);
/* The staged kernel with its fused prologue: y = W . quantise(f(x)) (+ residual), with
 * f = RMSNorm(x) * norm_w (mode 1), x (mode 2) or SwiGLU(x, x2) (mode 3); x_dev/x2_dev are f32
 * [batch][cols], batch <= 8.  One launch replaces norm/activation kernel + quantiser + matvec. */
CMLD_API int32_t cmld_gemv_fused(const cmld_weight *w, int32_t mode, const float *x_dev, const float *x2_dev,
                                 const float *norm_w_dev, float eps, int32_t batch, float *y_dev,
                                 const float *residual_dev);
/* RMSNorm (rms_norm_into, src/tensor/mod.rs:2707): out_dev and/or act_dev may be NULL. */
CMLD_API int32_t cmld_rms_norm(const float *x_dev, const float *w_dev, int64_t cols, int32_t batch, float eps,
                               float *out_dev, int32_t act_kind, void *act_dev);
/* SwiGLU (src/inference.rs:13231-13236): out = g/(1+exp(-g))*u. */
CMLD_API int32_t cmld_silu_mul(const float *g_dev, const float *u_dev, int64_t cols, int32_t batch, float *out_dev,
                               int32_t act_kind, void *act_dev);
/* Greedy argmax (greedy_sample, src/inference.rs:8904): lowest index wins ties. */
CMLD_API int32_t cmld_argmax(const float *x_dev, int64_t n, int32_t batch, uint32_t *idx_out_host);
/* Single-query GQA attention over an f16 cache [kv_head][max_pos][head_dim]
 * (attention_context_for_head_into_with_kernels, src/inference.rs:30287): q_dev[n_heads][hd]
 * f32, n_pos cached positions, out_dev[n_heads][hd]. */
CMLD_API int32_t cmld_attention_decode(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                       int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int64_t max_pos,
                                       int64_t n_pos, float scale, float *out_dev);
/* The same attention with every f32 sum in the CPU path's order (attention_context_for_head_into_with_kernels,
 * src/inference.rs:30287-30466; dot_product, src/tensor/mod.rs:3464-3480): the kernel the engine runs by
 * default.  The output has the CPU path's bits. */
CMLD_API int32_t cmld_attention_decode_ordered(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                               int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int64_t max_pos,
                                               int64_t n_pos, float scale, float *out_dev);

/* cmld_attention_decode without any allocator call (no counterpart in the reference; added for
 * hosts that cannot call cudaMalloc when they need attention: the device is fully owned by their
 * own pool, their latency path forbids allocator calls, or their CUDA binding has no allocator).
 * The split-range partials live in a fixed ~1.2 MiB array inside the library image, present once
 * on every GPU that loads the library until the process exits.  Limits: n_heads <= 64 and
 * head_dim <= 128 (anything larger returns CMLD_ERR_SHAPE; use cmld_attention_decode).  The first
 * call on each device resolves the array's device address; make that call before starting any
 * stream capture.  All calls share the array: it keeps the previous call's bytes (the counters
 * that must start at zero are cleared on every call), and two calls that overlap on the GPU
 * race.  Same arguments and same result bits as cmld_attention_decode. */
CMLD_API int32_t cmld_attention_decode_noalloc(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                               int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int64_t max_pos,
                                               int64_t n_pos, float scale, float *out_dev);
/* Time `iters` back-to-back launches of cmld_gemv with CUDA events around one CUDA-graph replay of
 * them (so the host's enqueue rate is not measured); the weights are `n_copies` distinct matrices
 * visited round-robin so that the stream comes from HBM when their total exceeds the L2.
 * Returns the mean milliseconds per launch. */
CMLD_API int32_t cmld_gemv_time(cmld_weight *const *copies, int32_t n_copies, const void *act_dev, int32_t batch,
                                float *y_dev, int32_t warmup, int32_t iters, float *ms_per_launch_out);

#ifdef __cplusplus
}
#endif
#endif /* CAMELID_B200_H */
