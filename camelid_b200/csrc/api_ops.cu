// Operator-level C ABI: the kernels of the decode path on caller-owned device buffers.
// Used by the microbenchmarks and the kernel-level parity tests; all work runs on the
// calling thread's current device, default stream, and returns after completion.
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace cmld {
int32_t weight_alloc(Weight &w, int32_t qt, int64_t rows, int64_t cols);
void weight_free(Weight &w);
int32_t weight_upload(Weight &w, int32_t qt, int64_t rows, int64_t cols, const void *wire, uint64_t nbytes, cudaStream_t s);
}  // namespace cmld

using namespace cmld;

static int32_t sync_ok(const char *what) {
  cudaError_t ce = cudaStreamSynchronize(nullptr);
  if (ce != cudaSuccess) return fail(CMLD_ERR_CUDA, "%s: %s", what, cudaGetErrorString(ce));
  return CMLD_OK;
}

// Status word for the staged kernel's bounded waits, one per device, made on first use.
static int32_t *op_status(void) {
  static int32_t *words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], 4) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, 4);
  }
  return words[dev];
}

// Partial-sum scratch of the batched matvec for the operator-level calls: one per device, grown on demand
// (never inside a stream capture: a capture is preceded by warm-up launches of the same shape).
static float *op_scratch(int64_t floats) {
  static float *buf[64] = {nullptr};
  static int64_t cap[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cap[dev] < floats) {
    if (buf[dev]) {
      cudaDeviceSynchronize();
      cudaFree(buf[dev]);
    }
    buf[dev] = nullptr;
    cap[dev] = 0;
    if (cudaMalloc(&buf[dev], (size_t)floats * 4) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cap[dev] = floats;
  }
  return buf[dev];
}

static int32_t check_op_status(const char *what) {
  int32_t *w = op_status(), st = 0;
  if (!w) return CMLD_OK;
  if (cudaMemcpy(&st, w, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return fail(CMLD_ERR_CUDA, "%s: status read failed", what);
  if (st != 0) {
    cudaMemset(w, 0, 4);
    return fail(st, "%s: a bounded device-side wait gave up (status %d)", what, st);
  }
  return CMLD_OK;
}

static int g_gemv_pdl = 0;            // cmld_gemv_time: chain its launches with programmatic dependent launch
static int g_gemv_kernel_choice = 0;  // 0 auto (staged when the shape fits), 1 generic kernel only
static int g_gemv_mma_min_batch = 1 << 30;  // rows from which the int8 mma.sync kernel is used (opt-in: bit 3 of the choice from 9 rows, bit 2 from 1)
static int g_gemv_tc5_min_batch = 9;        // rows from which the tcgen05 kernel is used (bit 4 of the choice: never; bit 5: from 1 row)

// One matvec launch on the default stream: staged kernel if it takes the shape, else the generic one.
static int32_t gemv_launch(const cmld_weight *w, const uint8_t *act, int32_t batch, float *y, const float *residual,
                           cudaStream_t stream = nullptr, bool pdl = false) {
  GemvJob probe{w->data, w->qt, w->rows, w->cols, w->stride, y, residual, w->rows};
  if (g_gemv_kernel_choice == 0 && batch >= g_gemv_tc5_min_batch && batch < g_gemv_mma_min_batch && gemv_tc5_fits(&probe, 1, std::min(batch, 32))) {
    // several rows: one pass over the weights per 32 rows on the tcgen05 tensor cores, same bits as the one-row kernels
    const int64_t need = gemv_tc5_pack_bytes(w->cols);
    uint8_t *pack = reinterpret_cast<uint8_t *>(op_scratch((need + 3) / 4));
    if (!pack) return fail(CMLD_ERR_OOM, "gemv: no room for %lld bytes of packed activations", (long long)need);
    for (int b0 = 0; b0 < batch; b0 += 32) {
      const int nb = std::min(32, batch - b0);
      GemvJob j{w->data, w->qt, w->rows, w->cols, w->stride, y + (int64_t)b0 * w->rows, residual ? residual + (int64_t)b0 * w->rows : nullptr, w->rows};
      CMLD_TRY(launch_gemv_tc5(&j, 1, act + (int64_t)b0 * act_row_stride(w->cols), nb, pack, need, op_status(), stream, nullptr));
    }
    return CMLD_OK;
  }
  if (g_gemv_kernel_choice == 0 && batch >= g_gemv_mma_min_batch && batch <= 32) {
    // more than 8 rows: one pass over the weights on the tensor cores
    const int64_t need = gemv_mma_scratch_floats(&probe, 1, batch);
    if (need >= 0) {
      float *scratch = need > 0 ? op_scratch(need) : nullptr;
      if (need > 0 && !scratch) return fail(CMLD_ERR_OOM, "gemv: no room for %lld floats of partial sums", (long long)need);
      const int32_t rc = launch_gemv_mma(&probe, 1, act, batch, scratch, need, op_status(), stream, pdl, nullptr);
      if (rc != CMLD_ERR_UNSUPPORTED) return rc;
    }
  }
  const int fit = g_gemv_kernel_choice == 0 ? gemv_pipe_fit_batch(&probe, 1) : 0;
  const int pass = fit > 0 ? fit : 8;
  for (int b0 = 0; b0 < batch; b0 += pass) {
    const int nb = std::min(pass, batch - b0);
    GemvJob j{w->data, w->qt, w->rows, w->cols, w->stride, y + (int64_t)b0 * w->rows, residual ? residual + (int64_t)b0 * w->rows : nullptr, w->rows};
    const uint8_t *a = act + (int64_t)b0 * act_row_stride(w->cols);
    int32_t rc = CMLD_ERR_UNSUPPORTED;
    if (fit > 0) {
      GemvPrologue pro{};
      pro.mode = 0;
      pro.act_k = pro.act_0 = a;
      rc = launch_gemv_pipe(&j, 1, nb, pro, op_status(), stream, pdl);
    }
    if (rc == CMLD_ERR_UNSUPPORTED) rc = launch_gemv(&j, 1, a, nb, stream);
    CMLD_TRY(rc);
  }
  return CMLD_OK;
}

// One CTA per destination row: up to two byte ranges of the source row (the block bytes, and the
// per-row scale array that the Q8_0 and Q6_K layouts keep behind them).
struct ShardSeg {
  int64_t src_off, dst_off, len;
};
__global__ void weight_shard_kernel(const uint8_t *__restrict__ src, int64_t src_stride, uint8_t *__restrict__ dst,
                                    int64_t dst_stride, int64_t block_rows, int64_t first_block, int64_t block_step,
                                    ShardSeg s0, ShardSeg s1) {
  const int64_t r = blockIdx.x;
  const int64_t src_row = (first_block + (r / block_rows) * block_step) * block_rows + r % block_rows;
  const uint8_t *sp = src + src_row * src_stride;
  uint8_t *dp = dst + r * dst_stride;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const ShardSeg g = k ? s1 : s0;
    if (((g.src_off | g.dst_off | g.len | src_stride | dst_stride) & 15) == 0) {
      const uint4 *a = reinterpret_cast<const uint4 *>(sp + g.src_off);
      uint4 *b = reinterpret_cast<uint4 *>(dp + g.dst_off);
      for (int64_t i = threadIdx.x; i < g.len / 16; i += blockDim.x) b[i] = a[i];
    } else {
      for (int64_t i = threadIdx.x; i < g.len; i += blockDim.x) dp[g.dst_off + i] = sp[g.src_off + i];
    }
  }
}

extern "C" {

int32_t cmld_weight_shard(const cmld_weight *src, int64_t block_rows, int64_t first_block, int64_t block_step,
                          int64_t n_blocks, int64_t col0, int64_t n_cols, cmld_weight **out) {
  if (!src || !out) return fail(CMLD_ERR_INVALID, "null weight or out pointer");
  *out = nullptr;
  if (block_rows <= 0 || n_blocks <= 0 || first_block < 0 || block_step < 1 ||
      (first_block + (n_blocks - 1) * block_step + 1) * block_rows > src->rows)
    return fail(CMLD_ERR_SHAPE, "row blocks %lld + %lld*k (k < %lld) of %lld rows leave the %lld-row tensor",
                (long long)first_block, (long long)block_step, (long long)n_blocks, (long long)block_rows, (long long)src->rows);
  const int64_t blk = src->qt == CMLD_F32 ? 1 : (src->qt == CMLD_Q8_0 ? 32 : 256);
  if (col0 < 0 || n_cols <= 0 || col0 + n_cols > src->cols || col0 % blk || n_cols % blk)
    return fail(CMLD_ERR_SHAPE, "columns %lld..%lld are not whole %lld-value blocks of the %lld-column tensor", (long long)col0,
                (long long)(col0 + n_cols), (long long)blk, (long long)src->cols);
  cmld_weight *w = new cmld_weight();
  int32_t rc = weight_alloc(*w, src->qt, block_rows * n_blocks, n_cols);
  if (rc != CMLD_OK) {
    delete w;
    return rc;
  }
  ShardSeg s0{0, 0, 0}, s1{0, 0, 0};
  switch (src->qt) {
    case CMLD_F32: s0 = {col0 * 4, 0, n_cols * 4}; break;
    case CMLD_Q4_K: s0 = {col0 / 256 * 144, 0, n_cols / 256 * 144}; break;
    case CMLD_Q6_K:
      s0 = {col0 / 256 * 208, 0, n_cols / 256 * 208};
      s1 = {src->cols / 256 * 208 + col0 / 256 * 2, n_cols / 256 * 208, n_cols / 256 * 2};
      break;
    default:  // Q8_0
      s0 = {col0, 0, n_cols};
      s1 = {src->cols + col0 / 32 * 2, n_cols, n_cols / 32 * 2};
      break;
  }
  // the padding behind a row is never read as data, but keep it defined
  cudaError_t ce = cudaMemset(w->data, 0, (size_t)(w->rows * w->stride));
  if (ce == cudaSuccess) {
    weight_shard_kernel<<<(unsigned)w->rows, 256>>>(src->data, src->stride, w->data, w->stride, block_rows, first_block,
                                                    block_step, s0, s1);
    ce = cudaGetLastError();
  }
  if (ce == cudaSuccess) rc = sync_ok("weight_shard");
  else rc = fail(CMLD_ERR_CUDA, "weight_shard: %s", cudaGetErrorString(ce));
  if (rc != CMLD_OK) {
    weight_free(*w);
    delete w;
    return rc;
  }
  *out = w;
  return CMLD_OK;
}

int32_t cmld_weight_create(int32_t qtype, int64_t rows, int64_t cols, const void *wire, uint64_t nbytes, cmld_weight **out) {
  if (!out) return fail(CMLD_ERR_INVALID, "null out pointer");
  *out = nullptr;
  cmld_weight *w = new cmld_weight();
  int32_t rc = weight_upload(*w, qtype, rows, cols, wire, nbytes, nullptr);
  if (rc != CMLD_OK) {
    weight_free(*w);
    delete w;
    return rc;
  }
  *out = w;
  return CMLD_OK;
}

int32_t cmld_weight_synth(int32_t qtype, uint64_t seed, uint64_t stream, int64_t row0, int64_t rows, int64_t cols,
                          float sigma, cmld_weight **out) {
  if (!out) return fail(CMLD_ERR_INVALID, "null out pointer");
  *out = nullptr;
  if (qtype == CMLD_Q8_0_HOST36) return fail(CMLD_ERR_UNSUPPORTED, "synthetic weights are generated in wire types only");
  cmld_weight *w = new cmld_weight();
  int32_t rc = weight_alloc(*w, qtype, rows, cols);
  if (rc == CMLD_OK) rc = launch_synth(*w, seed, stream, row0, sigma, nullptr);
  if (rc == CMLD_OK) rc = sync_ok("weight_synth");
  if (rc != CMLD_OK) {
    weight_free(*w);
    delete w;
    return rc;
  }
  *out = w;
  return CMLD_OK;
}

int32_t cmld_weight_destroy(cmld_weight *w) {
  if (!w) return CMLD_OK;
  weight_free(*w);
  delete w;
  return CMLD_OK;
}

int64_t cmld_weight_wire_bytes(const cmld_weight *w) { return w ? wire_row_bytes(w->qt, w->cols) * w->rows : 0; }

int32_t cmld_weight_export_wire(const cmld_weight *w, void *wire_out_host) {
  if (!w || !wire_out_host) return fail(CMLD_ERR_INVALID, "null weight or output");
  const int64_t n = cmld_weight_wire_bytes(w);
  if (w->qt == CMLD_F32) {
    CMLD_CUDA(cudaMemcpy(wire_out_host, w->data, (size_t)n, cudaMemcpyDeviceToHost));
    return CMLD_OK;
  }
  uint8_t *tmp = nullptr;
  CMLD_CUDA(cudaMalloc(&tmp, (size_t)n));
  int32_t rc = launch_unpack_to_wire(*w, tmp, nullptr);
  if (rc == CMLD_OK && cudaMemcpy(wire_out_host, tmp, (size_t)n, cudaMemcpyDeviceToHost) != cudaSuccess)
    rc = fail(CMLD_ERR_CUDA, "export copy failed");
  cudaFree(tmp);
  return rc;
}

int32_t cmld_weight_dequant(const cmld_weight *w, int64_t row0, int64_t nrows, float *out_dev) {
  if (!w || !out_dev) return fail(CMLD_ERR_INVALID, "null weight or output");
  if (row0 < 0 || nrows < 0 || row0 + nrows > w->rows) return fail(CMLD_ERR_INVALID, "rows %lld+%lld out of range", (long long)row0, (long long)nrows);
  CMLD_TRY(launch_dequant(*w, row0, nrows, out_dev, nullptr));
  return sync_ok("weight_dequant");
}

int64_t cmld_act_row_bytes(int64_t cols) { return act_row_stride(cols); }

int32_t cmld_act_quantize(int32_t act_kind, const float *x_dev, int64_t cols, int32_t batch, void *act_dev) {
  if (!x_dev || !act_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (act_kind != CMLD_ACT_Q8_0 && act_kind != CMLD_ACT_Q8_K) return fail(CMLD_ERR_INVALID, "unknown activation format %d", act_kind);
  NormQuantArgs a{};
  a.x = x_dev;
  a.cols = cols;
  a.batch = batch;
  a.act = static_cast<uint8_t *>(act_dev);
  a.act2 = a.act;
  a.act_q8_0 = act_kind == CMLD_ACT_Q8_0;
  a.act_q8_k = act_kind == CMLD_ACT_Q8_K;
  CMLD_TRY(launch_norm_quant(a, nullptr));
  return sync_ok("act_quantize");
}

int32_t cmld_act_export(int32_t act_kind, const void *act_dev, int64_t cols, int32_t batch, int8_t *codes_out, float *scales_out) {
  if (!act_dev || !codes_out || !scales_out) return fail(CMLD_ERR_INVALID, "null buffer");
  const int64_t stride = act_row_stride(cols);
  const int64_t nsc = act_kind == CMLD_ACT_Q8_0 ? cols / 32 : cols / 256;
  const uint8_t *a = static_cast<const uint8_t *>(act_dev);
  for (int b = 0; b < batch; ++b) {
    CMLD_CUDA(cudaMemcpy(codes_out + (int64_t)b * cols, a + b * stride, (size_t)cols, cudaMemcpyDeviceToHost));
    CMLD_CUDA(cudaMemcpy(scales_out + (int64_t)b * nsc, a + b * stride + act_scale_off(cols), (size_t)nsc * 4, cudaMemcpyDeviceToHost));
  }
  return CMLD_OK;
}

int32_t cmld_gemv(const cmld_weight *w, const void *act_dev, int32_t batch, float *y_dev, const float *residual_dev) {
  if (!w || !act_dev || !y_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (w->qt == CMLD_F32) return fail(CMLD_ERR_UNSUPPORTED, "gemv over f32 weights is not part of this path");
  if (batch < 1) return fail(CMLD_ERR_INVALID, "batch %d", batch);
  CMLD_TRY(gemv_launch(w, static_cast<const uint8_t *>(act_dev), batch, y_dev, residual_dev));
  CMLD_TRY(sync_ok("gemv"));
  return check_op_status("gemv");
}

// The parallel evaluation of the sequential f32 sum on n device-resident non-negative terms: sums_host[0] by the
// usual path, sums_host[1] by walking the same event list with every step checked and every second run forced to
// be replayed term by term.  Both must equal the one-accumulator loop bit for bit.
int32_t cmld_exact_sum_selftest(const float *terms_dev, int32_t n, float *sums_host) {
  if (!terms_dev || !sums_host) return fail(CMLD_ERR_INVALID, "exact sum self-test: null argument");
  float *out = nullptr;
  CMLD_CUDA(cudaMalloc(&out, 2 * sizeof(float)));
  int32_t rc = launch_exact_sum_selftest(terms_dev, n, out, nullptr);
  if (rc == CMLD_OK && cudaMemcpy(sums_host, out, 2 * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess)
    rc = fail(CMLD_ERR_CUDA, "exact sum self-test: %s", cudaGetErrorString(cudaGetLastError()));
  cudaFree(out);
  return rc;
}

// Runs the receiving side of a peer-memory sum against an arrival word that nobody raises: the wait must run
// out after timeout_ms, record the status word and let the kernel finish.  Returns what the status word said
// (CMLD_ERR_TIMEOUT when the bound works); the context stays usable.
int32_t cmld_peer_wait_selftest(int32_t timeout_ms) {
  if (timeout_ms < 1 || timeout_ms > 5000) return fail(CMLD_ERR_INVALID, "timeout_ms %d out of 1..=5000", timeout_ms);
  const int hidden = 256;
  uint8_t *buf = nullptr;
  CMLD_CUDA(cudaMalloc(&buf, (size_t)(2 * kPeerRows * hidden + hidden) * 4 + 64));
  cudaMemset(buf, 0, (size_t)(2 * kPeerRows * hidden + hidden) * 4 + 64);
  float *parts = reinterpret_cast<float *>(buf), *out = parts + 2 * kPeerRows * hidden;
  uint32_t *flag = reinterpret_cast<uint32_t *>(out + hidden), *epoch = flag + 2;
  const uint32_t one = 1;
  cudaMemcpy(epoch, &one, 4, cudaMemcpyHostToDevice);  // one arrival expected, none will come
  GemvPeer rx{};
  rx.rx_n = 2;
  rx.rx_part = parts;
  rx.rx_flag = flag;
  rx.rx_epoch = epoch;
  rx.rx_out = out;
  rx.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  int32_t rc = launch_peer_reduce(rx, 1, hidden, op_status(), false, nullptr);
  if (rc == CMLD_OK) rc = sync_ok("peer_wait_selftest");
  int32_t st = 0;
  if (rc == CMLD_OK && cudaMemcpy(&st, op_status(), 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "status read failed");
  cudaMemset(op_status(), 0, 4);
  cudaFree(buf);
  if (rc != CMLD_OK) return rc;
  if (st == CMLD_ERR_TIMEOUT) return fail(CMLD_ERR_TIMEOUT, "the wait ran out after %d ms as it should", timeout_ms);
  return fail(CMLD_ERR_STATE, "the wait did not report a timeout (status %d)", st);
}

// Sampling over a logits row on the device (sample_gumbel, sample_gumbel_filtered, sample_min_p_mask and the uniform
// generator of src/cuda_resident/sampling.cuh), results returned to the host.
static int32_t sample_fetch(uint32_t *dev, uint32_t *host, const char *what) {
  CMLD_TRY(sync_ok(what));
  CMLD_CUDA(cudaMemcpy(host, dev, 4, cudaMemcpyDeviceToHost));
  return CMLD_OK;
}
int32_t cmld_sample_gumbel(const float *logits_dev, int32_t n, float inv_temp, uint64_t seed, uint32_t *token_out) {
  if (!logits_dev || !token_out || n < 1) return fail(CMLD_ERR_INVALID, "sample_gumbel: bad arguments");
  uint32_t *d = reinterpret_cast<uint32_t *>(op_scratch(1));
  if (!d) return fail(CMLD_ERR_OOM, "sample_gumbel: no scratch");
  CMLD_TRY(launch_sample_gumbel(logits_dev, n, inv_temp, seed, d, nullptr));
  return sample_fetch(d, token_out, "sample_gumbel");
}
int32_t cmld_sample_gumbel_filtered(const float *logits_dev, int32_t n, float temperature, float min_p, uint64_t seed, uint32_t *token_out) {
  if (!logits_dev || !token_out || n < 1) return fail(CMLD_ERR_INVALID, "sample_gumbel_filtered: bad arguments");
  uint32_t *d = reinterpret_cast<uint32_t *>(op_scratch(1));
  if (!d) return fail(CMLD_ERR_OOM, "sample_gumbel_filtered: no scratch");
  CMLD_TRY(launch_sample_gumbel_filtered(logits_dev, n, temperature, min_p, seed, d, nullptr));
  return sample_fetch(d, token_out, "sample_gumbel_filtered");
}
int32_t cmld_sample_min_p_mask(const float *logits_dev, int32_t n, float min_p, int32_t *mask_out) {
  if (!logits_dev || !mask_out || n < 1) return fail(CMLD_ERR_INVALID, "sample_min_p_mask: bad arguments");
  int32_t *d = reinterpret_cast<int32_t *>(op_scratch(n));
  if (!d) return fail(CMLD_ERR_OOM, "sample_min_p_mask: no scratch");
  CMLD_TRY(launch_min_p_mask(logits_dev, n, min_p, d, nullptr));
  CMLD_TRY(sync_ok("sample_min_p_mask"));
  CMLD_CUDA(cudaMemcpy(mask_out, d, (size_t)n * 4, cudaMemcpyDeviceToHost));
  return CMLD_OK;
}
int32_t cmld_sample_uniforms(uint64_t seed, int32_t n, float *out) {
  if (!out || n < 1) return fail(CMLD_ERR_INVALID, "sample_uniforms: bad arguments");
  float *d = op_scratch(n);
  if (!d) return fail(CMLD_ERR_OOM, "sample_uniforms: no scratch");
  CMLD_TRY(launch_sample_uniforms(seed, n, d, nullptr));
  CMLD_TRY(sync_ok("sample_uniforms"));
  CMLD_CUDA(cudaMemcpy(out, d, (size_t)n * 4, cudaMemcpyDeviceToHost));
  return CMLD_OK;
}

int32_t cmld_gemv_select_kernel(int32_t choice) {
  if (choice < 0 || choice > 63) return fail(CMLD_ERR_INVALID, "kernel choice %d", choice);
  g_gemv_kernel_choice = choice & 1;
  g_gemv_pdl = (choice >> 1) & 1;
  g_gemv_mma_min_batch = (choice & 4) ? 1 : ((choice & 8) ? 9 : (1 << 30));
  g_gemv_tc5_min_batch = (choice & 16) ? (1 << 30) : ((choice & 32) ? 1 : 9);
  return CMLD_OK;
}

int32_t cmld_gemv_fused(const cmld_weight *w, int32_t mode, const float *x_dev, const float *x2_dev, const float *norm_w_dev,
                        float eps, int32_t batch, float *y_dev, const float *residual_dev) {
  if (!w || !x_dev || !y_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (mode < 1 || mode > 3) return fail(CMLD_ERR_INVALID, "mode %d not in 1..3", mode);
  if ((mode == 1 && !norm_w_dev) || (mode == 3 && !x2_dev)) return fail(CMLD_ERR_INVALID, "missing operand for mode %d", mode);
  if (w->qt == CMLD_F32) return fail(CMLD_ERR_UNSUPPORTED, "gemv over f32 weights is not part of this path");
  if (batch < 1 || batch > 8) return fail(CMLD_ERR_INVALID, "batch %d not in 1..8", batch);
  GemvJob j{w->data, w->qt, w->rows, w->cols, w->stride, y_dev, residual_dev, w->rows};
  GemvPrologue pro{};
  pro.mode = mode;
  pro.x = x_dev;
  pro.x2 = x2_dev;
  pro.norm_w = norm_w_dev;
  pro.x_stride = w->cols;
  pro.eps = eps;
  const int32_t rc = launch_gemv_pipe(&j, 1, batch, pro, op_status(), nullptr, false);
  if (rc == CMLD_ERR_UNSUPPORTED) return fail(rc, "the staged kernel does not take a %lld x %lld matrix at batch %d", (long long)w->rows, (long long)w->cols, batch);
  CMLD_TRY(rc);
  CMLD_TRY(sync_ok("gemv_fused"));
  return check_op_status("gemv_fused");
}

int32_t cmld_gemv_time(cmld_weight *const *copies, int32_t n_copies, const void *act_dev, int32_t batch, float *y_dev,
                       int32_t warmup, int32_t iters, float *ms_per_launch_out) {
  if (!copies || n_copies < 1 || !act_dev || !y_dev || !ms_per_launch_out || iters < 1) return fail(CMLD_ERR_INVALID, "bad arguments");
  for (int i = 0; i < n_copies; ++i)
    if (!copies[i] || copies[i]->qt == CMLD_F32) return fail(CMLD_ERR_INVALID, "bad weight %d", i);
  // The launches are captured into one CUDA graph so that the host's enqueue rate is not what
  // is measured; the graph is replayed once untimed (with the warm-up launches) and once timed.
  cudaStream_t st = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  CMLD_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  CMLD_CUDA(cudaEventCreate(&e0));
  CMLD_CUDA(cudaEventCreate(&e1));
  op_status();  // make the status word before capture
  int32_t rc = CMLD_OK;
  const uint8_t *act = static_cast<const uint8_t *>(act_dev);
  for (int it = 0; it < warmup && rc == CMLD_OK; ++it) rc = gemv_launch(copies[it % n_copies], act, batch, y_dev, nullptr, st, false);
  if (rc == CMLD_OK && cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "graph capture failed to start");
  if (rc == CMLD_OK) {
    for (int it = 0; it < iters && rc == CMLD_OK; ++it) rc = gemv_launch(copies[it % n_copies], act, batch, y_dev, nullptr, st, g_gemv_pdl != 0);
    cudaError_t ce = cudaStreamEndCapture(st, &graph);
    if (rc == CMLD_OK && ce != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
  }
  if (rc == CMLD_OK && cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "graph instantiate failed");
  if (rc == CMLD_OK) {
    cudaGraphLaunch(exec, st);
    cudaEventRecord(e0, st);
    cudaGraphLaunch(exec, st);
    cudaEventRecord(e1, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) rc = fail(CMLD_ERR_CUDA, "gemv_time: %s", cudaGetErrorString(cudaGetLastError()));
  }
  if (rc == CMLD_OK) rc = check_op_status("gemv_time");
  float ms = 0.0f;
  if (rc == CMLD_OK) cudaEventElapsedTime(&ms, e0, e1);
  if (exec) cudaGraphExecDestroy(exec);
  if (graph) cudaGraphDestroy(graph);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(st);
  *ms_per_launch_out = ms / (float)iters;
  return rc;
}

int32_t cmld_rms_norm(const float *x_dev, const float *w_dev, int64_t cols, int32_t batch, float eps, float *out_dev,
                      int32_t act_kind, void *act_dev) {
  if (!x_dev || !w_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  NormQuantArgs a{};
  a.x = x_dev;
  a.weight = w_dev;
  a.eps = eps;
  a.cols = cols;
  a.batch = batch;
  a.out = out_dev;
  a.act = a.act2 = static_cast<uint8_t *>(act_dev);
  a.act_q8_0 = act_dev && act_kind == CMLD_ACT_Q8_0;
  a.act_q8_k = act_dev && act_kind == CMLD_ACT_Q8_K;
  CMLD_TRY(launch_norm_quant(a, nullptr));
  return sync_ok("rms_norm");
}

int32_t cmld_silu_mul(const float *g_dev, const float *u_dev, int64_t cols, int32_t batch, float *out_dev, int32_t act_kind,
                      void *act_dev) {
  if (!g_dev || !u_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  NormQuantArgs a{};
  a.x = g_dev;
  a.x2 = u_dev;
  a.cols = cols;
  a.batch = batch;
  a.out = out_dev;
  a.act = a.act2 = static_cast<uint8_t *>(act_dev);
  a.act_q8_0 = act_dev && act_kind == CMLD_ACT_Q8_0;
  a.act_q8_k = act_dev && act_kind == CMLD_ACT_Q8_K;
  CMLD_TRY(launch_norm_quant(a, nullptr));
  return sync_ok("silu_mul");
}

int32_t cmld_argmax(const float *x_dev, int64_t n, int32_t batch, uint32_t *idx_out_host) {
  if (!x_dev || !idx_out_host || n < 1 || batch < 1) return fail(CMLD_ERR_INVALID, "bad arguments");
  const int nb = argmax_blocks();
  uint8_t *scratch = nullptr;
  const size_t bytes = (size_t)batch * nb * 8 + (size_t)batch * 8 + (size_t)batch * 4;
  CMLD_CUDA(cudaMalloc(&scratch, bytes));
  cudaMemset(scratch, 0, bytes);
  float *pv = reinterpret_cast<float *>(scratch);
  int32_t *pi = reinterpret_cast<int32_t *>(scratch + (size_t)batch * nb * 4);
  uint32_t *ticket = reinterpret_cast<uint32_t *>(scratch + (size_t)batch * nb * 8);
  int32_t *out = reinterpret_cast<int32_t *>(scratch + (size_t)batch * nb * 8 + (size_t)batch * 8);
  int32_t rc = launch_argmax(x_dev, n, batch, pv, pi, ticket, out, nullptr, nullptr, nullptr, nullptr);
  std::vector<int32_t> host(batch);
  if (rc == CMLD_OK && cudaMemcpy(host.data(), out, (size_t)batch * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
    rc = fail(CMLD_ERR_CUDA, "argmax copy failed");
  cudaFree(scratch);
  for (int i = 0; i < batch && rc == CMLD_OK; ++i) idx_out_host[i] = (uint32_t)host[i];
  return rc;
}

int32_t cmld_attention_decode(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev, int32_t n_heads,
                              int32_t n_kv_heads, int32_t head_dim, int64_t max_pos, int64_t n_pos, float scale, float *out_dev) {
  if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (n_pos < 1 || n_pos > max_pos) return fail(CMLD_ERR_INVALID, "n_pos %lld out of range", (long long)n_pos);
  const int n_splits = (int)std::max<int64_t>(1, std::min<int64_t>(37, max_pos / 32));
  const size_t part_bytes = (size_t)n_heads * n_splits * (head_dim + 2) * 4;
  uint8_t *scratch = nullptr;
  CMLD_CUDA(cudaMalloc(&scratch, part_bytes + (size_t)n_kv_heads * 4 + 8));
  cudaMemset(scratch, 0, part_bytes + (size_t)n_kv_heads * 4 + 8);
  int32_t *pos_slot = reinterpret_cast<int32_t *>(scratch + part_bytes + (size_t)n_kv_heads * 4);
  const int32_t ps[2] = {(int32_t)(n_pos - 1), 0};
  cudaMemcpy(pos_slot, ps, 8, cudaMemcpyHostToDevice);
  AttnArgs a{};
  a.q = q_dev;
  a.k_cache = static_cast<const __half *>(k_cache_dev);
  a.v_cache = static_cast<const __half *>(v_cache_dev);
  a.positions = pos_slot;
  a.slots = pos_slot + 1;
  a.n_heads = n_heads;
  a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim;
  a.batch = 1;
  a.n_splits = n_splits;
  a.max_pos = max_pos;
  a.scale = scale;
  a.part = reinterpret_cast<float *>(scratch);
  a.tickets = reinterpret_cast<uint32_t *>(scratch + part_bytes);
  a.out = out_dev;
  a.q_stride = (int64_t)n_heads * head_dim;
  a.cluster = n_pos <= 2048 ? 1 : 0;  // the engine's rule: short contexts merge their ranges inside a cluster
  int32_t rc = launch_attention(a, nullptr);
  if (rc == CMLD_OK) rc = sync_ok("attention_decode");
  cudaFree(scratch);
  return rc;
}

// The reference-order attention of the decode step (attn_ordered.cu; contexts it does not take use the
// plain reference-order kernel): the output has the CPU path's bits.
int32_t cmld_attention_decode_ordered(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev, int32_t n_heads,
                                      int32_t n_kv_heads, int32_t head_dim, int64_t max_pos, int64_t n_pos, float scale,
                                      float *out_dev) {
  if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(CMLD_ERR_INVALID, "null buffer");
  if (n_pos < 1 || n_pos > max_pos) return fail(CMLD_ERR_INVALID, "n_pos %lld out of range", (long long)n_pos);
  if (n_kv_heads < 1 || n_heads % n_kv_heads) return fail(CMLD_ERR_SHAPE, "n_heads must be a multiple of n_kv_heads");
  int32_t *pos_slot = nullptr;
  CMLD_CUDA(cudaMalloc(&pos_slot, 8));
  const int32_t ps[2] = {(int32_t)(n_pos - 1), 0};
  cudaMemcpy(pos_slot, ps, 8, cudaMemcpyHostToDevice);
  AttnArgs a{};
  a.q = q_dev;
  a.k_cache = static_cast<const __half *>(k_cache_dev);
  a.v_cache = static_cast<const __half *>(v_cache_dev);
  a.positions = pos_slot;
  a.slots = pos_slot + 1;
  a.n_heads = n_heads;
  a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim;
  a.batch = 1;
  a.n_splits = 1;
  a.max_pos = max_pos;
  a.scale = scale;
  a.out = out_dev;
  a.q_stride = (int64_t)n_heads * head_dim;
  int64_t cap = 0;
  for (int64_t c : {1024, 2048, 4096, 8192})
    if (cap == 0 && n_pos <= c) cap = c;
  // CMLD_ATTN_PHASES=1: print where the cluster kernel's time goes (CTA 0's clock at the end of each phase)
  unsigned long long *phases = nullptr;
  if (getenv("CMLD_ATTN_PHASES") && cudaMalloc(&phases, 64) == cudaSuccess) cudaMemset(phases, 0, 64);
  a.phase_ns = phases;
  int32_t rc;
  if (cap > 0 && attention_ordered_fits(n_heads, n_kv_heads, head_dim, cap)) rc = launch_attention_ordered(a, cap, nullptr);
  else rc = launch_attention_exact(a, nullptr);
  if (rc == CMLD_OK) rc = sync_ok("attention_decode_ordered");
  if (phases) {
    unsigned long long h[8] = {0};
    cudaMemcpy(h, phases, 64, cudaMemcpyDeviceToHost);
    if (h[5])
      fprintf(stderr, "attention phases (us): scores %.2f, maxima %.2f, weights %.2f, sums %.2f, scaling %.2f, chains %.2f\n", (h[1] - h[0]) * 1e-3,
              (h[2] - h[1]) * 1e-3, (h[3] - h[2]) * 1e-3, (h[4] - h[3]) * 1e-3, (h[6] - h[4]) * 1e-3, (h[5] - h[6]) * 1e-3);
    cudaFree(phases);
  }
  cudaFree(pos_slot);
  return rc;
}

}  // extern "C"
