// Collectives for the sharded engine: one process per GPU, NCCL over NVLink / NVSwitch.
//
// The reference has no tensor or expert parallelism (its only multi-node mode is a two-stage TCP
// pipeline, src/distributed.rs in the Camelid tree), so this is new design: a dense model is split
// tensor-parallel (q/k/v/gate/up by rows, o/down by columns on 256-value boundaries, lm_head by
// vocabulary rows) with one all-reduce of [rows][hidden] f32 per sublayer; a Mixtral-shaped model is
// split expert-parallel (expert e lives on rank e % n) with one all-reduce per MoE layer; greedy
// argmax over a sharded vocabulary is one all-reduce(max) of a packed (value, index) key.
//
// NCCL is bound at run time (dlopen), not at link time: a host process that also loads another
// copy of libnccl.so.2 (PyTorch bundles its own) must end up with exactly one, and a process that
// never shards must not need the library at all.  Order: a copy already in the process, then the
// path in CMLD_NCCL_PATH, then the loader's default search.
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <chrono>
#include <memory>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace cmld {

namespace {
struct NcclApi {
  void *handle = nullptr;
  decltype(&::ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&::ncclCommInitRank) CommInitRank = nullptr;
  decltype(&::ncclCommDestroy) CommDestroy = nullptr;
  decltype(&::ncclCommAbort) CommAbort = nullptr;
  decltype(&::ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  decltype(&::ncclAllReduce) AllReduce = nullptr;
  decltype(&::ncclAllGather) AllGather = nullptr;
  decltype(&::ncclGetErrorString) GetErrorString = nullptr;
  bool ok = false;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) {
    const char *path = getenv("CMLD_NCCL_PATH");
    if (path && *path) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  }
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return;
  g_nccl.handle = h;
  g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(dlsym(h, "ncclCommAbort"));
  g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
  g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(h, "ncclAllReduce"));
  g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(h, "ncclAllGather"));
  g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  g_nccl.ok = g_nccl.CommAbort && g_nccl.CommGetAsyncError && g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllReduce && g_nccl.AllGather &&
              g_nccl.GetErrorString;
}

int32_t need_nccl() {
  std::call_once(g_nccl_once, load_nccl);
  if (!g_nccl.ok) return fail(CMLD_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded (set CMLD_NCCL_PATH): sharded engines need NCCL");
  return CMLD_OK;
}
}  // namespace

#define CMLD_NCCL(expr)                                                                          \
  do {                                                                                           \
    ncclResult_t r__ = (expr);                                                                   \
    if (r__ != ncclSuccess && r__ != ncclInProgress)                                             \
      return ::cmld::fail(CMLD_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, g_nccl.GetErrorString(r__), __FILE__, __LINE__); \
  } while (0)

int32_t comm_unique_id(uint8_t *out128) {
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  CMLD_TRY(need_nccl());
  ncclUniqueId id;
  CMLD_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(out128, &id, 128);
  return CMLD_OK;
}

int32_t comm_init(void **comm_out, const uint8_t *id128, int rank, int world) {
  CMLD_TRY(need_nccl());
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclComm_t comm = nullptr;
  CMLD_NCCL(g_nccl.CommInitRank(&comm, world, id, rank));
  *comm_out = comm;
  return CMLD_OK;
}

// Teardown is ncclCommAbort, not ncclCommDestroy: the engine has drained its stream by then, and
// abort, unlike destroy, does not wait for the other ranks of the node to make the same call.
void comm_destroy(void *comm) {
  if (comm && g_nccl.ok) g_nccl.CommAbort(static_cast<ncclComm_t>(comm));
}

// Waits for the stream like cudaStreamSynchronize, but gives up: when the stream is still busy
// after limit_ms, or NCCL reports an asynchronous error (a peer went away), the communicator is
// aborted, which makes its kernels return, and the call reports a timeout.  *comm is null then.
int32_t comm_wait_stream(void **comm, cudaStream_t s, int64_t limit_ms, void (*before_abort)(void *), void *ctx) {
  const auto t0 = std::chrono::steady_clock::now();
  int spins = 0;
  for (;;) {
    const cudaError_t q = cudaStreamQuery(s);
    if (q == cudaSuccess) return CMLD_OK;
    if (q != cudaErrorNotReady) return fail(CMLD_ERR_CUDA, "stream failed: %s", cudaGetErrorString(q));
    bool give_up = false;
    if ((++spins & 1023) == 0) {
      ncclResult_t async = ncclSuccess;
      if (g_nccl.CommGetAsyncError(static_cast<ncclComm_t>(*comm), &async) != ncclSuccess || (async != ncclSuccess && async != ncclInProgress))
        give_up = true;
      const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms > limit_ms) give_up = true;
      if (ms > 50) std::this_thread::sleep_for(std::chrono::microseconds(200));  // long wait: stop burning a core
    }
    if (give_up) {
      const bool dbg = getenv("CMLD_DEBUG_COMM") != nullptr;
      if (dbg) fprintf(stderr, "[cmld comm] giving up on the stream; aborting the communicator\n");
      // The abort runs on a helper thread: it raises the communicator's abort flag at once (the
      // collective's kernel sees it and returns) but then waits until every CUDA graph that captured
      // the communicator is gone, and those can only be freed once the stream has drained — which is
      // this thread's job.  Every wait here is bounded; a helper that never returns is left behind.
      ncclComm_t c = static_cast<ncclComm_t>(*comm);
      *comm = nullptr;
      auto done = std::make_shared<std::atomic<bool>>(false);
      std::thread helper([c, done] {
        g_nccl.CommAbort(c);
        done->store(true);
      });
      const auto t1 = std::chrono::steady_clock::now();
      auto waited_ms = [&] { return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t1).count(); };
      while (cudaStreamQuery(s) == cudaErrorNotReady && waited_ms() < 20000) std::this_thread::sleep_for(std::chrono::milliseconds(1));
      if (dbg) fprintf(stderr, "[cmld comm] stream drained=%d after %lld ms\n", (int)(cudaStreamQuery(s) != cudaErrorNotReady), (long long)waited_ms());
      if (before_abort) before_abort(ctx);  // idle graphs are freed at once, which ends the helper's wait for them
      while (!done->load() && waited_ms() < 40000) {
        cudaStreamQuery(s);
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      if (dbg) fprintf(stderr, "[cmld comm] abort returned=%d after %lld ms\n", (int)done->load(), (long long)waited_ms());
      if (done->load()) helper.join();
      else helper.detach();
      return fail(CMLD_ERR_TIMEOUT, "a collective did not finish within %lld ms (a peer rank stopped answering): communicator aborted",
                  (long long)limit_ms);
    }
  }
}

int32_t comm_allreduce_sum_f32(void *comm, float *buf, int64_t count, cudaStream_t s) {
  CMLD_NCCL(g_nccl.AllReduce(buf, buf, (size_t)count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm), s));
  return CMLD_OK;
}

int32_t comm_allreduce_max_u64(void *comm, unsigned long long *buf, int64_t count, cudaStream_t s) {
  CMLD_NCCL(g_nccl.AllReduce(buf, buf, (size_t)count, ncclUint64, ncclMax, static_cast<ncclComm_t>(comm), s));
  return CMLD_OK;
}

int32_t comm_allgather_f32(void *comm, const float *send, float *recv, int64_t count_per_rank, cudaStream_t s) {
  CMLD_NCCL(g_nccl.AllGather(send, recv, (size_t)count_per_rank, ncclFloat32, static_cast<ncclComm_t>(comm), s));
  return CMLD_OK;
}

}  // namespace cmld
