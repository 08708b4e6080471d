// Compiled by tests/test_abi.py against include/camelid_b200.h and linked with libcamelid_b200.a: the header's
// prototypes are what a caller of CudaResidentDecode::new / forward_token (src/cuda_resident.rs:15748, :19548 in
// the Camelid tree) would bind, so they have to compile as C++ and resolve against the archive.  Runs without a
// GPU: only argument checks and the error channel are exercised.
#include <cstdio>
#include <cstring>

#include "camelid_b200.h"

int main() {
  if (std::strncmp(cmld_version(), "camelid_b200", 12) != 0) return 1;
  cmld_engine *e = nullptr;
  if (cmld_engine_create(nullptr, &e) != 1) return 2;  // CMLD_ERR_INVALID
  if (std::strlen(cmld_last_error()) == 0) return 3;
  cmld_config cfg{};
  cfg.n_layers = 1, cfg.n_heads = 3, cfg.n_kv_heads = 2, cfg.head_dim = 32, cfg.hidden = 96, cfg.ffn_dim = 128;
  cfg.max_pos = 16, cfg.vocab = 96, cfg.eps = 1e-5f, cfg.rope_theta = 10000.0f, cfg.device = -1;
  const int32_t rc = cmld_engine_create(&cfg, &e);  // heads not divisible by kv heads
  if (rc == 0 || std::strstr(cmld_last_error(), "n_kv_heads") == nullptr) return 4;
  if (cmld_engine_set_filled(nullptr, 0) != 1) return 5;
  // prototypes of the per-token path: taking their addresses forces the archive to provide them
  int32_t (*fwd)(cmld_engine *, const float *, const float *, const float *, int64_t, float, int32_t, uint32_t *) = &cmld_engine_forward_token;
  int32_t (*seed)(cmld_engine *, int32_t, const float *, const float *, int64_t) = &cmld_engine_seed_layer;
  if (!fwd || !seed) return 6;
  std::printf("ok %s devices=%d\n", cmld_version(), cmld_device_count());
  return 0;
}
