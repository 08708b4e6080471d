// Generic quantised matvec: any shape, any batch, every f32 operation in the order of Camelid's CPU
// dots (the kernel itself is in exact.cu).  The staged kernel in gemv_pipe.cu is the fast path for
// the shapes it takes; this is what runs for the rest (narrow test models, widths that are not a
// multiple of 256 or that would need more chain lanes than a warp has).
#include "common.cuh"

namespace cmld {

// All jobs of one launch share `cols` and read the same activation buffer (Q8_0 jobs its Q8_0 codes,
// K-quant jobs its Q8_K codes; the caller passes the matching buffer, which for a mixed group means
// separate calls).
int32_t launch_gemv(const GemvJob *jobs, int n_jobs, const uint8_t *act, int32_t batch, cudaStream_t s) {
  if (n_jobs < 1) return fail(CMLD_ERR_INVALID, "gemv: %d jobs in one launch", n_jobs);
  for (int k = 0; k < n_jobs; ++k) {
    if (jobs[k].cols != jobs[0].cols) return fail(CMLD_ERR_SHAPE, "gemv: jobs of one launch must share cols");
    CMLD_TRY(launch_gemv_exact(jobs[k], act, batch, s));
  }
  return CMLD_OK;
}

}  // namespace cmld
