// The launch sequence of the tensor-core GCA backward (bf16, S = L = D = 64).
//
// Two passes over the retrieved (query chunk, slot) pairs, in this order:
//   1. q-major  (gca_bwd_q_sm100.cu):  dQ, the dw partials, and for every (row, slot) the two
//      per-row terms the other pass needs, (log2|w| - LSE) / c and -Di, into the workspace;
//   2. kv-major (gca_bwd_kv_sm100.cu): dK, dV over the inverse retrieval index, with the scores
//      recomputed TRANSPOSED and the per-row terms added through one extra MMA K step.
// The reference splits its backward the same way and hands Di from one kernel to the other
// (ltriton/gca.py:318-410 -> :484-572 through `delta`, stored :385, loaded :459).  Neither pass
// uses atomics, so gradients are bit-reproducible.
#include "gca_common.cuh"

namespace gca {

int launch_bwd_kv_tc(const GcaBwdArgs& a, const Csr& csr, const uint4* rowterm, int sms, cudaStream_t stream);
int launch_bwd_q_tc(const GcaBwdArgs& a, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream);

bool bwd_tc_available() { return true; }

// partials per (row block, head, slot) that the q-major pass writes: one per 16-row quarter
int bwd_tc_dw_parts() { return 4; }

// Stage order inside one call: the q-major pass first (it writes the per-row terms), then the
// kv-major pass, which reads them.  A caller that runs the stages in separate calls must keep
// that order on the stream (or synchronise between them).
int launch_bwd_tc(const GcaBwdArgs& a, const Csr& csr, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream, unsigned stages) {
  if (a.dtype != GCA_BF16 || a.S != 64 || a.L != 64 || a.D != 64 || a.K > 32) return GCA_ERR_ALGO;
  int rc;
  if (stages & GCA_BWD_STAGE_Q) {
    if ((rc = launch_bwd_q_tc(a, dw_part, rowterm, sms, stream))) return rc;
  }
  if (stages & GCA_BWD_STAGE_KV) {
    if ((rc = launch_bwd_kv_tc(a, csr, rowterm, sms, stream))) return rc;
  }
  return 0;
}

}  // namespace gca
