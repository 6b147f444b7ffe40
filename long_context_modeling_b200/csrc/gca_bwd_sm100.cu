// placeholder until the tensor-core backward is in
#include "gca_common.cuh"
namespace gca {
bool bwd_tc_available() { return false; }
int launch_bwd_tc(const GcaBwdArgs&, const Csr&, float*, cudaStream_t) { return GCA_ERR_ALGO; }
}
