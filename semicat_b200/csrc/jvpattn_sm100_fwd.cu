#include "jvpattn_common.cuh"
namespace jvpattn {
bool sm100_fwd_supported(const FwdArgs &) { return false; }
cudaError_t sm100_fwd(const FwdArgs &, cudaStream_t) { return cudaErrorNotSupported; }
}
