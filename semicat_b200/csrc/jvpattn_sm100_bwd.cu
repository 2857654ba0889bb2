#include "jvpattn_common.cuh"
namespace jvpattn {
bool sm100_bwd_supported(const BwdArgs &) { return false; }
cudaError_t sm100_bwd(const BwdArgs &, cudaStream_t) { return cudaErrorNotSupported; }
size_t sm100_bwd_workspace_bytes(int, int, int, int, int, int) { return 0; }
}
