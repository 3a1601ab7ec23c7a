#include "launch.h"
namespace ab200 {
bool sm100_bwd_supported(int, const Params&) { return false; }
cudaError_t launch_sm100_bwd_dkdv(int, const Params&, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_sm100_bwd_dq(int, const Params&, cudaStream_t) { return cudaErrorNotSupported; }
}
