#include "launch.h"
namespace ab200 {
bool sm100_fwd_supported(int, const Params&) { return false; }
cudaError_t launch_sm100_fwd(int, const Params&, cudaStream_t) { return cudaErrorNotSupported; }
}
