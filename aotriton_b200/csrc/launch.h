// Host-side declarations shared by the kernel translation units and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include "common.cuh"

namespace ab200 {

// Integer dropout threshold: keep iff (int32)philox_word > threshold.
// Restates `((dropout_p - 0.5) * 0xFFFFFFFF).to(tl.int32)` of ROCm/aotriton
// modules/flash/kernel/fwd_kernel.py:195 -- fp32 arithmetic, the literal rounds
// to 2^32 in fp32, conversion truncates toward zero and saturates.
inline int32_t dropout_threshold(float dropout_p) {
  float x = (dropout_p - 0.5f) * 4294967296.0f;
  if (!(x == x)) return 0;
  if (x >= 2147483647.0f) return 2147483647;
  if (x <= -2147483648.0f) return (int32_t)(-2147483647 - 1);
  return (int32_t)truncf(x);
}

void count_launch();

// which: 0 forward, 1 dK/dV, 2 dQ(+dBias).  dtype: ab200_dtype value.
cudaError_t launch_general(int which, int dtype, const Params& p, cudaStream_t st);
cudaError_t launch_preprocess(int dtype, const Params& p, cudaStream_t st);
cudaError_t launch_dropout_sign(int dtype, const View4& r, int batch, int heads, int rows, int cols, float dropout_p,
                                const uint64_t* seed, const uint64_t* off1, uint64_t off2, cudaStream_t st);

// tcgen05 kernels (sm100_fwd.cu / sm100_bwd.cu).  *_supported say whether the shape is
// inside the kernel's range; the launchers assume it is.
bool sm100_fwd_supported(int dtype, const Params& p);
cudaError_t launch_sm100_fwd(int dtype, const Params& p, cudaStream_t st);
bool sm100_bwd_supported(int dtype, const Params& p);
cudaError_t launch_sm100_bwd_dkdv(int dtype, const Params& p, cudaStream_t st);
cudaError_t launch_sm100_bwd_dq(int dtype, const Params& p, cudaStream_t st);
// Fused backward: dK, dV and the dQ partials in one kernel (partials added to the fp32 accumulator
// `dq_acc`, zero on entry, contiguous in dQ's logical order), then dQ = cast(sm_scale * dq_acc).
bool sm100_bwd_fused_supported(int dtype, const Params& p);
cudaError_t launch_sm100_bwd_fused(int dtype, const Params& p, float* dq_acc, cudaStream_t st);
cudaError_t launch_postprocess(int dtype, const View4& dq, const float* acc, float scale, cudaStream_t st);
// Words the tcgen05 kernels of the current device set when a bounded wait ran out (0 = none).
// Reading synchronises the device.
unsigned int sm100_fwd_status(bool reset);
unsigned int sm100_bwd_status(bool reset);

}  // namespace ab200
