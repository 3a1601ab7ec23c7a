// Host-side declarations shared by the kernel translation units and the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include <tuple>
#include <type_traits>
#include <utility>
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

// Every CUDA runtime / driver call the launch path makes goes through this table.  Normally the
// entries forward to CUDA.  Tests can switch to a pretended sm_100 device (no GPU needed: device
// queries answer, symbol look-ups and launches are recorded and skipped) and can make the n-th call of
// any entry return an error code, to check that each failure comes back to the caller as that code
// with nothing launched after it (ab200_debug_host_calls).  No test ever makes a device fault.
enum HostCallId : int { kCallGetDevice = 0, kCallSetDevice, kCallStreamDevice, kCallDeviceAttr, kCallFuncSetSmem,
                        kCallSymbolAddress, kCallMemsetAsync, kCallLaunch, kCallEncodeTiled, kCallStreamSync,
                        kNumHostCalls };
struct HostCalls {
  cudaError_t (*get_device)(int* dev);
  cudaError_t (*set_device)(int dev);
  cudaError_t (*stream_device)(cudaStream_t st, int* dev);
  cudaError_t (*device_attr)(int* value, cudaDeviceAttr attr, int dev);
  cudaError_t (*func_set_smem)(const void* fn, int bytes);
  cudaError_t (*symbol_address)(void** ptr, const void* symbol);
  cudaError_t (*memset_async)(void* ptr, int value, size_t bytes, cudaStream_t st);
  cudaError_t (*launch)(const void* fn, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t st);
  // cuTensorMapEncodeTiled; returns a CUresult (0 = success, 100 = no encoder available)
  int (*encode_tiled)(CUtensorMap* map, CUtensorMapDataType type, cuuint32_t rank, void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* estr,
                      CUtensorMapInterleave il, CUtensorMapSwizzle sw, CUtensorMapL2promotion l2,
                      CUtensorMapFloatOOBfill fill);
  cudaError_t (*stream_sync)(cudaStream_t st);
  bool (*have_encoder)();
};
const HostCalls& host();
// true while the table pretends a device: nothing learnt from it may be remembered for real launches
bool host_pretends();

// kernel<<<grid, block, smem, st>>>(args...) through the table.  The arguments are converted to the
// kernel's exact parameter types and copied, as the launch API takes one pointer per parameter.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "argument count differs from the kernel's parameter list");
  std::tuple<std::remove_cv_t<std::remove_reference_t<KArgs>>...> copy(std::forward<Args>(args)...);
  void* ptrs[sizeof...(KArgs) > 0 ? sizeof...(KArgs) : 1];
  std::apply([&](auto&... a) { int i = 0; ((ptrs[i++] = (void*)&a), ...); }, copy);
  return host().launch(reinterpret_cast<const void*>(kernel), grid, block, ptrs, smem, st);
}

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
