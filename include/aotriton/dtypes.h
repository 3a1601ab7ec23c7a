// Element-type tags of TensorView (ROCm/aotriton include/aotriton/dtypes.h:12-25).
// The numeric values are part of the ABI: callers store them in TensorView.
#ifndef AOTRITON_V2_API_DTYPES_H
#define AOTRITON_V2_API_DTYPES_H

#include <aotriton/config.h>
#include <stdint.h>

namespace AOTRITON_NS {

enum AOTRITON_API DType : int32_t {
  kUnknown = 0,
  // floating point
  kFloat32 = 1, kFloat16 = 2, kBFloat16 = 3,
  // signed integers
  kInt8 = 10, kInt16 = 11, kInt32 = 12, kInt64 = 13,
  // unsigned integers
  kUInt8 = 20, kUInt16 = 21, kUInt32 = 22, kUInt64 = 23,
};

}  // namespace AOTRITON_NS

#endif
