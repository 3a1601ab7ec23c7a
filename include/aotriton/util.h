// Non-owning tensor views, lazily allocated tensors and GPU identification for the
// operator API.  Same types, member order and semantics as ROCm/aotriton
// include/aotriton/util.h (TensorView :78-158, TensorView<0> :161-209, LazyTensor
// :225-246, GPU queries :248-251), so that code written against that header
// compiles and links unchanged.  Strides are counted in elements.
#ifndef AOTRITON_V2_API_UTIL_H
#define AOTRITON_V2_API_UTIL_H

#include <aotriton/config.h>
#include "dtypes.h"
#include "runtime.h"
#include <array>
#include <cstdint>
#include <functional>
#include <string_view>

namespace AOTRITON_NS {

// Bit-packing helpers used to build the Gpu enumeration.
constexpr uint64_t CAT64(uint32_t high, uint32_t low) { return (uint64_t(high) << 32) | uint64_t(low); }
constexpr uint32_t CAT32(uint16_t high, uint16_t low) { return (uint32_t(high) << 16) | uint32_t(low); }
constexpr uint64_t TRICAT(uint16_t high, uint16_t mid, uint16_t low) {
  return (uint64_t(high) << 32) | (uint64_t(mid) << 16) | uint64_t(low);
}

template<typename T>
T AOTRITON_API cdiv(T numerator, T denominator) {
  return (numerator + (denominator - 1)) / denominator;
}

// PCI vendor ids double as vendor tags.
enum AOTRITON_API GpuVendor : uint16_t {
  kAMD = 0x1002,
  kNVIDIA = 0x10de,
  kINTEL = 0x8086,
};

// vendor:arch:mod triples.  This build knows exactly one architecture.
enum AOTRITON_API Gpu : uint64_t {
  GPU_ARCH_UNKNOWN = 0,
  GPU_NVIDIA_ARCH_SM100_MOD0 = TRICAT(GpuVendor::kNVIDIA, 0x100, 0),
};

inline uint32_t Gpu2VendorArch(uint64_t gpu) { return (gpu & 0xFFFF'FFFF'0000) >> 16; }

template<int Rank>
class AOTRITON_API TensorView {
 public:
  TensorView() {}

  TensorView(intptr_t base, std::array<uint64_t, Rank> sizes, std::array<uint64_t, Rank> strides, DType dtype)
    : base_(reinterpret_cast<void*>(base)), sizes_(sizes), strides_(strides), dtype_(dtype) {}

  // Wrap anything that looks like an at::Tensor.
  template<typename Tensor>
  TensorView(const Tensor& tensor, std::function<DType(const Tensor&)> dtype_extractor) {
    base_ = tensor.data_ptr();
    for (int i = 0; i < Rank; i++) {
      sizes_[i] = tensor.size(i);
      strides_[i] = tensor.stride(i);
    }
    dtype_ = dtype_extractor(tensor);
  }

  operator bool() const { return base_ != nullptr; }

  uint64_t size(int i) const { return sizes_[i]; }
  uint64_t stride(int i) const { return strides_[i]; }
  std::array<uint64_t, Rank> sizes() const { return sizes_; }
  std::array<uint64_t, Rank> strides() const { return strides_; }
  const uint64_t* size_ptr() const { return sizes_.data(); }
  const uint64_t* stride_ptr() const { return strides_.data(); }
  void* data_ptr() const { return base_; }
  DType dtype() const { return dtype_; }

  // Addresses of the members, for launch APIs that take void** kernel parameters.
  void* kparam_data_ptr() const { return const_cast<void*>(static_cast<const void*>(&base_)); }
  void* kparam_stride(int i) const { return const_cast<void*>(static_cast<const void*>(&strides_[i])); }

  static TensorView<Rank> get_null_tensor(DType dtype) {
    return TensorView<Rank>{0, std::array<uint64_t, Rank>{}, std::array<uint64_t, Rank>{}, dtype};
  }

 private:
  void* base_ = nullptr;
  std::array<uint64_t, Rank> sizes_{};
  std::array<uint64_t, Rank> strides_{};
  DType dtype_ = kUnknown;
};

// Rank-0 view: a device scalar (Philox seed/offset, atomic counter).
template<>
class AOTRITON_API TensorView<0> {
 public:
  TensorView() {}
  TensorView(intptr_t base, DType dtype) : base_(reinterpret_cast<void*>(base)), dtype_(dtype) {}

  operator bool() const { return base_ != nullptr; }
  uint64_t size(int i) const { return i == 0 ? 1 : 0; }
  uint64_t stride(int i) const { return i == 0 ? 1 : 0; }
  std::array<uint64_t, 0> sizes() const { return {}; }
  std::array<uint64_t, 0> strides() const { return {}; }
  void* data_ptr() const { return base_; }
  DType dtype() const { return dtype_; }
  void* kparam_data_ptr() const { return const_cast<void*>(static_cast<const void*>(&base_)); }

  static TensorView<0> get_null_tensor(DType dtype) { return TensorView<0>{0, dtype}; }

 private:
  void* base_ = nullptr;
  DType dtype_ = kUnknown;
};

#ifndef aotriton_v2_EXPORTS
extern template class TensorView<1>;
extern template class TensorView<2>;
extern template class TensorView<3>;
extern template class TensorView<4>;
#endif

// A tensor the library may or may not need (backward's delta and fp32 dQ
// accumulator).  The caller supplies C function pointers (no std::function, to
// keep the struct layout independent of the C++ standard library) that allocate
// on first use and release afterwards; `eager` short-circuits both with a
// caller-managed view.
template<int Rank>
struct LazyTensor {
  void* cookie = nullptr;
  TensorView<Rank> (*acquire)(LazyTensor<Rank>* self) = nullptr;
  void (*dispose)(LazyTensor<Rank>* self) = nullptr;
  TensorView<Rank> eager;

  operator bool() const { return eager || cookie != nullptr || acquire != nullptr || dispose != nullptr; }

  void free() {
    if (dispose && cookie) {
      (*dispose)(this);
      cookie = nullptr;
    }
  }
};

Gpu AOTRITON_API getGpuFromStream(hipStream_t);
bool AOTRITON_API isArchExperimentallySupported(hipStream_t);
int AOTRITON_API getMultiProcessorCount(hipStream_t stream);
bool AOTRITON_API isArchTechPreview(hipStream_t);

}  // namespace AOTRITON_NS

#endif
