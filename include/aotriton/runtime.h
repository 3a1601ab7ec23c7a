// Stream wrapper of the operator API (ROCm/aotriton include/aotriton/runtime.h:15-31).
// It exists so that bindings can pass "a stream" without knowing the handle type;
// a default-constructed Stream is the default (NULL) stream.
#ifndef AOTRITON_V2_API_RUNTIME_H
#define AOTRITON_V2_API_RUNTIME_H

#include <hip/hip_runtime.h>
#include <aotriton/config.h>

namespace AOTRITON_NS {

template<typename Handle>
class AOTRITON_API StreamTemplate {
 public:
  StreamTemplate() = default;
  StreamTemplate(Handle h) : stream_(h) {}
  Handle native() const { return stream_; }

 private:
  Handle stream_ = nullptr;
};

using Stream = StreamTemplate<hipStream_t>;

}  // namespace AOTRITON_NS

#endif
