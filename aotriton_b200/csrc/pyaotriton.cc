// Python module `pyaotriton`: the same names the Python tests and the tuner of
// ROCm/aotriton import (bindings/module.cc:32-113, hipruntime.cc:11-95,
// hipmemory.cc:15-69, lazy_tensor/main.cc:17-34, modules/flash/bindings/v2.cc:26-50,
// v3.cc:21-186), bound to this library's C++ operator API.
//
// Differences a caller can observe:
//   * Stream(handle: int) is accepted in addition to Stream(); handle is a
//     cudaStream_t as an integer (torch.cuda.current_stream().cuda_stream).
//   * lazy_tensor.dq_acc / delta allocate through a small stream-keyed caching pool over
//     cudaMalloc, so the module does not link against libtorch; lazy_tensor.dq_acc_from /
//     delta_from take a Python callable instead, which is how the torch allocator is used
//     (the reference's lazy tensors call at::zeros / at::empty,
//     bindings/lazy_tensor/lazy_tensor_template.h:19-97).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <aotriton/flash.h>
#include <aotriton/util.h>
#include <aotriton_b200.h>
#include <cuda_runtime_api.h>

#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

namespace py = pybind11;
namespace aotriton = AOTRITON_NS;

namespace {

// ---- device scratch pool for lazy tensors -------------------------------------
// Blocks go back to a free list instead of cudaFree, so disposing a lazy tensor right after an
// asynchronous launch never synchronises the device.  The free lists are keyed by (device,
// stream): a block is only handed out again for work on the stream its previous user ran on,
// where the new kernels queue behind the old ones (what a stream-ordered caching allocator does).
class ScratchPool {
 public:
  using Key = std::pair<int, intptr_t>;
  void* take(int device, intptr_t stream, size_t bytes) {
    bytes = (bytes + 511) & ~size_t(511);
    if (bytes == 0) bytes = 512;
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto& fl = free_[Key(device, stream)];
      auto it = fl.lower_bound(bytes);
      if (it != fl.end() && it->first <= 2 * bytes) {
        void* p = it->second;
        sizes_[p] = it->first;
        fl.erase(it);
        return p;
      }
    }
    int old = -1;
    cudaGetDevice(&old);
    if (device >= 0 && device != old) cudaSetDevice(device);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (device >= 0 && device != old) cudaSetDevice(old);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lock(mu_);
    sizes_[p] = bytes;
    return p;
  }
  void give(int device, intptr_t stream, void* p) {
    if (!p) return;
    std::lock_guard<std::mutex> lock(mu_);
    free_[Key(device, stream)].emplace(sizes_[p], p);
  }

 private:
  std::mutex mu_;
  std::map<Key, std::multimap<size_t, void*>> free_;
  std::map<void*, size_t> sizes_;
};

ScratchPool& pool() {
  static ScratchPool* p = new ScratchPool;   // leaked on purpose: outlives CUDA teardown order issues
  return *p;
}

// Cookies of lazy tensors that have not been disposed yet.  A LazyTensor is a plain struct that
// callers copy around (into the params struct, for one); only the copy inside the operator call
// is cleared by free(), so a stale copy used for a second call must be recognised here.
class LiveCookies {
 public:
  void add(void* c) { std::lock_guard<std::mutex> l(mu_); live_.insert(c); }
  bool alive(void* c) { std::lock_guard<std::mutex> l(mu_); return live_.count(c) != 0; }
  bool remove(void* c) { std::lock_guard<std::mutex> l(mu_); return live_.erase(c) != 0; }
 private:
  std::mutex mu_;
  std::set<void*> live_;
};
LiveCookies& cookies() {
  static LiveCookies* c = new LiveCookies;
  return *c;
}

template <int Rank>
aotriton::TensorView<Rank> contiguous_f32_view(const aotriton::TensorView<Rank>& like, void* mem, uint64_t* numel) {
  std::array<uint64_t, Rank> sizes = like.sizes(), strides{};
  uint64_t n = 1;
  for (int i = Rank - 1; i >= 0; --i) { strides[i] = n; n *= sizes[i]; }
  if (numel) *numel = n;
  return aotriton::TensorView<Rank>(reinterpret_cast<intptr_t>(mem), sizes, strides, aotriton::kFloat32);
}

template <int Rank, bool Zeroed>
struct LazyHelper {
  struct Ctx {
    aotriton::TensorView<Rank> like;
    int device;
    intptr_t stream;      // the stream the operator call will launch on (0 = the default stream)
    void* mem = nullptr;
  };
  static aotriton::TensorView<Rank> acquire(aotriton::LazyTensor<Rank>* self) {
    auto* ctx = static_cast<Ctx*>(self->cookie);
    if (!ctx || !cookies().alive(ctx)) return aotriton::TensorView<Rank>();   // a lazy tensor serves one call
    uint64_t n = 0;
    contiguous_f32_view<Rank>(ctx->like, nullptr, &n);
    if (!ctx->mem) {
      ctx->mem = pool().take(ctx->device, ctx->stream, n * sizeof(float));
      if (ctx->mem && Zeroed)
        cudaMemsetAsync(ctx->mem, 0, n * sizeof(float), reinterpret_cast<cudaStream_t>(ctx->stream));
    }
    if (!ctx->mem) return aotriton::TensorView<Rank>();
    return contiguous_f32_view<Rank>(ctx->like, ctx->mem, nullptr);
  }
  static void dispose(aotriton::LazyTensor<Rank>* self) {
    auto* ctx = static_cast<Ctx*>(self->cookie);
    if (!ctx || !cookies().remove(ctx)) return;
    pool().give(ctx->device, ctx->stream, ctx->mem);
    delete ctx;
  }
  static aotriton::TensorView<Rank> acquire_eager(aotriton::LazyTensor<Rank>* self) { return self->eager; }

  static aotriton::LazyTensor<Rank> make(const aotriton::TensorView<Rank>& like, int device, intptr_t stream) {
    auto* ctx = new Ctx;
    ctx->like = like;
    ctx->device = device;
    ctx->stream = stream;
    cookies().add(ctx);
    aotriton::LazyTensor<Rank> lt;
    lt.cookie = ctx;
    lt.acquire = &acquire;
    lt.dispose = &dispose;
    return lt;
  }
  static aotriton::LazyTensor<Rank> make_eager(const aotriton::TensorView<Rank>& view) {
    aotriton::LazyTensor<Rank> lt;
    lt.acquire = &acquire_eager;
    lt.eager = view;
    return lt;
  }
};

// Lazy tensor whose memory comes from a Python callable (called at most once, when the operator
// really needs the tensor): the callable returns an object with data_ptr(), e.g. a torch tensor
// made by torch.empty / torch.zeros on the current stream, which the lazy tensor keeps alive until
// the operator disposes of it.  The operator runs with the GIL released, so both callbacks take it.
template <int Rank>
struct PyLazy {
  struct Ctx {
    aotriton::TensorView<Rank> like;
    py::object factory, tensor;
  };
  static aotriton::TensorView<Rank> acquire(aotriton::LazyTensor<Rank>* self) {
    auto* ctx = static_cast<Ctx*>(self->cookie);
    if (!ctx || !cookies().alive(ctx)) return aotriton::TensorView<Rank>();
    py::gil_scoped_acquire gil;
    try {
      if (!ctx->tensor || ctx->tensor.is_none()) ctx->tensor = ctx->factory();
      const intptr_t ptr = ctx->tensor.attr("data_ptr")().template cast<intptr_t>();
      return contiguous_f32_view<Rank>(ctx->like, reinterpret_cast<void*>(ptr), nullptr);
    } catch (py::error_already_set& e) {
      e.discard_as_unraisable("pyaotriton lazy tensor factory");
      return aotriton::TensorView<Rank>();
    }
  }
  static void dispose(aotriton::LazyTensor<Rank>* self) {
    auto* ctx = static_cast<Ctx*>(self->cookie);
    if (!ctx || !cookies().remove(ctx)) return;
    py::gil_scoped_acquire gil;
    delete ctx;
  }
  static aotriton::LazyTensor<Rank> make(const aotriton::TensorView<Rank>& like, py::object factory) {
    auto* ctx = new Ctx;
    ctx->like = like;
    ctx->factory = std::move(factory);
    cookies().add(ctx);
    aotriton::LazyTensor<Rank> lt;
    lt.cookie = ctx;
    lt.acquire = &acquire;
    lt.dispose = &dispose;
    return lt;
  }
};

// Plain cudaMalloc'ed buffer for callers that keep their tensors on the host.
class HipMemory {
 public:
  ~HipMemory() { release(); }
  void alloc(size_t size) {
    release();
    last_ = static_cast<hipError_t>(cudaMalloc(&mem_, size));
    if (last_ == hipSuccess) size_ = size;
  }
  void release() {
    if (mem_) last_ = static_cast<hipError_t>(cudaFree(mem_));
    mem_ = nullptr; size_ = 0;
  }
  intptr_t get_pointer() const { return reinterpret_cast<intptr_t>(mem_); }
  void load_from_host(intptr_t ptr, size_t nbytes) {
    if (mem_ && nbytes <= size_)
      last_ = static_cast<hipError_t>(cudaMemcpy(mem_, reinterpret_cast<void*>(ptr), nbytes, cudaMemcpyHostToDevice));
  }
  void store_to_host(intptr_t ptr, size_t nbytes) {
    if (mem_ && nbytes <= size_)
      last_ = static_cast<hipError_t>(cudaMemcpy(reinterpret_cast<void*>(ptr), mem_, nbytes, cudaMemcpyDeviceToHost));
  }
  void zero_memory() { if (mem_) last_ = static_cast<hipError_t>(cudaMemset(mem_, 0, size_)); }
  hipError_t last_state() const { return last_; }

 private:
  void* mem_ = nullptr;
  size_t size_ = 0;
  hipError_t last_ = hipSuccess;
};

template <int Rank>
void def_tensorview(py::module_& m, const char* name) {
  using TV = aotriton::TensorView<Rank>;
  py::class_<TV>(m, name)
      .def(py::init<intptr_t, std::array<uint64_t, Rank>, std::array<uint64_t, Rank>, aotriton::DType>())
      .def("size", &TV::size)
      .def("stride", &TV::stride)
      .def_property_readonly("sizes", &TV::sizes)
      .def_property_readonly("strides", &TV::strides)
      .def_property_readonly("data_ptr", [](const TV& t) { return reinterpret_cast<intptr_t>(t.data_ptr()); })
      .def_property_readonly("dtype", &TV::dtype);
}

void def_hip_errors(py::module_& m) {
  py::enum_<hipError_t> e(m, "hipError_t", py::module_local());
#define EV(name) e.value(#name, name)
  EV(hipSuccess); EV(hipErrorInvalidValue); EV(hipErrorOutOfMemory); EV(hipErrorMemoryAllocation);
  EV(hipErrorNotInitialized); EV(hipErrorInitializationError); EV(hipErrorDeinitialized);
  EV(hipErrorProfilerDisabled); EV(hipErrorProfilerNotInitialized); EV(hipErrorProfilerAlreadyStarted);
  EV(hipErrorProfilerAlreadyStopped); EV(hipErrorInvalidConfiguration); EV(hipErrorInvalidPitchValue);
  EV(hipErrorInvalidSymbol); EV(hipErrorInvalidDevicePointer); EV(hipErrorInvalidMemcpyDirection);
  EV(hipErrorInsufficientDriver); EV(hipErrorMissingConfiguration); EV(hipErrorPriorLaunchFailure);
  EV(hipErrorInvalidDeviceFunction); EV(hipErrorNoDevice); EV(hipErrorInvalidDevice); EV(hipErrorInvalidImage);
  EV(hipErrorInvalidContext); EV(hipErrorContextAlreadyCurrent); EV(hipErrorMapFailed);
  EV(hipErrorMapBufferObjectFailed); EV(hipErrorUnmapFailed); EV(hipErrorArrayIsMapped); EV(hipErrorAlreadyMapped);
  EV(hipErrorNoBinaryForGpu); EV(hipErrorAlreadyAcquired); EV(hipErrorNotMapped); EV(hipErrorNotMappedAsArray);
  EV(hipErrorNotMappedAsPointer); EV(hipErrorECCNotCorrectable); EV(hipErrorUnsupportedLimit);
  EV(hipErrorContextAlreadyInUse); EV(hipErrorPeerAccessUnsupported); EV(hipErrorInvalidKernelFile);
  EV(hipErrorInvalidGraphicsContext); EV(hipErrorInvalidSource); EV(hipErrorFileNotFound);
  EV(hipErrorSharedObjectSymbolNotFound); EV(hipErrorSharedObjectInitFailed); EV(hipErrorOperatingSystem);
  EV(hipErrorInvalidHandle); EV(hipErrorInvalidResourceHandle); EV(hipErrorIllegalState); EV(hipErrorNotFound);
  EV(hipErrorNotReady); EV(hipErrorIllegalAddress); EV(hipErrorLaunchOutOfResources); EV(hipErrorLaunchTimeOut);
  EV(hipErrorPeerAccessAlreadyEnabled); EV(hipErrorPeerAccessNotEnabled); EV(hipErrorSetOnActiveProcess);
  EV(hipErrorContextIsDestroyed); EV(hipErrorAssert); EV(hipErrorHostMemoryAlreadyRegistered);
  EV(hipErrorHostMemoryNotRegistered); EV(hipErrorLaunchFailure); EV(hipErrorCooperativeLaunchTooLarge);
  EV(hipErrorNotSupported); EV(hipErrorStreamCaptureUnsupported); EV(hipErrorStreamCaptureInvalidated);
  EV(hipErrorStreamCaptureMerge); EV(hipErrorStreamCaptureUnmatched); EV(hipErrorStreamCaptureUnjoined);
  EV(hipErrorStreamCaptureIsolation); EV(hipErrorStreamCaptureImplicit); EV(hipErrorCapturedEvent);
  EV(hipErrorStreamCaptureWrongThread); EV(hipErrorGraphExecUpdateFailure); EV(hipErrorUnknown);
  EV(hipErrorRuntimeMemory); EV(hipErrorRuntimeOther); EV(hipErrorTbd);
#undef EV
  e.export_values();
  m.def("hipDeviceSynchronize", []() { return static_cast<hipError_t>(::hipDeviceSynchronize()); });
  m.def("hipGetLastError", []() { return static_cast<hipError_t>(::hipGetLastError()); });
}

void def_v2(py::module_& root) {
  py::module_ v2 = root.def_submodule("v2", "v2 API namespace");
  py::module_ m = v2.def_submodule("flash", "Flash Attention API");
  m.def("check_gpu", &aotriton::v2::flash::check_gpu, py::arg("stream"));
  m.def("debug_simulate_encoded_softmax", &aotriton::v2::flash::debug_simulate_encoded_softmax,
        "Write +0.5/-0.5 according to the dropout keep bit", py::call_guard<py::gil_scoped_release>(),
        py::arg("r"), py::arg("dropout_p"), py::arg("philox_seed_ptr"), py::arg("philox_offset1"),
        py::arg("philox_offset2"), py::arg("stream") = aotriton::Stream());
  m.def("attn_fwd", &aotriton::v2::flash::attn_fwd, py::call_guard<py::gil_scoped_release>());
  m.def("attn_fwd_compact_varlen", &aotriton::v2::flash::attn_fwd_compact_varlen,
        py::call_guard<py::gil_scoped_release>());
  m.def("attn_bwd", &aotriton::v2::flash::attn_bwd, py::call_guard<py::gil_scoped_release>());
  m.def("attn_bwd_compact_varlen", &aotriton::v2::flash::attn_bwd_compact_varlen,
        py::call_guard<py::gil_scoped_release>());
}

void def_v3(py::module_& root) {
  using aotriton::v3::flash::attn_bwd_params;
  using aotriton::v3::flash::attn_fwd_params;
  using aotriton::v3::flash::attn_options;
  py::module_ v3 = root.def_submodule("v3", "v3 API namespace");
  py::module_ m = v3.def_submodule("flash", "Flash Attention Operators");
  py::class_<attn_options>(m, "attn_options")
      .def(py::init<>())
      .def_readwrite("force_backend_index", &attn_options::force_backend_index)
      .def_readwrite("deterministic", &attn_options::deterministic);
  py::class_<attn_fwd_params> f(m, "attn_fwd_params");
  f.def(py::init<>());
#define RW(name) f.def_readwrite(#name, &attn_fwd_params::name)
  RW(Q); RW(K); RW(V); RW(B); RW(Sm_scale); RW(L); RW(Out); RW(cu_seqlens_q); RW(cu_seqlens_k);
  RW(Max_seqlen_q); RW(Max_seqlen_k); RW(seq_strides_q); RW(seq_strides_k); RW(dropout_p);
  RW(philox_seed_ptr); RW(philox_offset1); RW(philox_offset2); RW(philox_seed_output);
  RW(philox_offset_output); RW(encoded_softmax); RW(persistent_atomic_counter); RW(causal_type);
  RW(varlen_type); RW(window_left); RW(window_right);
#undef RW
  f.def_readonly_static("kVersion", &attn_fwd_params::kVersion);
  py::class_<attn_bwd_params> b(m, "attn_bwd_params");
  b.def(py::init<>());
#define RW(name) b.def_readwrite(#name, &attn_bwd_params::name)
  RW(Q); RW(K); RW(V); RW(B); RW(Sm_scale); RW(Out); RW(DO); RW(DK); RW(DV); RW(DQ); RW(DB); RW(L); RW(D);
  RW(cu_seqlens_q); RW(cu_seqlens_k); RW(Max_seqlen_q); RW(Max_seqlen_k); RW(seq_strides_q);
  RW(seq_strides_k); RW(dropout_p); RW(philox_seed_ptr); RW(philox_offset1); RW(philox_offset2);
  RW(causal_type); RW(varlen_type); RW(window_left); RW(window_right); RW(DQ_ACC);
#undef RW
  b.def_readonly_static("kVersion", &attn_bwd_params::kVersion);
  m.def("attn_fwd", &aotriton::v3::flash::attn_fwd, "Flash Attention Operator Forward Pass",
        py::call_guard<py::gil_scoped_release>(), py::arg("params"), py::arg("params_version"),
        py::arg("stream") = aotriton::Stream(), py::arg("options") = nullptr);
  m.def("attn_bwd", &aotriton::v3::flash::attn_bwd, "Flash Attention Operator Backward Pass",
        py::call_guard<py::gil_scoped_release>(), py::arg("params"), py::arg("params_version"),
        py::arg("stream") = aotriton::Stream(), py::arg("options") = nullptr);
}

void def_lazy(py::module_& root) {
  py::module_ m = root.def_submodule("lazy_tensor", "lazy_tensor API namespace");
  py::class_<aotriton::LazyTensor<4>>(m, "LT4");
  py::class_<aotriton::LazyTensor<2>>(m, "LT2");
  m.def("dq_acc", &LazyHelper<4, true>::make, py::arg("like"), py::arg("device"), py::arg("stream") = 0);
  m.def("delta", &LazyHelper<2, false>::make, py::arg("like"), py::arg("device"), py::arg("stream") = 0);
  m.def("dq_acc_from", &PyLazy<4>::make, py::arg("like"), py::arg("factory"));
  m.def("delta_from", &PyLazy<2>::make, py::arg("like"), py::arg("factory"));
  m.def("eager_delta", &LazyHelper<2, false>::make_eager);
  m.def("eager_null_dq_acc", &LazyHelper<4, false>::make_eager);
}

}  // namespace

PYBIND11_MODULE(pyaotriton, m) {
  m.doc() = "aotriton operator API backed by sm_100a CUDA kernels";
  py::class_<aotriton::Stream>(m, "Stream")
      .def(py::init<>())
      .def(py::init([](intptr_t handle) { return aotriton::Stream(reinterpret_cast<hipStream_t>(handle)); }));
  py::enum_<aotriton::DType>(m, "DType")
      .value("kUnknown", aotriton::kUnknown)
      .value("kFloat32", aotriton::kFloat32)
      .value("kFloat16", aotriton::kFloat16)
      .value("kBFloat16", aotriton::kBFloat16)
      .value("kInt8", aotriton::kInt8)
      .value("kInt16", aotriton::kInt16)
      .value("kInt32", aotriton::kInt32)
      .value("kInt64", aotriton::kInt64)
      .value("kUInt8", aotriton::kUInt8)
      .value("kUInt16", aotriton::kUInt16)
      .value("kUInt32", aotriton::kUInt32)
      .value("kUInt64", aotriton::kUInt64)
      .export_values();
  def_hip_errors(m);
  def_tensorview<4>(m, "T4");
  def_tensorview<2>(m, "T2");
  def_tensorview<1>(m, "T1");
  py::class_<HipMemory>(m, "HipMemory")
      .def(py::init<>())
      .def("alloc", &HipMemory::alloc)
      .def("free", &HipMemory::release)
      .def("get_pointer", &HipMemory::get_pointer)
      .def("last_state", &HipMemory::last_state)
      .def("load_from_host", &HipMemory::load_from_host)
      .def("store_to_host", &HipMemory::store_to_host)
      .def("zero_memory", &HipMemory::zero_memory);
  using T0 = aotriton::TensorView<0>;
  py::class_<T0>(m, "T0")
      .def(py::init<intptr_t, aotriton::DType>())
      .def("size", &T0::size)
      .def("stride", &T0::stride)
      .def_property_readonly("sizes", &T0::sizes)
      .def_property_readonly("strides", &T0::strides)
      .def_property_readonly("data_ptr", [](const T0& t) { return reinterpret_cast<intptr_t>(t.data_ptr()); })
      .def_property_readonly("dtype", &T0::dtype);
#define AB200_STR2(x) #x
#define AB200_STR(x) AB200_STR2(x)
  m.def("get_name_suffix", []() -> std::string { return AB200_STR(AOTRITON_NAME_SUFFIX); });
  m.def("launch_count", []() { return ab200_launch_count(); });
  m.def("set_kernel_family", [](int f) { return ab200_set_kernel_family(f); });
  m.def("last_fwd_family", []() { return ab200_last_fwd_family(); });
  m.def("last_bwd_family", []() { return ab200_last_bwd_family(); });
  m.def("stream_check", [](aotriton::Stream s) { return static_cast<hipError_t>(ab200_stream_check(s.native())); },
        py::call_guard<py::gil_scoped_release>(), py::arg("stream") = aotriton::Stream());
  m.def("kernel_status", [](bool reset) { return ab200_kernel_status(reset ? 1 : 0); }, py::arg("reset") = false);
  def_v2(m);
  def_v3(m);
  def_lazy(m);
}
