// extern "C" entry points of include/aotriton_b200.h: host-side validation,
// translation of the POD argument structs into kernel parameters, and the choice
// between the tcgen05 kernels and the general kernels.  No device memory is
// allocated here, nothing synchronises, and there is no CPU path: if no kernel can
// take the problem the call fails with an error code.
//
// Error vocabulary follows ROCm/aotriton (python/codegen/template/op.cc:21-71):
// unknown GPU -> hipErrorNoBinaryForGpu (209), unsupported functional ->
// hipErrorNotSupported (801), malformed arguments -> hipErrorInvalidValue (1).
#include <atomic>
#include <mutex>
#include <cstdio>
#include <cstdlib>

#include "../../include/aotriton_b200.h"
#include "launch.h"

namespace ab200 {

static std::atomic<uint64_t> g_launches{0};
static thread_local int g_family = 0;   // per calling thread, so concurrent callers do not interfere
static thread_local int t_last_fwd = 0, t_last_bwd = 0;
// Test hook of the bounded waits (ab200_debug_bounded_wait_test): which copy the producer leaves
// out and the wait limit of the calling thread's next launches.
static thread_local int t_drop_copy = 0;
static thread_local unsigned int t_wait_limit_kcycles = 0;
// Devices on which a kernel reported that a bounded wait ran out (seen by ab200_kernel_status or
// ab200_stream_check): further launches there are refused until the word is reset.
static std::atomic<uint64_t> g_failed_devices{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- host-call table -------------------------------------------------------------------------
namespace {
std::atomic<int> g_fake_device{0};              // 1: pretend an sm_100 device, skip symbol look-ups and launches
std::atomic<int> g_fail_call{-1}, g_fail_code{0}, g_fail_after{0};
std::atomic<uint64_t> g_call_count[kNumHostCalls];

// true when this call is the one a test asked to fail; counts the call either way
bool injected(int id, cudaError_t* code) {
  g_call_count[id].fetch_add(1, std::memory_order_relaxed);
  if (g_fail_call.load(std::memory_order_relaxed) != id) return false;
  if (g_fail_after.fetch_sub(1, std::memory_order_relaxed) != 0) return false;
  *code = static_cast<cudaError_t>(g_fail_code.load(std::memory_order_relaxed));
  return true;
}
bool fake() { return g_fake_device.load(std::memory_order_relaxed) != 0; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn driver_encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

cudaError_t h_get_device(int* dev) {
  cudaError_t c;
  if (injected(kCallGetDevice, &c)) return c;
  if (fake()) { *dev = 0; return cudaSuccess; }
  return cudaGetDevice(dev);
}
cudaError_t h_set_device(int dev) {
  cudaError_t c;
  if (injected(kCallSetDevice, &c)) return c;
  if (fake()) return cudaSuccess;
  return cudaSetDevice(dev);
}
cudaError_t h_stream_device(cudaStream_t st, int* dev) {
  cudaError_t c;
  if (injected(kCallStreamDevice, &c)) return c;
  if (fake()) { *dev = 0; return cudaSuccess; }
#if CUDART_VERSION >= 12080
  return cudaStreamGetDevice(st, dev);
#else
  (void)st;
  return cudaGetDevice(dev);
#endif
}
cudaError_t h_device_attr(int* value, cudaDeviceAttr attr, int dev) {
  cudaError_t c;
  if (injected(kCallDeviceAttr, &c)) return c;
  if (fake()) {
    *value = attr == cudaDevAttrComputeCapabilityMajor ? 10 : (attr == cudaDevAttrMultiProcessorCount ? 148 : 0);
    return cudaSuccess;
  }
  return cudaDeviceGetAttribute(value, attr, dev);
}
cudaError_t h_func_set_smem(const void* fn, int bytes) {
  cudaError_t c;
  if (injected(kCallFuncSetSmem, &c)) return c;
  if (fake()) return cudaSuccess;
  return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
cudaError_t h_symbol_address(void** ptr, const void* symbol) {
  cudaError_t c;
  if (injected(kCallSymbolAddress, &c)) return c;
  if (fake()) { *ptr = reinterpret_cast<void*>(uintptr_t(0x1000)); return cudaSuccess; }   // never dereferenced
  return cudaGetSymbolAddress(ptr, symbol);
}
cudaError_t h_memset_async(void* ptr, int value, size_t bytes, cudaStream_t st) {
  cudaError_t c;
  if (injected(kCallMemsetAsync, &c)) return c;
  if (fake()) return cudaSuccess;
  return cudaMemsetAsync(ptr, value, bytes, st);
}
cudaError_t h_launch(const void* fn, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t st) {
  cudaError_t c;
  if (injected(kCallLaunch, &c)) return c;
  if (fake()) return cudaSuccess;
  return cudaLaunchKernel(fn, grid, block, args, smem, st);
}
int h_encode_tiled(CUtensorMap* map, CUtensorMapDataType type, cuuint32_t rank, void* base, const cuuint64_t* dims,
                   const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* estr, CUtensorMapInterleave il,
                   CUtensorMapSwizzle sw, CUtensorMapL2promotion l2, CUtensorMapFloatOOBfill fill) {
  cudaError_t c;
  if (injected(kCallEncodeTiled, &c)) return (int)c;
  if (fake()) { *map = CUtensorMap{}; return 0; }
  EncodeTiledFn enc = driver_encoder();
  if (!enc) return 100;     // CUDA_ERROR_NO_DEVICE: no driver to encode with
  return (int)enc(map, type, rank, base, dims, strides, box, estr, il, sw, l2, fill);
}
cudaError_t h_stream_sync(cudaStream_t st) {
  cudaError_t c;
  if (injected(kCallStreamSync, &c)) return c;
  if (fake()) return cudaSuccess;
  return cudaStreamSynchronize(st);
}
bool h_have_encoder() { return fake() || driver_encoder() != nullptr; }
}  // namespace

bool host_pretends() { return fake(); }

const HostCalls& host() {
  static const HostCalls table = {h_get_device,  h_set_device,   h_stream_device, h_device_attr,
                                  h_func_set_smem, h_symbol_address, h_memset_async, h_launch,
                                  h_encode_tiled,  h_stream_sync,   h_have_encoder};
  return table;
}

namespace {

enum : int { kErrInvalidValue = 1, kErrNoBinaryForGpu = 209, kErrLaunchFailure = 719, kErrNotSupported = 801 };

struct DeviceInfo { int major = 0, minor = 0, sms = 0; bool known = false; };

// Device properties are immutable, so a racy double initialisation is harmless; the
// mutex only keeps the table itself consistent.
DeviceInfo device_info(int dev) {
  static std::mutex mu;
  static DeviceInfo table[64];
  if (dev < 0 || dev >= 64) return DeviceInfo{};
  std::lock_guard<std::mutex> lock(mu);
  if (!table[dev].known) {
    DeviceInfo d;
    if (host().device_attr(&d.major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
        host().device_attr(&d.minor, cudaDevAttrComputeCapabilityMinor, dev) == cudaSuccess &&
        host().device_attr(&d.sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) {
      d.known = true;
      if (!fake()) table[dev] = d;       // (a pretended device is not remembered)
      else return d;
    } else {
      (void)cudaGetLastError();
    }
  }
  return table[dev];
}

int stream_device(cudaStream_t st) {
  int dev = -1;
  if (st != nullptr && host().stream_device(st, &dev) == cudaSuccess) return dev;
  if (!fake()) (void)cudaGetLastError();
  if (host().get_device(&dev) != cudaSuccess) { if (!fake()) (void)cudaGetLastError(); return -1; }
  return dev;
}

int check_device(cudaStream_t st) {
  int dev = stream_device(st);
  if (dev < 0) return kErrNoBinaryForGpu;
  DeviceInfo d = device_info(dev);
  if (!d.known || d.major != 10) return kErrNoBinaryForGpu;   // kernels are built for sm_100a only
  if (dev < 64 && ((g_failed_devices.load(std::memory_order_relaxed) >> dev) & 1u)) return kErrLaunchFailure;
  return 0;
}

// The stream decides the device (like the reference, which derives everything from the stream):
// while an entry point runs, the stream's device is the current one, so that launches, symbol
// look-ups and attribute settings all address it even if the caller's current device differs.
struct DeviceGuard {
  int old_ = -1;
  bool switched_ = false;
  explicit DeviceGuard(cudaStream_t st) {
    const int dev = stream_device(st);
    if (dev >= 0 && host().get_device(&old_) == cudaSuccess && old_ != dev)
      switched_ = host().set_device(dev) == cudaSuccess;
    if (!fake()) (void)cudaGetLastError();
  }
  ~DeviceGuard() { if (switched_) { (void)host().set_device(old_); } }
};

bool rows_16byte(const ab200_view4& v) {
  return v.ptr != nullptr && (reinterpret_cast<uintptr_t>(v.ptr) & 15u) == 0 && v.stride[3] == 1 &&
         v.stride[0] % 8 == 0 && v.stride[1] % 8 == 0 && v.stride[2] % 8 == 0;
}

View4 to_view(const ab200_view4& v) {
  View4 r; r.ptr = v.ptr;
  for (int i = 0; i < 4; ++i) { r.n[i] = v.size[i]; r.s[i] = v.stride[i]; }
  return r;
}

bool inner_contiguous(const ab200_view4& v) { return v.ptr == nullptr || v.stride[3] == 1; }

int fill_common(const ab200_attn_problem& a, Params& p) {
  if (a.dtype < AB200_DTYPE_FP32 || a.dtype > AB200_DTYPE_BF16) return kErrNotSupported;
  if (a.batch < 0 || a.num_head_q <= 0 || a.num_head_k <= 0 || a.max_seqlen_q < 0 || a.max_seqlen_k < 0)
    return kErrInvalidValue;
  if (a.head_dim_qk <= 0 || a.head_dim_vo <= 0) return kErrInvalidValue;
  if (a.head_dim_qk > 512 || a.head_dim_vo > 512) return kErrNotSupported;   // head-dim rounding fails beyond 512
  if (a.num_head_q % a.num_head_k != 0) return kErrInvalidValue;
  if (a.causal_type < 0 || a.causal_type > 3) return kErrNotSupported;
  if (!(a.dropout_p >= 0.f) || a.dropout_p > 1.f) return kErrInvalidValue;
  p.batch = a.batch; p.hq = a.num_head_q; p.hk = a.num_head_k; p.group = a.num_head_q / a.num_head_k;
  p.max_sq = a.max_seqlen_q; p.max_sk = a.max_seqlen_k; p.dqk = a.head_dim_qk; p.dvo = a.head_dim_vo;
  p.sm_scale = a.sm_scale; p.qk_scale = a.sm_scale * kLog2e;
  p.dropout_p = a.dropout_p;
  p.dropout_on = a.dropout_p > 0.f ? 1 : 0;
  p.dropout_scale = p.dropout_on ? 1.0f / (1.0f - a.dropout_p) : 1.0f;
  p.idropout = p.dropout_on ? dropout_threshold(a.dropout_p) : 0;
  p.causal_type = a.causal_type; p.causal = a.causal_type != 0;
  p.window_left = a.window_left; p.window_right = a.window_right;
  p.cu_q = a.cu_seqlens_q; p.cu_k = a.cu_seqlens_k; p.ss_q = a.seq_strides_q; p.ss_k = a.seq_strides_k;
  if (a.cu_seqlens_q != nullptr) {
    if (a.cu_seqlens_k == nullptr) return kErrInvalidValue;
    if ((a.seq_strides_q == nullptr) != (a.seq_strides_k == nullptr)) return kErrInvalidValue;
    p.varlen_mode = a.varlen_type == AB200_VARLEN_PADDED ? 2 : 1;
    if (p.varlen_mode == 2) { p.ss_q = nullptr; p.ss_k = nullptr; }
  } else {
    p.varlen_mode = 0; p.ss_q = nullptr; p.ss_k = nullptr; p.cu_k = nullptr;
  }
  p.seed_ptr = a.philox_seed; p.off1_ptr = a.philox_offset1; p.off2 = a.philox_offset2;
  p.philox_head_offset = a.philox_head_offset; p.philox_hq = a.philox_num_head_q;
  p.wait_limit_kcycles = t_wait_limit_kcycles; p.drop_copy = t_drop_copy;
  return 0;
}

// ---- static selection table ---------------------------------------------------------------
// What the reference looks up in its tuning database (tables FLASH$op_attn_fwd / FLASH$op_attn_bwd,
// keyed by dtype, head-dim bin, bias, dropout, causal and sequence-length bins) is a fixed table here:
// the first row whose dtype set and head-dim bound cover the problem names the kernel variant and
// the head-dim instantiation.  Alignment, the caller's forced family and the fused-backward request
// are applied on top (ab200_select_variant).
enum : int { kOpFwd = 0, kOpBwd = 1 };
enum : int { kVarGeneral = 1, kVarTcgen05 = 2, kVarTcgen05Fused = 3 };
struct SelectionRow { int op; unsigned dtype_mask; int dmax; int hd; int variant; };
constexpr unsigned kHalfTypes = (1u << AB200_DTYPE_FP16) | (1u << AB200_DTYPE_BF16);
constexpr unsigned kAllTypes = kHalfTypes | (1u << AB200_DTYPE_FP32);
constexpr SelectionRow kSelection[] = {
    {kOpFwd, kHalfTypes, 64, 64, kVarTcgen05},   {kOpFwd, kHalfTypes, 128, 128, kVarTcgen05},
    {kOpFwd, kHalfTypes, 256, 256, kVarTcgen05}, {kOpFwd, kAllTypes, 512, 0, kVarGeneral},
    {kOpBwd, kHalfTypes, 64, 64, kVarTcgen05},   {kOpBwd, kHalfTypes, 128, 128, kVarTcgen05},
    {kOpBwd, kHalfTypes, 256, 256, kVarTcgen05}, {kOpBwd, kAllTypes, 512, 0, kVarGeneral},
};

bool want_sm100(int family) { return family != 1; }
int family_flags(int family) {
  return family == 1 ? AB200_SELECT_FORCE_GENERAL : (family == 2 ? AB200_SELECT_FORCE_TCGEN05 : 0);
}
// The fused backward is chosen on request only (family 3): on the benchmark shapes the two-kernel
// backward is faster, because the fp32 atomics of the dQ partials saturate the L2.
bool want_fused(int family) { return family == 3; }

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_check_gpu(void* stream) { return check_device(static_cast<cudaStream_t>(stream)); }

int ab200_multiprocessor_count(void* stream) {
  int dev = stream_device(static_cast<cudaStream_t>(stream));
  if (dev < 0) return 0;
  return device_info(dev).sms;
}

int ab200_select_variant(int op, int dtype, int head_dim_qk, int head_dim_vo, int flags) {
  if (op != kOpFwd && op != kOpBwd) return -kErrInvalidValue;
  if (dtype < AB200_DTYPE_FP32 || dtype > AB200_DTYPE_BF16) return -kErrNotSupported;
  if (head_dim_qk <= 0 || head_dim_vo <= 0) return -kErrInvalidValue;
  const int dmax = head_dim_qk > head_dim_vo ? head_dim_qk : head_dim_vo;
  const bool tc_ok = (flags & AB200_SELECT_ALIGNED) && head_dim_qk % 8 == 0 && head_dim_vo % 8 == 0 &&
                     !(flags & AB200_SELECT_FORCE_GENERAL);
  for (const SelectionRow& r : kSelection) {
    if (r.op != op || !((r.dtype_mask >> dtype) & 1u) || dmax > r.dmax) continue;
    if (r.variant != kVarGeneral && !tc_ok) continue;
    if (r.variant == kVarGeneral && (flags & AB200_SELECT_FORCE_TCGEN05)) return -kErrNotSupported;
    int variant = r.variant;
    if (op == kOpBwd && variant == kVarTcgen05 && (flags & AB200_SELECT_FUSED_REQUESTED) &&
        !(flags & AB200_SELECT_DBIAS) && r.hd == 128)
      variant = kVarTcgen05Fused;
    return variant | (r.hd << 8);
  }
  return -kErrNotSupported;      // head dim beyond 512
}

int ab200_set_kernel_family(int family) {
  int old = g_family;
  if (family >= 0 && family <= 3) g_family = family;
  return old;
}
int ab200_last_fwd_family(void) { return t_last_fwd; }
int ab200_last_bwd_family(void) { return t_last_bwd; }
unsigned int ab200_kernel_status(int reset) {
  unsigned int f = sm100_fwd_status(reset != 0), b = sm100_bwd_status(reset != 0);
  const unsigned int v = f ? f : b;
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    if (reset) g_failed_devices.fetch_and(~(uint64_t(1) << dev));
    else if (v != 0 && v != 0xffffffffu) g_failed_devices.fetch_or(uint64_t(1) << dev);
  }
  return v;
}

int ab200_stream_check(void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(st);
  cudaError_t e = host().stream_sync(st);
  if (e != cudaSuccess) return (int)e;
  return ab200_kernel_status(0) != 0 ? kErrLaunchFailure : 0;
}

void ab200_debug_host_calls(int fake_device, int fail_call, int fail_code, int fail_after) {
  g_fake_device.store(fake_device ? 1 : 0);
  g_fail_code.store(fail_code);
  g_fail_after.store(fail_after);
  g_fail_call.store(fail_call >= 0 && fail_call < kNumHostCalls ? fail_call : -1);
  for (auto& c : g_call_count) c.store(0);
}
uint64_t ab200_debug_host_call_count(int call) {
  return call >= 0 && call < kNumHostCalls ? g_call_count[call].load() : 0;
}

void ab200_debug_bounded_wait_test(int drop_copy, unsigned int wait_limit_kcycles) {
  t_drop_copy = (drop_copy >= 0 && drop_copy <= 3) ? drop_copy : 0;
  t_wait_limit_kcycles = wait_limit_kcycles;
}
uint64_t ab200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* ab200_version(void) { return "aotriton_b200 0.1 (sm_100a; API level of aotriton 0.14)"; }

int ab200_debug_simulate_encoded_softmax(const ab200_view4* r, int32_t dtype, int32_t batch, int32_t num_head_q,
                                         int32_t rows, int32_t cols, float dropout_p, const uint64_t* philox_seed,
                                         const uint64_t* philox_offset1, uint64_t philox_offset2, void* stream) {
  if (r == nullptr || r->ptr == nullptr) return kErrInvalidValue;
  if (dtype < AB200_DTYPE_FP32 || dtype > AB200_DTYPE_BF16) return kErrNotSupported;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  return (int)launch_dropout_sign(dtype, to_view(*r), batch, num_head_q, rows, cols, dropout_p, philox_seed,
                                  philox_offset1, philox_offset2, st);
}

int ab200_attn_fwd(const ab200_attn_fwd_args* a, void* stream) {
  if (a == nullptr) return kErrInvalidValue;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (int e = fill_common(a->prob, p)) return e;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->out.ptr) return kErrInvalidValue;
  if (!inner_contiguous(a->q) || !inner_contiguous(a->k) || !inner_contiguous(a->v) || !inner_contiguous(a->out))
    return kErrInvalidValue;
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  p.q = to_view(a->q); p.k = to_view(a->k); p.v = to_view(a->v); p.out = to_view(a->out);
  p.bias = to_view(a->bias); p.has_bias = a->bias.ptr != nullptr; p.bias_vec = rows_16byte(a->bias);
  p.lse = a->lse;
  p.seed_out = a->philox_seed_output; p.off_out = a->philox_offset_output;

  const int family = g_family;
  cudaError_t err;
  const int sel = ab200_select_variant(kOpFwd, a->prob.dtype, p.dqk, p.dvo,
                                       family_flags(family) | (sm100_fwd_supported(a->prob.dtype, p) ? AB200_SELECT_ALIGNED : 0));
  if (sel < 0) return -sel;
  if ((sel & 0xff) >= kVarTcgen05) {
    err = launch_sm100_fwd(a->prob.dtype, p, st);
    t_last_fwd = 2;
  } else {
    err = launch_general(0, a->prob.dtype, p, st);
    t_last_fwd = 1;
  }
  if (err != cudaSuccess) return (int)err;
  if (a->encoded_softmax.ptr != nullptr) {
    // The mask dump reuses the forward's head count, Max_seqlen_q/k and Philox inputs
    // (modules/flash/csrc/attn_debug.cc:13-29): rows/cols passed here size the grid only.
    View4 r = to_view(a->encoded_softmax);
    err = launch_dropout_sign(a->prob.dtype, r, p.batch, p.hq, p.max_sq, p.max_sk, p.dropout_p, p.seed_ptr,
                              p.off1_ptr, p.off2, st);
  }
  return (int)err;
}

static int fill_bwd(const ab200_attn_bwd_args* a, Params& p, bool need_outputs) {
  if (a == nullptr) return kErrInvalidValue;
  if (int e = fill_common(a->prob, p)) return e;
  if (!a->out.ptr || !a->dout.ptr || !a->delta) return kErrInvalidValue;
  if (!inner_contiguous(a->out) || !inner_contiguous(a->dout)) return kErrInvalidValue;
  p.out = to_view(a->out); p.dout = to_view(a->dout); p.delta = a->delta;
  p.lse = const_cast<float*>(a->lse);
  if (need_outputs) {
    if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->lse) return kErrInvalidValue;
    if (!inner_contiguous(a->q) || !inner_contiguous(a->k) || !inner_contiguous(a->v) || !inner_contiguous(a->dq) ||
        !inner_contiguous(a->dk) || !inner_contiguous(a->dv))
      return kErrInvalidValue;
  }
  p.q = to_view(a->q); p.k = to_view(a->k); p.v = to_view(a->v);
  p.bias = to_view(a->bias); p.has_bias = a->bias.ptr != nullptr; p.bias_vec = rows_16byte(a->bias);
  p.dq = to_view(a->dq); p.dk = to_view(a->dk); p.dv = to_view(a->dv); p.dbias = to_view(a->dbias);
  // dBias is skipped when absent or when all its strides are zero
  // (modules/flash/kernel/bwd_kernel_dq.py:265-266).
  p.has_dbias = a->dbias.ptr != nullptr &&
                (a->dbias.stride[0] | a->dbias.stride[1] | a->dbias.stride[2] | a->dbias.stride[3]) != 0;
  return 0;
}

int ab200_bwd_preprocess(const ab200_attn_bwd_args* a, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (int e = fill_bwd(a, p, false)) return e;
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  return (int)launch_preprocess(a->prob.dtype, p, st);
}

int ab200_bwd_dkdv(const ab200_attn_bwd_args* a, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (int e = fill_bwd(a, p, true)) return e;
  if (!a->dk.ptr || !a->dv.ptr) return kErrInvalidValue;
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  const int sel = ab200_select_variant(kOpBwd, a->prob.dtype, p.dqk, p.dvo,
                                       family_flags(g_family) | (sm100_bwd_supported(a->prob.dtype, p) ? AB200_SELECT_ALIGNED : 0));
  if (sel < 0) return -sel;
  if ((sel & 0xff) >= kVarTcgen05) {
    t_last_bwd = 2;
    return (int)launch_sm100_bwd_dkdv(a->prob.dtype, p, st);
  }
  t_last_bwd = 1;
  return (int)launch_general(1, a->prob.dtype, p, st);
}

int ab200_bwd_dq(const ab200_attn_bwd_args* a, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (int e = fill_bwd(a, p, true)) return e;
  if (!a->dq.ptr) return kErrInvalidValue;
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  const int sel = ab200_select_variant(kOpBwd, a->prob.dtype, p.dqk, p.dvo,
                                       family_flags(g_family) | (sm100_bwd_supported(a->prob.dtype, p) ? AB200_SELECT_ALIGNED : 0));
  if (sel < 0) return -sel;
  if ((sel & 0xff) >= kVarTcgen05) {
    t_last_bwd = 2;
    return (int)launch_sm100_bwd_dq(a->prob.dtype, p, st);
  }
  t_last_bwd = 1;
  return (int)launch_general(2, a->prob.dtype, p, st);
}

int ab200_bwd_uses_dq_acc(const ab200_attn_bwd_args* a, void* stream) {
  if (a == nullptr || a->deterministic || !want_fused(g_family)) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (fill_bwd(a, p, true) != 0 || !a->dq.ptr || !a->dk.ptr || !a->dv.ptr) return 0;
  if (check_device(st) != 0) return 0;
  const int sel = ab200_select_variant(kOpBwd, a->prob.dtype, p.dqk, p.dvo,
                                       AB200_SELECT_FUSED_REQUESTED | (p.has_dbias ? AB200_SELECT_DBIAS : 0) |
                                           (sm100_bwd_supported(a->prob.dtype, p) ? AB200_SELECT_ALIGNED : 0));
  return sel > 0 && (sel & 0xff) == kVarTcgen05Fused && sm100_bwd_fused_supported(a->prob.dtype, p) ? 1 : 0;
}

int ab200_bwd_fused(const ab200_attn_bwd_args* a, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Params p{};
  if (int e = fill_bwd(a, p, true)) return e;
  if (!a->dq.ptr || !a->dk.ptr || !a->dv.ptr || !a->dq_acc) return kErrInvalidValue;
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  if (!want_sm100(g_family) || !sm100_bwd_fused_supported(a->prob.dtype, p)) return kErrNotSupported;
  t_last_bwd = 3;
  return (int)launch_sm100_bwd_fused(a->prob.dtype, p, a->dq_acc, st);
}

int ab200_bwd_postprocess(const ab200_attn_bwd_args* a, void* stream) {
  if (a == nullptr || !a->dq.ptr || !a->dq_acc) return kErrInvalidValue;
  if (a->prob.dtype < AB200_DTYPE_FP32 || a->prob.dtype > AB200_DTYPE_BF16) return kErrNotSupported;
  if (!inner_contiguous(a->dq)) return kErrInvalidValue;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  View4 dq = to_view(a->dq);
  dq.n[3] = a->prob.head_dim_qk;
  return (int)launch_postprocess(a->prob.dtype, dq, a->dq_acc, a->prob.sm_scale, st);
}

int ab200_attn_bwd(const ab200_attn_bwd_args* a, void* stream) {
  if (a == nullptr) return kErrInvalidValue;
  if (!a->dq.ptr || !a->dk.ptr || !a->dv.ptr) return kErrInvalidValue;
  if (int e = ab200_bwd_preprocess(a, stream)) return e;
  if (a->dq_acc != nullptr && ab200_bwd_uses_dq_acc(a, stream)) {
    if (int e = ab200_bwd_fused(a, stream)) return e;
    return ab200_bwd_postprocess(a, stream);
  }
  if (int e = ab200_bwd_dkdv(a, stream)) return e;
  return ab200_bwd_dq(a, stream);
}

// --- backward with the delta scratch inside the library image -----------------------------
// For hosts that have no device memory left to lend and no allocator to call back into.  The
// array below is what `args->delta` would otherwise point to.  In host code its name is only a
// handle: the device address is looked up once per device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) float g_static_delta[AB200_STATIC_DELTA_FLOATS];

namespace {
// Device address of g_static_delta on `dev`, which must be the current device; nullptr on error.
float* static_delta_address(int dev, cudaError_t* err) {
  static std::mutex mu;
  static float* table[64] = {};
  *err = cudaSuccess;
  if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    int cur = -1;
    if ((*err = host().get_device(&cur)) != cudaSuccess) return nullptr;
    if (cur != dev) { *err = cudaErrorInvalidDevice; return nullptr; }   // symbol lookup is per current device
    float* ptr = nullptr;
    if ((*err = host().symbol_address(reinterpret_cast<void**>(&ptr), reinterpret_cast<const void*>(&g_static_delta))) !=
        cudaSuccess)
      return nullptr;
    if (fake()) return ptr;       // (a pretended device's address is not remembered)
    table[dev] = ptr;
  }
  return table[dev];
}
}  // namespace

int ab200_attn_bwd_static_scratch(const ab200_attn_bwd_args* a, void* stream) {
  if (a == nullptr) return kErrInvalidValue;
  if (!a->dq.ptr || !a->dk.ptr || !a->dv.ptr) return kErrInvalidValue;
  const ab200_attn_problem& pr = a->prob;
  // Rows of the logsumexp / delta matrix: dense and padded layouts are (batch*Hq, max_sq);
  // token-packed varlen is (Hq, tokens in the packed q tensor).
  const bool packed = pr.cu_seqlens_q != nullptr && pr.varlen_type != AB200_VARLEN_PADDED;
  // The kernels index delta up to the packed token count, which they read on the device
  // (cu_seqlens_q[batch], or seq_strides_q[batch]); the host can only bound it by the extent the
  // caller declares for q, so a packed call without that extent is refused.
  if (packed && a->q.size[2] <= 0) {
    std::fprintf(stderr, "[aotriton_b200] ab200_attn_bwd_static_scratch: token-packed varlen needs q.size[2] "
                         "(the packed token count) to bound the built-in scratch\n");
    return kErrInvalidValue;
  }
  const long long dense_rows = (long long)pr.batch * (long long)pr.max_seqlen_q;
  const long long tokens = packed ? ((long long)a->q.size[2] < dense_rows ? (long long)a->q.size[2] : dense_rows)
                                  : dense_rows;
  const long long need = (long long)pr.num_head_q * tokens;
  if (need < 0 || need > (long long)AB200_STATIC_DELTA_FLOATS) {
    std::fprintf(stderr,
                 "[aotriton_b200] ab200_attn_bwd_static_scratch: delta needs %lld floats, the built-in scratch "
                 "holds %u; use ab200_attn_bwd with a caller-provided delta buffer\n",
                 need, (unsigned)AB200_STATIC_DELTA_FLOATS);
    return kErrInvalidValue;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = check_device(st)) return e;
  DeviceGuard guard(st);
  cudaError_t cerr;
  float* delta = static_delta_address(stream_device(st), &cerr);
  if (delta == nullptr) return (int)cerr;
  ab200_attn_bwd_args b = *a;
  b.delta = delta;
  return ab200_attn_bwd(&b, stream);
}

// --- HIP-named runtime helpers used by the Python tests of the reference
// (bindings/hipruntime.cc:92-93).  CUDA and HIP number their common errors alike.
AB200_API int hipGetLastError(void) { return (int)cudaGetLastError(); }
AB200_API int hipDeviceSynchronize(void) { return (int)cudaDeviceSynchronize(); }

}  // extern "C"
