// C++ operator API (include/aotriton/flash.h, util.h) on top of the C-ABI launcher.
//
// Mirrors the host logic of ROCm/aotriton modules/flash/csrc/attn_fwd.cc:49-149,
// attn_bwd.cc:56-160, attn_check.cc:36-46, attn_debug.cc:31-69 and v3src/util.cc:65-117:
// version check, shape inference from the views, varlen detection, lazy tensors
// acquired before and released after the backward launches.  What the reference
// does next -- tuning-database lookup, kernel image loading -- has no counterpart
// here: the call goes straight to ab200_attn_fwd / ab200_attn_bwd.
#define aotriton_v2_EXPORTS 1
#include <aotriton/flash.h>
#include <aotriton/util.h>
#include <aotriton_b200.h>

#include <cstdio>
#include <cstdlib>
#include <cstdarg>

namespace AOTRITON_NS {

template class TensorView<1>;
template class TensorView<2>;
template class TensorView<3>;
template class TensorView<4>;

namespace {

// AOTRITON_DEBUG_LEVEL=0..5 enables stderr logging, like the reference's AOTRITON_LOG.
int debug_level() {
  static int level = [] {
    const char* e = std::getenv("AOTRITON_DEBUG_LEVEL");
    return e ? std::atoi(e) : 0;
  }();
  return level;
}

void log_debug(const char* fmt, ...) {
  if (debug_level() < 4) return;
  va_list ap;
  va_start(ap, fmt);
  std::fprintf(stderr, "[aotriton_b200] ");
  std::vfprintf(stderr, fmt, ap);
  std::fprintf(stderr, "\n");
  va_end(ap);
}

ab200_view4 cview(const TensorView<4>& t) {
  ab200_view4 v;
  v.ptr = t.data_ptr();
  for (int i = 0; i < 4; ++i) {
    v.size[i] = t ? (int64_t)t.size(i) : 0;
    v.stride[i] = t ? (int64_t)t.stride(i) : 0;
  }
  return v;
}

int cdtype(DType d) {
  switch (d) {
    case kFloat32: return AB200_DTYPE_FP32;
    case kFloat16: return AB200_DTYPE_FP16;
    case kBFloat16: return AB200_DTYPE_BF16;
    default: return AB200_DTYPE_UNKNOWN;
  }
}

template <typename P>
void fill_problem(const P& in, ab200_attn_problem& pr) {
  pr.dtype = cdtype(in.Q.dtype());
  int batch = (int)in.Q.size(0);
  pr.num_head_q = (int)in.Q.size(1);
  pr.num_head_k = (int)in.K.size(1);
  pr.max_seqlen_q = (int)in.Q.size(2);
  pr.max_seqlen_k = (int)in.K.size(2);
  pr.head_dim_qk = (int)in.Q.size(3);
  pr.head_dim_vo = (int)in.V.size(3);
  pr.cu_seqlens_q = nullptr; pr.cu_seqlens_k = nullptr; pr.seq_strides_q = nullptr; pr.seq_strides_k = nullptr;
  if (in.cu_seqlens_q) {   // varlen: batch is the number of sequences
    batch = (int)in.cu_seqlens_q.size(0) - 1;
    pr.max_seqlen_q = in.Max_seqlen_q;
    pr.cu_seqlens_q = static_cast<const int32_t*>(in.cu_seqlens_q.data_ptr());
  }
  if (in.cu_seqlens_k) {
    pr.max_seqlen_k = in.Max_seqlen_k;
    pr.cu_seqlens_k = static_cast<const int32_t*>(in.cu_seqlens_k.data_ptr());
  }
  if (in.seq_strides_q) pr.seq_strides_q = static_cast<const int32_t*>(in.seq_strides_q.data_ptr());
  if (in.seq_strides_k) pr.seq_strides_k = static_cast<const int32_t*>(in.seq_strides_k.data_ptr());
  pr.batch = batch;
  pr.sm_scale = in.Sm_scale;
  pr.causal_type = in.causal_type;
  pr.window_left = in.window_left;
  pr.window_right = in.window_right;
  pr.varlen_type = in.varlen_type;
  pr.dropout_p = in.dropout_p;
  pr.philox_seed = static_cast<const uint64_t*>(in.philox_seed_ptr.data_ptr());
  pr.philox_offset1 = static_cast<const uint64_t*>(in.philox_offset1.data_ptr());
  pr.philox_offset2 = in.philox_offset2;
  pr.philox_head_offset = 0;
  pr.philox_num_head_q = 0;
}

// force_backend_index: -1 automatic, 0 general kernels, 1 tcgen05 kernels, 2 automatic with the
// fused (dQ accumulator) backward where it applies.
struct FamilyGuard {
  int old_ = -1; bool active_ = false;
  explicit FamilyGuard(const v3::flash::attn_options* o) {
    if (o && o->force_backend_index >= 0) {
      active_ = true;
      old_ = ab200_set_kernel_family(o->force_backend_index == 0 ? 1 : (o->force_backend_index == 1 ? 2 : 3));
    }
  }
  ~FamilyGuard() { if (active_) ab200_set_kernel_family(old_); }
};

}  // namespace

Gpu getGpuFromStream(hipStream_t stream) {
  return ab200_check_gpu(stream) == 0 ? GPU_NVIDIA_ARCH_SM100_MOD0 : GPU_ARCH_UNKNOWN;
}
bool isArchExperimentallySupported(hipStream_t) { return false; }
bool isArchTechPreview(hipStream_t) { return false; }
int getMultiProcessorCount(hipStream_t stream) { return ab200_multiprocessor_count(stream); }

namespace v2::flash {

hipError_t check_gpu(AOTRITON_NS::Stream stream) {
  return static_cast<hipError_t>(ab200_check_gpu(stream.native()));
}

hipError_t debug_simulate_encoded_softmax(AOTRITON_NS::TensorView<4> r, float dropout_p,
                                          AOTRITON_NS::TensorView<0> philox_seed,
                                          AOTRITON_NS::TensorView<0> philox_offset1, uint64_t philox_offset2,
                                          AOTRITON_NS::Stream stream) {
  ab200_view4 v = cview(r);
  return static_cast<hipError_t>(ab200_debug_simulate_encoded_softmax(
      &v, cdtype(r.dtype()), (int)r.size(0), (int)r.size(1), (int)r.size(2), (int)r.size(3), dropout_p,
      static_cast<const uint64_t*>(philox_seed.data_ptr()), static_cast<const uint64_t*>(philox_offset1.data_ptr()),
      philox_offset2, stream.native()));
}

}  // namespace v2::flash

namespace v3::flash {

attn_fwd_params::attn_fwd_params() {}
attn_bwd_params::attn_bwd_params() {}

hipError_t attn_fwd(const attn_fwd_params& in, int32_t params_version, AOTRITON_NS::Stream stream,
                    const attn_options* options) {
  if (params_version != attn_fwd_params::kVersion) return hipErrorInvalidSymbol;
  ab200_attn_fwd_args a{};
  fill_problem(in, a.prob);
  a.q = cview(in.Q); a.k = cview(in.K); a.v = cview(in.V); a.bias = cview(in.B); a.out = cview(in.Out);
  a.lse = static_cast<float*>(in.L.data_ptr());
  a.philox_seed_output = static_cast<uint64_t*>(in.philox_seed_output.data_ptr());
  a.philox_offset_output = static_cast<uint64_t*>(in.philox_offset_output.data_ptr());
  a.encoded_softmax = cview(in.encoded_softmax);
  if (in.encoded_softmax) {
    a.encoded_softmax_rows = (int)in.encoded_softmax.size(2);
    a.encoded_softmax_cols = (int)in.encoded_softmax.size(3);
  }
  a.persistent_atomic_counter = static_cast<int32_t*>(in.persistent_atomic_counter.data_ptr());
  log_debug("attn_fwd B=%d Hq=%d Hk=%d Sq=%d Sk=%d Dqk=%d Dvo=%d causal=%d varlen=%d p=%g", a.prob.batch,
            a.prob.num_head_q, a.prob.num_head_k, a.prob.max_seqlen_q, a.prob.max_seqlen_k, a.prob.head_dim_qk,
            a.prob.head_dim_vo, a.prob.causal_type, a.prob.varlen_type, a.prob.dropout_p);
  FamilyGuard guard(options);
  return static_cast<hipError_t>(ab200_attn_fwd(&a, stream.native()));
}

hipError_t attn_bwd(const attn_bwd_params& in, int32_t params_version, AOTRITON_NS::Stream stream,
                    const attn_options* options) {
  if (params_version != attn_bwd_params::kVersion) return hipErrorInvalidSymbol;
  ab200_attn_bwd_args a{};
  fill_problem(in, a.prob);
  a.q = cview(in.Q); a.k = cview(in.K); a.v = cview(in.V); a.bias = cview(in.B);
  a.out = cview(in.Out); a.dout = cview(in.DO);
  a.dq = cview(in.DQ); a.dk = cview(in.DK); a.dv = cview(in.DV); a.dbias = cview(in.DB);
  a.lse = static_cast<const float*>(in.L.data_ptr());
  a.deterministic = options ? (options->deterministic ? 1 : 0) : 0;
  // delta: use the eager view if the caller supplied one, else ask the caller's allocator.
  TensorView<2> delta = in.D.eager;
  if (!delta && in.D.acquire) delta = (*in.D.acquire)(&in.D);
  hipError_t err;
  if (!delta) {
    err = hipErrorInvalidValue;
  } else {
    a.delta = static_cast<float*>(delta.data_ptr());
    // dQ accumulator: acquired (zero-filled by the caller's allocator) only when the fused form
    // will run, i.e. not for deterministic calls (modules/flash/csrc/attn_bwd.cc:140-154).
    FamilyGuard guard_acc(options);
    if (in.DQ_ACC && ab200_bwd_uses_dq_acc(&a, stream.native())) {
      TensorView<4> acc = in.DQ_ACC.eager;
      if (!acc && in.DQ_ACC.acquire) acc = (*in.DQ_ACC.acquire)(&in.DQ_ACC);
      if (acc && acc.dtype() == kFloat32) a.dq_acc = static_cast<float*>(acc.data_ptr());
    }
    log_debug("attn_bwd B=%d Hq=%d Hk=%d Sq=%d Sk=%d Dqk=%d Dvo=%d causal=%d varlen=%d p=%g", a.prob.batch,
              a.prob.num_head_q, a.prob.num_head_k, a.prob.max_seqlen_q, a.prob.max_seqlen_k, a.prob.head_dim_qk,
              a.prob.head_dim_vo, a.prob.causal_type, a.prob.varlen_type, a.prob.dropout_p);
    err = static_cast<hipError_t>(ab200_attn_bwd(&a, stream.native()));
  }
  // Lazy tensors are released before returning, whatever happened (attn_bwd.cc:157-158).
  in.D.free();
  in.DQ_ACC.free();
  return err;
}

}  // namespace v3::flash

namespace v2::flash {

namespace {
void causal_fields(bool is_causal, int32_t wl, int32_t wr, int8_t& type, int32_t& left, int32_t& right) {
  if (!is_causal) { type = v3::flash::CausalType::None; left = 0; right = 0; return; }
  type = v3::flash::CausalType::WindowedAttention;
  left = wl; right = wr;
}
}  // namespace

hipError_t attn_fwd_compact_varlen(T4 q, T4 k, T4 v, T4 b, T1 cu_seqlens_q, T1 cu_seqlens_k, int32_t max_seqlen_q,
                                   int32_t max_seqlen_k, float sm_scale, T2 softmax_lse, T4 out, float dropout_p,
                                   T0 philox_seed, T0 philox_offset1, uint64_t philox_offset2, T0 philox_seed_output,
                                   T0 philox_offset_output, T4 encoded_softmax, bool is_causal, int32_t window_left,
                                   int32_t window_right, AOTRITON_NS::Stream stream) {
  v3::flash::attn_fwd_params p;
  p.Q = q; p.K = k; p.V = v; p.B = b; p.Sm_scale = sm_scale; p.L = softmax_lse; p.Out = out;
  p.cu_seqlens_q = cu_seqlens_q; p.cu_seqlens_k = cu_seqlens_k;
  p.Max_seqlen_q = max_seqlen_q; p.Max_seqlen_k = max_seqlen_k;
  p.dropout_p = dropout_p; p.philox_seed_ptr = philox_seed; p.philox_offset1 = philox_offset1;
  p.philox_offset2 = philox_offset2; p.philox_seed_output = philox_seed_output;
  p.philox_offset_output = philox_offset_output; p.encoded_softmax = encoded_softmax;
  causal_fields(is_causal, window_left, window_right, p.causal_type, p.window_left, p.window_right);
  p.varlen_type = cu_seqlens_q ? v3::flash::VarlenType::CompactVarlen : v3::flash::VarlenType::None;
  return v3::flash::attn_fwd(p, v3::flash::attn_fwd_params::kVersion, stream, nullptr);
}

hipError_t attn_fwd(T4 q, T4 k, T4 v, T4 b, float sm_scale, T2 softmax_lse, T4 out, float dropout_p, T0 philox_seed,
                    T0 philox_offset1, uint64_t philox_offset2, T0 philox_seed_output, T0 philox_offset_output,
                    T4 encoded_softmax, bool is_causal, int32_t window_left, int32_t window_right,
                    AOTRITON_NS::Stream stream) {
  return attn_fwd_compact_varlen(q, k, v, b, T1(), T1(), 0, 0, sm_scale, softmax_lse, out, dropout_p, philox_seed,
                                 philox_offset1, philox_offset2, philox_seed_output, philox_offset_output,
                                 encoded_softmax, is_causal, window_left, window_right, stream);
}

hipError_t attn_bwd_compact_varlen(T4 q, T4 k, T4 v, T1 cu_seqlens_q, T1 cu_seqlens_k, int32_t max_seqlen_q,
                                   int32_t max_seqlen_k, T4 b, float sm_scale, T4 out, T4 dout, T4 dq, T4 dk, T4 dv,
                                   T4 db, T2 softmax_lse, T2 delta, float dropout_p, T0 philox_seed, T0 philox_offset1,
                                   uint64_t philox_offset2, bool is_causal, int32_t window_left, int32_t window_right,
                                   AOTRITON_NS::Stream stream) {
  v3::flash::attn_bwd_params p;
  p.Q = q; p.K = k; p.V = v; p.B = b; p.Sm_scale = sm_scale; p.Out = out; p.DO = dout;
  p.DQ = dq; p.DK = dk; p.DV = dv; p.DB = db; p.L = softmax_lse;
  p.D.eager = delta;
  p.cu_seqlens_q = cu_seqlens_q; p.cu_seqlens_k = cu_seqlens_k;
  p.Max_seqlen_q = max_seqlen_q; p.Max_seqlen_k = max_seqlen_k;
  p.dropout_p = dropout_p; p.philox_seed_ptr = philox_seed; p.philox_offset1 = philox_offset1;
  p.philox_offset2 = philox_offset2;
  causal_fields(is_causal, window_left, window_right, p.causal_type, p.window_left, p.window_right);
  p.varlen_type = cu_seqlens_q ? v3::flash::VarlenType::CompactVarlen : v3::flash::VarlenType::None;
  return v3::flash::attn_bwd(p, v3::flash::attn_bwd_params::kVersion, stream, nullptr);
}

hipError_t attn_bwd(T4 q, T4 k, T4 v, T4 b, float sm_scale, T4 out, T4 dout, T4 dq, T4 dk, T4 dv, T4 db,
                    T2 softmax_lse, T2 delta, float dropout_p, T0 philox_seed, T0 philox_offset1,
                    uint64_t philox_offset2, bool is_causal, int32_t window_left, int32_t window_right,
                    AOTRITON_NS::Stream stream) {
  return attn_bwd_compact_varlen(q, k, v, T1(), T1(), 0, 0, b, sm_scale, out, dout, dq, dk, dv, db, softmax_lse,
                                 delta, dropout_p, philox_seed, philox_offset1, philox_offset2, is_causal,
                                 window_left, window_right, stream);
}

}  // namespace v2::flash

}  // namespace AOTRITON_NS
