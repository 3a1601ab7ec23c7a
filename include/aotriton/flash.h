// FlashAttention operator API -- drop-in for ROCm/aotriton include/aotriton/flash.h.
//
//   v2::flash   check_gpu, debug_simulate_encoded_softmax            (flash.h:12-26)
//   v3::flash   attn_options, CausalType, WindowValue, VarlenType,
//               attn_fwd_params/attn_fwd, attn_bwd_params/attn_bwd   (flash.h:28-182)
//
// Struct members keep the reference's order and types because the structs are
// filled by callers and read by the library across a shared-object boundary.
// The entry points validate on the host, translate to the C-ABI of
// include/aotriton_b200.h and launch sm_100a kernels asynchronously.
#ifndef AOTRITON_V3_API_FLASH_ATTN_H
#define AOTRITON_V3_API_FLASH_ATTN_H

#include <aotriton/config.h>
#include "runtime.h"
#include "util.h"
#include "cpp_tune.h"

namespace AOTRITON_NS::v2::flash {

// hipSuccess iff the stream's device is one this library has kernels for.
hipError_t AOTRITON_API check_gpu(AOTRITON_NS::Stream stream);

// Fills r (batch x heads x max_seqlen_q x max_seqlen_k) with +0.5 / -0.5 according
// to the dropout keep bit, so tests can recover the mask the kernels use.
hipError_t AOTRITON_API debug_simulate_encoded_softmax(AOTRITON_NS::TensorView<4> r,
                                                       float dropout_p,
                                                       AOTRITON_NS::TensorView<0> philox_seed,
                                                       AOTRITON_NS::TensorView<0> philox_offset1,
                                                       uint64_t philox_offset2,
                                                       AOTRITON_NS::Stream stream);

}  // namespace AOTRITON_NS::v2::flash

namespace AOTRITON_NS::v3::flash {

using T4 = AOTRITON_NS::TensorView<4>;
using T2 = AOTRITON_NS::TensorView<2>;
using T1 = AOTRITON_NS::TensorView<1>;
using T0 = AOTRITON_NS::TensorView<0>;
using LT2 = AOTRITON_NS::LazyTensor<2>;
using LT4 = AOTRITON_NS::LazyTensor<4>;

// Per-call knobs.  force_backend_index: -1 automatic, 0 the general kernels,
// 1 the tcgen05 kernels (hipErrorNotSupported if the shape is outside their
// range), 2 automatic, with the fused backward where it applies: it uses DQ_ACC
// and adds dQ partials with floating-point atomics (run-to-run differences in
// the last bits).  deterministic: true never uses the fused backward; the automatic
// choice does not either, since the two-kernel backward measured faster.
struct AOTRITON_API attn_options {
  int force_backend_index = -1;
  bool deterministic = false;
};

// Plain int8/int32 constants rather than enum classes: the values are stored
// into integer struct members by callers.
struct AOTRITON_API CausalType {
  static constexpr int8_t None = 0;
  static constexpr int8_t WindowedAttention = 3;
};

// Window sentinels: "as wide as the sequence, aligned to this corner".  Needed
// for varlen, where no single integer fits every sequence.
struct AOTRITON_API WindowValue {
  static constexpr int32_t TopLeftAligned = -2147483647;
  static constexpr int32_t BottomRightAligned = -2147483646;
};

struct AOTRITON_API VarlenType {
  static constexpr int8_t None = 0;
  static constexpr int8_t CompactVarlen = 1;
  static constexpr int8_t PaddedVarlen = 2;
  static constexpr int8_t StridedVarlen = 3;
};

struct AOTRITON_API attn_fwd_params {
  T4       Q;
  T4       K;
  T4       V;
  T4       B;                   // additive bias, null when unused
  T2       A;                   // alibi slopes: declared for layout, not supported
  float    Sm_scale;
  T2       L;                   // logsumexp out, may be null
  T4       Out;
  T1       cu_seqlens_q;        // int32, presence selects varlen
  T1       cu_seqlens_k;
  int32_t  Max_seqlen_q = 0;    // varlen only
  int32_t  Max_seqlen_k = 0;
  T1       seq_strides_q;       // strided varlen: per-sequence token offsets
  T1       seq_strides_k;
  float    dropout_p;
  T0       philox_seed_ptr;     // device uint64 scalars
  T0       philox_offset1;
  uint64_t philox_offset2;
  T0       philox_seed_output;  // may be null
  T0       philox_offset_output;
  T4       encoded_softmax;     // debugging only, normally null
  T0       persistent_atomic_counter;
  int8_t   causal_type;
  int8_t   varlen_type = 0;
  int32_t  window_left;
  int32_t  window_right;

  static constexpr int32_t kVersion = 3;
  attn_fwd_params();
};

hipError_t AOTRITON_API attn_fwd(const attn_fwd_params& params,
                                 int32_t params_version,
                                 AOTRITON_NS::Stream stream,
                                 const attn_options* options = nullptr);

struct AOTRITON_API attn_bwd_params {
  T4        Q;
  T4        K;
  T4        V;
  T4        B;
  float     Sm_scale;
  T4        Out;
  T4        DO;
  T4        DK;
  T4        DV;
  T4        DQ;
  T4        DB;
  T2        L;
  mutable LT2 D;                // delta scratch, acquired by the library
  T1        cu_seqlens_q;
  T1        cu_seqlens_k;
  int32_t   Max_seqlen_q = 0;
  int32_t   Max_seqlen_k = 0;
  T1        seq_strides_q;
  T1        seq_strides_k;
  float     dropout_p;
  T0        philox_seed_ptr;
  T0        philox_offset1;
  uint64_t  philox_offset2;
  int8_t    causal_type;
  int8_t    varlen_type = 0;
  int32_t   window_left;
  int32_t   window_right;
  mutable LT4 DQ_ACC;           // fp32 dQ accumulator; never acquired by this library

  static constexpr int32_t kVersion = 6;
  attn_bwd_params();
};

hipError_t AOTRITON_API attn_bwd(const attn_bwd_params& params,
                                 int32_t params_version,
                                 AOTRITON_NS::Stream stream,
                                 const attn_options* options = nullptr);

}  // namespace AOTRITON_NS::v3::flash

// The v2-named positional entry points.  ROCm/aotriton 0.14 no longer declares
// them (its flash.h:12-26 keeps only the two helpers above), so their argument
// lists are not pinned by the reference; they are thin forwards that fill the v3
// parameter structs.
namespace AOTRITON_NS::v2::flash {

using T4 = AOTRITON_NS::TensorView<4>;
using T2 = AOTRITON_NS::TensorView<2>;
using T1 = AOTRITON_NS::TensorView<1>;
using T0 = AOTRITON_NS::TensorView<0>;

hipError_t AOTRITON_API attn_fwd(T4 q, T4 k, T4 v, T4 b, float sm_scale, T2 softmax_lse, T4 out,
                                 float dropout_p, T0 philox_seed, T0 philox_offset1, uint64_t philox_offset2,
                                 T0 philox_seed_output, T0 philox_offset_output, T4 encoded_softmax,
                                 bool is_causal, int32_t window_left, int32_t window_right,
                                 AOTRITON_NS::Stream stream);

hipError_t AOTRITON_API attn_fwd_compact_varlen(T4 q, T4 k, T4 v, T4 b,
                                                T1 cu_seqlens_q, T1 cu_seqlens_k,
                                                int32_t max_seqlen_q, int32_t max_seqlen_k,
                                                float sm_scale, T2 softmax_lse, T4 out,
                                                float dropout_p, T0 philox_seed, T0 philox_offset1,
                                                uint64_t philox_offset2,
                                                T0 philox_seed_output, T0 philox_offset_output,
                                                T4 encoded_softmax,
                                                bool is_causal, int32_t window_left, int32_t window_right,
                                                AOTRITON_NS::Stream stream);

hipError_t AOTRITON_API attn_bwd(T4 q, T4 k, T4 v, T4 b, float sm_scale, T4 out, T4 dout,
                                 T4 dq, T4 dk, T4 dv, T4 db, T2 softmax_lse, T2 delta,
                                 float dropout_p, T0 philox_seed, T0 philox_offset1, uint64_t philox_offset2,
                                 bool is_causal, int32_t window_left, int32_t window_right,
                                 AOTRITON_NS::Stream stream);

hipError_t AOTRITON_API attn_bwd_compact_varlen(T4 q, T4 k, T4 v,
                                                T1 cu_seqlens_q, T1 cu_seqlens_k,
                                                int32_t max_seqlen_q, int32_t max_seqlen_k,
                                                T4 b, float sm_scale, T4 out, T4 dout,
                                                T4 dq, T4 dk, T4 dv, T4 db, T2 softmax_lse, T2 delta,
                                                float dropout_p, T0 philox_seed, T0 philox_offset1,
                                                uint64_t philox_offset2,
                                                bool is_causal, int32_t window_left, int32_t window_right,
                                                AOTRITON_NS::Stream stream);

}  // namespace AOTRITON_NS::v2::flash

#endif  // AOTRITON_V3_API_FLASH_ATTN_H
