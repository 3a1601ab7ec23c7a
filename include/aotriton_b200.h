/*
 * aotriton_b200.h -- C-ABI of the B200 FlashAttention launcher.
 *
 * Everything the C++ operator API (include/aotriton/flash.h) and the Python
 * bindings do on the device goes through the functions declared here.  The
 * signatures use plain pointers, integers and POD structs only, so the same
 * library can be bound from C, ctypes, cgo or any other FFI.
 *
 * Conventions
 *   - Every pointer inside the structs is a DEVICE pointer unless stated.
 *   - Strides are in ELEMENTS (not bytes), the innermost stride must be 1.
 *   - Logical tensor order is (batch, head, sequence, head_dim) whatever the
 *     storage order is; permuted storage (BSHD, THD) is expressed by strides.
 *   - Return value: 0 on success, otherwise a HIP/CUDA-compatible error
 *     number (see include/hip/hip_runtime.h for the names used).
 *   - All launches are asynchronous on `stream` (a cudaStream_t passed as
 *     void*; NULL is the default stream).  Nothing is allocated or freed.
 *
 * Each entry point cites the interface of ROCm/aotriton it stands in for.
 */
#ifndef AOTRITON_B200_CABI_H
#define AOTRITON_B200_CABI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_MSC_VER)
#define AB200_API __declspec(dllexport)
#else
#define AB200_API __attribute__((visibility("default")))
#endif

/* Element types; numeric values equal aotriton::DType (include/aotriton/dtypes.h:12-25). */
enum ab200_dtype {
  AB200_DTYPE_UNKNOWN = 0,
  AB200_DTYPE_FP32 = 1,
  AB200_DTYPE_FP16 = 2,
  AB200_DTYPE_BF16 = 3
};

/* causal_type values (include/aotriton/flash.h:76-81). */
enum { AB200_CAUSAL_NONE = 0, AB200_CAUSAL_WINDOWED = 3 };
/* window sentinels (include/aotriton/flash.h:83-86). */
enum { AB200_WINDOW_TOP_LEFT = -2147483647, AB200_WINDOW_BOTTOM_RIGHT = -2147483646 };
/* varlen_type values (include/aotriton/flash.h:88-93). */
enum { AB200_VARLEN_NONE = 0, AB200_VARLEN_COMPACT = 1, AB200_VARLEN_PADDED = 2, AB200_VARLEN_STRIDED = 3 };

/* A rank-4 strided view: logical (batch, head, seq, dim). ptr == NULL means "absent".
 * size[] are the extents of the tensor the view was taken from (for compact varlen the
 * sequence extent is the total token count); the tcgen05 kernels bound their bulk
 * copies with them. */
typedef struct ab200_view4 {
  void* ptr;
  int64_t size[4];
  int64_t stride[4];
} ab200_view4;

/*
 * Problem description shared by forward and backward
 * (fields of attn_fwd_params / attn_bwd_params, include/aotriton/flash.h:96-174,
 * after the inference done in modules/flash/csrc/attn_fwd.cc:59-75).
 */
typedef struct ab200_attn_problem {
  int32_t dtype;          /* ab200_dtype of Q/K/V/Out/bias and the gradients          */
  int32_t batch;          /* dense: Q.size(0); varlen: number of sequences            */
  int32_t num_head_q;
  int32_t num_head_k;     /* num_head_q % num_head_k == 0 (GQA)                        */
  int32_t max_seqlen_q;   /* dense: Q.size(2); varlen: Max_seqlen_q                    */
  int32_t max_seqlen_k;
  int32_t head_dim_qk;
  int32_t head_dim_vo;
  float sm_scale;
  int32_t causal_type;    /* AB200_CAUSAL_*                                            */
  int32_t window_left;    /* integers or AB200_WINDOW_* sentinels                      */
  int32_t window_right;
  int32_t varlen_type;    /* AB200_VARLEN_*                                            */
  const int32_t* cu_seqlens_q;   /* batch+1 entries, NULL when dense                  */
  const int32_t* cu_seqlens_k;
  const int32_t* seq_strides_q;  /* strided varlen: batch+1 entries, else NULL         */
  const int32_t* seq_strides_k;
  float dropout_p;
  const uint64_t* philox_seed;     /* device scalar, NULL -> 0                         */
  const uint64_t* philox_offset1;  /* device scalar, NULL -> 0                         */
  uint64_t philox_offset2;         /* host scalar added to *philox_offset1             */
  /* Sharding support: when a caller splits the q-head axis over several GPUs it
   * passes the position of this shard in the unsharded problem so that dropout
   * masks stay identical.  0/0 means "not sharded". */
  int32_t philox_head_offset;
  int32_t philox_num_head_q;
} ab200_attn_problem;

/* Forward tensors (attn_fwd_params, include/aotriton/flash.h:96-130). */
typedef struct ab200_attn_fwd_args {
  ab200_attn_problem prob;
  ab200_view4 q, k, v, bias, out;
  float* lse;                       /* (batch*Hq, max_seqlen_q) or (Hq, total_q); may be NULL */
  uint64_t* philox_seed_output;     /* may be NULL */
  uint64_t* philox_offset_output;   /* may be NULL */
  ab200_view4 encoded_softmax;      /* debugging aid, normally absent */
  int32_t encoded_softmax_rows;     /* size(2) of encoded_softmax */
  int32_t encoded_softmax_cols;     /* size(3) of encoded_softmax */
  int32_t* persistent_atomic_counter; /* accepted for compatibility, never required */
} ab200_attn_fwd_args;

/* Backward tensors (attn_bwd_params, include/aotriton/flash.h:138-174). */
typedef struct ab200_attn_bwd_args {
  ab200_attn_problem prob;
  ab200_view4 q, k, v, bias, out, dout;
  ab200_view4 dq, dk, dv, dbias;    /* dbias absent or all-zero strides -> not written; otherwise every entry inside
                                     * the sequences is written, zero where a causal or windowed problem masks it (the
                                     * reference stores dB only in the key blocks its loop visits,
                                     * modules/flash/kernel/bwd_inner_dq.py:200-204) */
  const float* lse;                 /* as written by the forward */
  float* delta;                     /* scratch, same shape as lse (the "D" lazy tensor) */
  int32_t deterministic;            /* attn_options::deterministic: non-zero forbids the fused form below */
  /* Optional fp32 dQ accumulator (the "DQ_ACC" lazy tensor, include/aotriton/flash.h:170): contiguous
   * in dq's logical order, dq.size[0] * dq.size[1] * dq.size[2] * head_dim_qk floats, ZERO on entry
   * (the reference's allocator callback returns zeros).  When it is given, `deterministic` is 0, the
   * fused form was asked for (kernel family 3) and the problem qualifies (ab200_bwd_uses_dq_acc),
   * ab200_attn_bwd runs the fused form: one kernel
   * produces dK, dV and adds dQ partials here with atomics, a conversion kernel writes dq.  The
   * accumulator holds the unscaled sum afterwards.  NULL selects the two-kernel form. */
  float* dq_acc;
} ab200_attn_bwd_args;

/* Replaces aotriton::v3::flash::attn_fwd's launch (modules/flash/csrc/attn_fwd.cc:49-149). */
AB200_API int ab200_attn_fwd(const ab200_attn_fwd_args* args, void* stream);

/* Replaces aotriton::v3::flash::attn_bwd's three launches
 * (modules/flash/csrc/attn_bwd.cc:56-160: bwd_preprocess, bwd_kernel_dk_dv, bwd_kernel_dq). */
AB200_API int ab200_attn_bwd(const ab200_attn_bwd_args* args, void* stream);

/*
 * Backward for callers that can neither hand the library a delta buffer nor let it ask an
 * allocator for one.  This entry point has no counterpart in the reference, whose backward
 * always obtains delta through the caller's LazyTensor allocator callback.
 *
 * Who needs it: hosts that planned all device memory up front and have none left to give
 * (fixed-arena inference or training runtimes), and FFI callers (C, Go, Java ...) that have
 * no device allocator to wire into a callback.  For them `args->delta` is ignored; delta
 * lives in a fixed array inside the library image instead (AB200_STATIC_DELTA_FLOATS floats
 * = 4 MiB, resident on every GPU that loads the library until the process exits).
 *
 *   - Limit: the logsumexp/delta matrix of the call (batch * num_head_q * max_seqlen_q
 *     floats; for token-packed varlen num_head_q * q.size[2]) must fit in the array,
 *     otherwise the call returns hipErrorInvalidValue (1), prints one line naming the limit
 *     to stderr, and launches nothing.  For token-packed varlen q.size[2] must be the packed
 *     token count, i.e. at least cu_seqlens_q[batch] (seq_strides_q[batch] for strided
 *     varlen): the kernels index delta up to that count, which only the device knows, so a
 *     packed call with q.size[2] <= 0 is refused as well.
 *   - The first call on each device looks up the array's device address; make that call
 *     with the device current and before any stream capture begins.  Later calls only launch.
 *   - Nothing is allocated or freed here, by the CUDA runtime or any other library.
 *   - All calls share the one array.  Each call overwrites the part it uses before reading
 *     it, so leftovers of earlier calls are harmless, but two calls whose kernels overlap on
 *     the GPU (different streams, no dependency) race on it: serialise them.
 * Everything else (inputs, outputs, return codes, asynchrony) is as for ab200_attn_bwd.
 */
#define AB200_STATIC_DELTA_FLOATS (1u << 20)
AB200_API int ab200_attn_bwd_static_scratch(const ab200_attn_bwd_args* args, void* stream);

/* 1 when ab200_attn_bwd would use args->dq_acc if it were given (kernel family 3 selected, tcgen05
 * kernels apply, head dim above 64, no dBias requested, deterministic == 0), else 0; lets a caller acquire the accumulator
 * only when it is needed, as attn_bwd does with the reference's lazy tensor
 * (modules/flash/csrc/attn_bwd.cc:140-158). */
AB200_API int ab200_bwd_uses_dq_acc(const ab200_attn_bwd_args* args, void* stream);

/* The fused form's two stages after ab200_bwd_preprocess: dK, dV and dQ partials into args->dq_acc
 * (the reference's fused / AITER-style backward with a dq accumulator, include/aotriton/flash.h:170),
 * then dq = cast(sm_scale * dq_acc) (modules/flash/kernel/bwd_postprocess.py:14-84). */
AB200_API int ab200_bwd_fused(const ab200_attn_bwd_args* args, void* stream);
AB200_API int ab200_bwd_postprocess(const ab200_attn_bwd_args* args, void* stream);

/* The three backward stages one by one (modules/flash/kernel/bwd_preprocess.py:28-250,
 * bwd_kernel_dk_dv.py:48-417, bwd_kernel_dq.py:45-389). */
AB200_API int ab200_bwd_preprocess(const ab200_attn_bwd_args* args, void* stream);
AB200_API int ab200_bwd_dkdv(const ab200_attn_bwd_args* args, void* stream);
AB200_API int ab200_bwd_dq(const ab200_attn_bwd_args* args, void* stream);

/* Replaces aotriton::v2::flash::debug_simulate_encoded_softmax
 * (modules/flash/csrc/attn_debug.cc:31-69, kernel/dropout_rng.py:86-126):
 * r[b,h,m,n] = +0.5 where the Philox keep bit is set, -0.5 elsewhere. */
AB200_API int ab200_debug_simulate_encoded_softmax(const ab200_view4* r, int32_t dtype,
                                                   int32_t batch, int32_t num_head_q,
                                                   int32_t rows, int32_t cols, float dropout_p,
                                                   const uint64_t* philox_seed,
                                                   const uint64_t* philox_offset1,
                                                   uint64_t philox_offset2, void* stream);

/* Replaces aotriton::v2::flash::check_gpu (modules/flash/csrc/attn_check.cc:36-46):
 * 0 when the stream's device is an sm_100 part, hipErrorNoBinaryForGpu (209) otherwise. */
AB200_API int ab200_check_gpu(void* stream);

/* Replaces aotriton::getMultiProcessorCount (v3src/util.cc:77-112). */
AB200_API int ab200_multiprocessor_count(void* stream);

/* Selects the kernel family: 0 = automatic (tcgen05 kernels where they apply),
 * 1 = force the general SIMT kernels, 2 = require tcgen05 kernels (unsupported
 * shapes then return hipErrorNotSupported), 3 = like 0, and the backward takes its
 * fused form whenever a dQ accumulator is supplied and the problem qualifies.
 * Counterpart of attn_options::force_backend_index (include/aotriton/flash.h:38-40).
 * Per calling thread.  Returns the old value. */
AB200_API int ab200_set_kernel_family(int family);

/* The static selection table, the counterpart of the reference's tuning-database lookup
 * (v3src/flash/autotune.*: tables FLASH$op_attn_fwd / FLASH$op_attn_bwd keyed by dtype, head-dim
 * bin, bias, dropout, causal and sequence-length bins).  op: 0 forward, 1 backward; flags: OR of
 * the AB200_SELECT_* bits.  Returns variant | (head-dim instantiation << 8) with variant
 * 1 = general kernels, 2 = tcgen05 kernels, 3 = tcgen05 kernels with the fused backward, or the
 * negated error code (hipErrorNotSupported for a head dim beyond 512 or when tcgen05 kernels were
 * required but cannot take the problem).  Pure function: needs no device. */
enum {
  AB200_SELECT_ALIGNED = 1,          /* tensors are 16-byte aligned with unit inner stride        */
  AB200_SELECT_DBIAS = 2,            /* backward: dBias requested                                 */
  AB200_SELECT_FUSED_REQUESTED = 4,  /* backward: family 3, dq_acc given, deterministic == 0      */
  AB200_SELECT_FORCE_GENERAL = 8,    /* kernel family 1                                           */
  AB200_SELECT_FORCE_TCGEN05 = 16    /* kernel family 2                                           */
};
AB200_API int ab200_select_variant(int op, int dtype, int head_dim_qk, int head_dim_vo, int flags);

/* Which family the most recent forward / backward launch of this thread used
 * (1 = general, 2 = tcgen05, 3 = tcgen05 with the fused backward); diagnostics for tests and
 * benchmarks. */
AB200_API int ab200_last_fwd_family(void);
AB200_API int ab200_last_bwd_family(void);

/* Health word of the tcgen05 kernels on the current device: 0, or a code naming the
 * bounded wait that ran out (the kernels never spin forever; they give up after about a
 * second, record where, and exit).  Synchronises the device.  reset != 0 clears the word.
 * The reference has no counterpart: its kernels contain no waits. */
AB200_API unsigned int ab200_kernel_status(int reset);

/* Synchronises `stream` and reports its device's health: 0, a CUDA error number, or
 * hipErrorLaunchFailure (719) when a kernel gave up on a bounded wait (ab200_kernel_status
 * then names the wait).  The health word is sticky: after a failure every CTA of every later
 * tcgen05 launch on that device returns at once WITHOUT writing its outputs, and once this
 * function or ab200_kernel_status has seen the failure the entry points refuse further
 * launches on the device with 719, until ab200_kernel_status(1) clears the word.
 * The reference has no counterpart (its kernels cannot time out); launch errors there
 * surface through hipGetLastError (modules/flash/tests/attn_torch_function.py:192-200). */
AB200_API int ab200_stream_check(void* stream);

/* Test hook for the time-out path of the bounded waits; no counterpart in the reference.
 * For the calling thread's following launches: `wait_limit_kcycles` bounds every in-kernel
 * wait (units of 1024 SM cycles, 0 = the default of about a second) and `drop_copy` makes
 * the producer leave out one tile copy (1 = the forward's first V block, 2 = the dK/dV
 * kernel's first Q/dO block, 3 = the dQ kernel's first V block, 0 = none; for head dims above
 * 128: 2 = the first block's Q of the dV and dO of the dK kernel, 3 = its V), so that a wait
 * runs out, the kernel records which one and returns normally.  Nothing faults or hangs:
 * the kernel takes a few limits to drain.  Call with (0, 0) to restore normal operation. */
AB200_API void ab200_debug_bounded_wait_test(int drop_copy, unsigned int wait_limit_kcycles);

/* Test hooks for the host side of the launch path; no counterpart in the reference.  Every CUDA
 * call the library makes on that path goes through one table.  fake_device != 0 makes the table
 * pretend an sm_100 device (148 SMs): device queries answer, symbol look-ups, attribute settings
 * and kernel launches are counted and skipped, so the whole host logic runs on a machine without
 * a GPU.  fail_call >= 0 makes the (fail_after + 1)-th call of that entry return fail_code
 * instead of doing anything: 0 get-device, 1 set-device, 2 stream-device, 3 device-attribute,
 * 4 function-attribute, 5 symbol-address, 6 memset, 7 kernel launch, 8 tensor-map encoder,
 * 9 stream-synchronise.  Resets the per-entry call counters.  (0, -1, 0, 0) restores normal
 * operation.  Process-wide; meant for single-threaded tests.  Nothing here touches a device. */
AB200_API void ab200_debug_host_calls(int fake_device, int fail_call, int fail_code, int fail_after);
AB200_API uint64_t ab200_debug_host_call_count(int call);

/* Number of kernels launched by this library since load (all threads). */
AB200_API uint64_t ab200_launch_count(void);

/* Library version string, e.g. "aotriton_b200 0.1 (sm_100a)". */
AB200_API const char* ab200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* AOTRITON_B200_CABI_H */
