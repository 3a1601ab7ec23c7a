"""ctypes binding of the C-ABI declared in include/aotriton_b200.h.

This is the reference-side stub a maintainer of another host language would write: POD
structs, raw device pointers, integer return codes.  torch is used only to obtain device
pointers, strides and the current stream.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libaotriton_v2.so"

DTYPE_FP32, DTYPE_FP16, DTYPE_BF16 = 1, 2, 3
CAUSAL_NONE, CAUSAL_WINDOWED = 0, 3
WINDOW_TOP_LEFT, WINDOW_BOTTOM_RIGHT = -2147483647, -2147483646
VARLEN_NONE, VARLEN_COMPACT, VARLEN_PADDED, VARLEN_STRIDED = 0, 1, 2, 3
STATIC_DELTA_FLOATS = 1 << 20   # AB200_STATIC_DELTA_FLOATS
SELECT_ALIGNED, SELECT_DBIAS, SELECT_FUSED_REQUESTED, SELECT_FORCE_GENERAL, SELECT_FORCE_TCGEN05 = 1, 2, 4, 8, 16

# Exported symbols, in header order (checked by the CPU test-suite).
SYMBOLS = [
    "ab200_attn_fwd", "ab200_attn_bwd", "ab200_attn_bwd_static_scratch", "ab200_bwd_uses_dq_acc",
    "ab200_bwd_fused", "ab200_bwd_postprocess", "ab200_bwd_preprocess", "ab200_bwd_dkdv", "ab200_bwd_dq",
    "ab200_debug_simulate_encoded_softmax", "ab200_check_gpu", "ab200_multiprocessor_count",
    "ab200_set_kernel_family", "ab200_select_variant", "ab200_last_fwd_family", "ab200_last_bwd_family",
    "ab200_kernel_status", "ab200_stream_check", "ab200_debug_bounded_wait_test", "ab200_debug_host_calls",
    "ab200_debug_host_call_count", "ab200_launch_count", "ab200_version",
]


class View4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("size", C.c_int64 * 4), ("stride", C.c_int64 * 4)]


class Problem(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("num_head_q", C.c_int32), ("num_head_k", C.c_int32),
        ("max_seqlen_q", C.c_int32), ("max_seqlen_k", C.c_int32), ("head_dim_qk", C.c_int32),
        ("head_dim_vo", C.c_int32), ("sm_scale", C.c_float), ("causal_type", C.c_int32),
        ("window_left", C.c_int32), ("window_right", C.c_int32), ("varlen_type", C.c_int32),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("seq_strides_q", C.c_void_p), ("seq_strides_k", C.c_void_p),
        ("dropout_p", C.c_float), ("philox_seed", C.c_void_p), ("philox_offset1", C.c_void_p),
        ("philox_offset2", C.c_uint64), ("philox_head_offset", C.c_int32), ("philox_num_head_q", C.c_int32),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("prob", Problem), ("q", View4), ("k", View4), ("v", View4), ("bias", View4), ("out", View4),
        ("lse", C.c_void_p), ("philox_seed_output", C.c_void_p), ("philox_offset_output", C.c_void_p),
        ("encoded_softmax", View4), ("encoded_softmax_rows", C.c_int32), ("encoded_softmax_cols", C.c_int32),
        ("persistent_atomic_counter", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("prob", Problem), ("q", View4), ("k", View4), ("v", View4), ("bias", View4), ("out", View4),
        ("dout", View4), ("dq", View4), ("dk", View4), ("dv", View4), ("dbias", View4),
        ("lse", C.c_void_p), ("delta", C.c_void_p), ("deterministic", C.c_int32), ("dq_acc", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load libaotriton_v2.so from the package directory; raises if it is missing."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise OSError(f"{LIB_PATH} not built; run `python -m aotriton_b200.build`")
        L = C.CDLL(str(LIB_PATH))
        for name in ("ab200_attn_fwd",):
            getattr(L, name).argtypes = [C.POINTER(FwdArgs), C.c_void_p]
        for name in ("ab200_attn_bwd", "ab200_attn_bwd_static_scratch", "ab200_bwd_preprocess", "ab200_bwd_dkdv",
                     "ab200_bwd_dq", "ab200_bwd_uses_dq_acc", "ab200_bwd_fused", "ab200_bwd_postprocess"):
            getattr(L, name).argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        L.ab200_debug_simulate_encoded_softmax.argtypes = [
            C.POINTER(View4), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
            C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        L.ab200_check_gpu.argtypes = [C.c_void_p]
        L.ab200_multiprocessor_count.argtypes = [C.c_void_p]
        L.ab200_select_variant.argtypes = [C.c_int] * 5
        L.ab200_set_kernel_family.argtypes = [C.c_int]
        L.ab200_kernel_status.argtypes = [C.c_int]
        L.ab200_kernel_status.restype = C.c_uint
        L.ab200_stream_check.argtypes = [C.c_void_p]
        L.ab200_debug_bounded_wait_test.argtypes = [C.c_int, C.c_uint]
        L.ab200_debug_bounded_wait_test.restype = None
        L.ab200_debug_host_calls.argtypes = [C.c_int] * 4
        L.ab200_debug_host_calls.restype = None
        L.ab200_debug_host_call_count.argtypes = [C.c_int]
        L.ab200_debug_host_call_count.restype = C.c_uint64
        L.ab200_launch_count.restype = C.c_uint64
        L.ab200_version.restype = C.c_char_p
        _lib = L
    return _lib


def _torch_dtype_code(t) -> int:
    import torch
    return {torch.float32: DTYPE_FP32, torch.float16: DTYPE_FP16, torch.bfloat16: DTYPE_BF16}[t.dtype]


def view4(t) -> View4:
    v = View4()
    if t is None:
        v.ptr = None
        return v
    assert t.dim() == 4
    v.ptr = t.data_ptr()
    for i in range(4):
        v.size[i] = t.shape[i]
        v.stride[i] = t.stride(i)
    return v


def _ptr(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def current_stream_handle() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def make_problem(q, k, v, *, sm_scale, causal_type=0, window_left=0, window_right=0, dropout_p=0.0,
                 philox_seed=None, philox_offset1=None, philox_offset2=0, cu_seqlens_q=None, cu_seqlens_k=None,
                 max_seqlen_q=0, max_seqlen_k=0, seq_strides_q=None, seq_strides_k=None, varlen_type=0,
                 philox_head_offset=0, philox_num_head_q=0) -> Problem:
    p = Problem()
    p.dtype = _torch_dtype_code(q)
    p.batch = q.shape[0]
    p.num_head_q, p.num_head_k = q.shape[1], k.shape[1]
    p.max_seqlen_q, p.max_seqlen_k = q.shape[2], k.shape[2]
    p.head_dim_qk, p.head_dim_vo = q.shape[3], v.shape[3]
    if cu_seqlens_q is not None:
        p.batch = cu_seqlens_q.numel() - 1
        p.max_seqlen_q, p.max_seqlen_k = max_seqlen_q, max_seqlen_k
        p.cu_seqlens_q, p.cu_seqlens_k = _ptr(cu_seqlens_q), _ptr(cu_seqlens_k)
        p.seq_strides_q, p.seq_strides_k = _ptr(seq_strides_q), _ptr(seq_strides_k)
        p.varlen_type = varlen_type or VARLEN_COMPACT
    p.sm_scale = sm_scale
    p.causal_type, p.window_left, p.window_right = causal_type, window_left, window_right
    p.dropout_p = dropout_p
    p.philox_seed, p.philox_offset1 = _ptr(philox_seed), _ptr(philox_offset1)
    p.philox_offset2 = philox_offset2
    p.philox_head_offset, p.philox_num_head_q = philox_head_offset, philox_num_head_q
    return p


def attn_fwd(q, k, v, out, lse, *, bias=None, philox_seed_output=None, philox_offset_output=None,
             encoded_softmax=None, stream=None, **problem) -> int:
    a = FwdArgs()
    a.prob = make_problem(q, k, v, **problem)
    a.q, a.k, a.v, a.bias, a.out = view4(q), view4(k), view4(v), view4(bias), view4(out)
    a.lse = _ptr(lse)
    a.philox_seed_output, a.philox_offset_output = _ptr(philox_seed_output), _ptr(philox_offset_output)
    a.encoded_softmax = view4(encoded_softmax)
    if encoded_softmax is not None:
        a.encoded_softmax_rows, a.encoded_softmax_cols = encoded_softmax.shape[2], encoded_softmax.shape[3]
    return lib().ab200_attn_fwd(C.byref(a), stream if stream is not None else current_stream_handle())


def make_bwd_args(q, k, v, out, dout, dq, dk, dv, lse, delta, *, bias=None, dbias=None, dq_acc=None,
                  deterministic=False, **problem) -> BwdArgs:
    """dq_acc: optional zero-filled fp32 tensor with dq's logical shape (contiguous) for the fused form."""
    a = BwdArgs()
    a.dq_acc = _ptr(dq_acc)
    a.deterministic = 1 if deterministic else 0
    a.prob = make_problem(q, k, v, **problem)
    a.q, a.k, a.v, a.bias, a.out, a.dout = view4(q), view4(k), view4(v), view4(bias), view4(out), view4(dout)
    a.dq, a.dk, a.dv, a.dbias = view4(dq), view4(dk), view4(dv), view4(dbias)
    a.lse, a.delta = _ptr(lse), _ptr(delta)
    return a


def attn_bwd(q, k, v, out, dout, dq, dk, dv, lse, delta, *, stream=None, stage="all", **kw) -> int:
    a = make_bwd_args(q, k, v, out, dout, dq, dk, dv, lse, delta, **kw)
    fn = {"all": "ab200_attn_bwd", "preprocess": "ab200_bwd_preprocess", "dkdv": "ab200_bwd_dkdv",
          "dq": "ab200_bwd_dq", "static_scratch": "ab200_attn_bwd_static_scratch", "fused": "ab200_bwd_fused",
          "postprocess": "ab200_bwd_postprocess", "uses_dq_acc": "ab200_bwd_uses_dq_acc"}[stage]
    return getattr(lib(), fn)(C.byref(a), stream if stream is not None else current_stream_handle())


def debug_simulate_encoded_softmax(r, dropout_p, philox_seed, philox_offset1, philox_offset2, stream=None) -> int:
    v = view4(r)
    return lib().ab200_debug_simulate_encoded_softmax(
        C.byref(v), _torch_dtype_code(r), r.shape[0], r.shape[1], r.shape[2], r.shape[3], dropout_p,
        _ptr(philox_seed), _ptr(philox_offset1), philox_offset2,
        stream if stream is not None else current_stream_handle())
