"""Python-side operator calls over the `pyaotriton` bindings.

Same functions, argument order and behaviour as the helper module the reference's tests use
(ROCm/aotriton modules/flash/tests/aotriton_flash.py:141-408): each builds TensorViews from torch
tensors, fills `attn_fwd_params` / `attn_bwd_params` and returns the operator's `hipError_t`.
Launches go to torch's current CUDA stream.
"""
from __future__ import annotations

import torch

from . import load_pyaotriton

_p = load_pyaotriton()
T0, T1, T2, T4, DType, Stream, hipError_t = _p.T0, _p.T1, _p.T2, _p.T4, _p.DType, _p.Stream, _p.hipError_t
hipGetLastError = _p.hipGetLastError
attn_options = _p.v3.flash.attn_options
_fwd, _fwd_params = _p.v3.flash.attn_fwd, _p.v3.flash.attn_fwd_params
_bwd, _bwd_params = _p.v3.flash.attn_bwd, _p.v3.flash.attn_bwd_params
_debug_mask = _p.v2.flash.debug_simulate_encoded_softmax


class CausalType:
    NONE = 0
    TOP_LEFT = 1
    BOTTOM_RIGHT = 2
    WINDOWED = 3


class WindowValue:
    NONE = 0
    TOP_LEFT_ALIGNED = -2147483647
    BOTTOM_RIGHT_ALIGNED = -2147483646


IVARLEN_TYPE = {"compact": 1, "padded": 2, "strided": 3}


def translate_causal(causal):
    """bool | (window_left, window_right) | CausalType constant -> (causal_type, left, right)."""
    if isinstance(causal, tuple):
        return CausalType.WINDOWED, int(causal[0]), int(causal[1])
    if isinstance(causal, bool):
        if causal:
            return CausalType.WINDOWED, WindowValue.TOP_LEFT_ALIGNED, WindowValue.TOP_LEFT_ALIGNED
        return CausalType.NONE, 0, 0
    if causal == CausalType.TOP_LEFT:
        return CausalType.WINDOWED, WindowValue.TOP_LEFT_ALIGNED, WindowValue.TOP_LEFT_ALIGNED
    if causal == CausalType.BOTTOM_RIGHT:
        return CausalType.WINDOWED, WindowValue.BOTTOM_RIGHT_ALIGNED, WindowValue.BOTTOM_RIGHT_ALIGNED
    assert causal == CausalType.NONE
    return CausalType.NONE, 0, 0


def cast_dtype(dtype):
    bits = dtype.itemsize * 8
    if dtype.is_floating_point:
        main = "BFloat" if dtype == torch.bfloat16 else "Float"
    else:
        main = "UInt" if "uint" in str(dtype) else "Int"
    return getattr(DType, f"k{main}{bits}")


def mk_aotensor(t, if_empty_then_like=None):
    """torch tensor -> TensorView of matching rank; None -> null view shaped like the other tensor;
    a 0- or 1-element rank-1 tensor -> T0 (device scalar)."""
    if t is None:
        like = if_empty_then_like
        rank = like.dim()
        klass = {1: T1, 2: T2, 4: T4}[rank]
        return klass(0, [0] * rank, [0] * rank, cast_dtype(like.dtype))
    if t.dim() == 1 and t.numel() in (0, 1):
        return T0(t.data_ptr(), cast_dtype(t.dtype))
    klass = {1: T1, 2: T2, 4: T4}[t.dim()]
    assert t.stride(-1) == 1, "the last stride of every tensor must be 1"
    return klass(t.data_ptr(), tuple(t.size()), tuple(t.stride()), cast_dtype(t.dtype))


def _stream():
    return Stream(torch.cuda.current_stream().cuda_stream)


def _fill_fwd(params, q, k, v, b, sm_scale, M, o, dropout_p, philox_seed, philox_offset1, philox_offset2,
              philox_seed_output, philox_offset_output, encoded_softmax, causal, atomic):
    params.Q, params.K, params.V = mk_aotensor(q), mk_aotensor(k), mk_aotensor(v)
    params.B = mk_aotensor(b, if_empty_then_like=q)
    params.Sm_scale = float(sm_scale)
    params.L = mk_aotensor(M, if_empty_then_like=torch.empty(0, 0, dtype=torch.float32))
    params.Out = mk_aotensor(o)
    params.dropout_p = float(dropout_p)
    params.philox_seed_ptr = mk_aotensor(philox_seed)
    params.philox_offset1 = mk_aotensor(philox_offset1)
    params.philox_offset2 = philox_offset2
    params.philox_seed_output = mk_aotensor(philox_seed_output)
    params.philox_offset_output = mk_aotensor(philox_offset_output)
    params.encoded_softmax = mk_aotensor(encoded_softmax, if_empty_then_like=q)
    params.persistent_atomic_counter = mk_aotensor(atomic)
    params.causal_type, params.window_left, params.window_right = translate_causal(causal)


def attn_fwd(q, k, v, b, sm_scale, M, o, dropout_p, philox_seed, philox_offset1, philox_offset2,
             philox_seed_output, philox_offset_output, encoded_softmax, causal, atomic, extargs=None):
    params = _fwd_params()
    _fill_fwd(params, q, k, v, b, sm_scale, M, o, dropout_p, philox_seed, philox_offset1, philox_offset2,
              philox_seed_output, philox_offset_output, encoded_softmax, causal, atomic)
    params.varlen_type = 0
    return _fwd(params, _fwd_params.kVersion, _stream(), extargs if extargs is not None else attn_options())


def attn_fwd_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, seq_strides_q,
                    seq_strides_k, b, sm_scale, M, o, dropout_p, philox_seed, philox_offset1, philox_offset2,
                    philox_seed_output, philox_offset_output, encoded_softmax, causal, atomic, varlen_type,
                    extargs=None):
    params = _fwd_params()
    _fill_fwd(params, q, k, v, b, sm_scale, M, o, dropout_p, philox_seed, philox_offset1, philox_offset2,
              philox_seed_output, philox_offset_output, encoded_softmax, causal, atomic)
    params.cu_seqlens_q, params.cu_seqlens_k = mk_aotensor(cu_seqlens_q), mk_aotensor(cu_seqlens_k)
    params.Max_seqlen_q, params.Max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    params.seq_strides_q = mk_aotensor(seq_strides_q, if_empty_then_like=cu_seqlens_q)
    params.seq_strides_k = mk_aotensor(seq_strides_k, if_empty_then_like=cu_seqlens_k)
    params.varlen_type = IVARLEN_TYPE[varlen_type]
    return _fwd(params, _fwd_params.kVersion, _stream(), extargs if extargs is not None else attn_options())


def _fill_bwd(params, q, k, v, b, sm_scale, o, dout, dq, dk, dv, db, dq_acc, L, delta, dropout_p, philox_seed,
              philox_offset1, philox_offset2, causal):
    params.Q, params.K, params.V = mk_aotensor(q), mk_aotensor(k), mk_aotensor(v)
    params.B = mk_aotensor(b, if_empty_then_like=q)
    params.Sm_scale = float(sm_scale)
    params.Out, params.DO = mk_aotensor(o), mk_aotensor(dout)
    params.DK, params.DV, params.DQ = mk_aotensor(dk), mk_aotensor(dv), mk_aotensor(dq)
    params.DB = mk_aotensor(db, if_empty_then_like=q)
    params.L = mk_aotensor(L)
    params.D = delta
    if dq_acc is not None:
        params.DQ_ACC = dq_acc
    params.dropout_p = float(dropout_p)
    params.philox_seed_ptr = mk_aotensor(philox_seed)
    params.philox_offset1 = mk_aotensor(philox_offset1)
    params.philox_offset2 = philox_offset2
    params.causal_type, params.window_left, params.window_right = translate_causal(causal)


def attn_bwd(q, k, v, b, sm_scale, o, dout, dq, dk, dv, db, dq_acc, L, delta, dropout_p, philox_seed,
             philox_offset1, philox_offset2, causal, extargs=None):
    params = _bwd_params()
    _fill_bwd(params, q, k, v, b, sm_scale, o, dout, dq, dk, dv, db, dq_acc, L, delta, dropout_p, philox_seed,
              philox_offset1, philox_offset2, causal)
    params.varlen_type = 0
    return _bwd(params, _bwd_params.kVersion, _stream(), extargs if extargs is not None else attn_options())


def attn_bwd_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, seq_strides_q,
                    seq_strides_k, b, sm_scale, o, dout, dq, dk, dv, db, dq_acc, L, delta, dropout_p,
                    philox_seed, philox_offset1, philox_offset2, causal, varlen_type, extargs=None):
    params = _bwd_params()
    _fill_bwd(params, q, k, v, b, sm_scale, o, dout, dq, dk, dv, db, dq_acc, L, delta, dropout_p, philox_seed,
              philox_offset1, philox_offset2, causal)
    params.cu_seqlens_q, params.cu_seqlens_k = mk_aotensor(cu_seqlens_q), mk_aotensor(cu_seqlens_k)
    params.Max_seqlen_q, params.Max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    params.seq_strides_q = mk_aotensor(seq_strides_q, if_empty_then_like=cu_seqlens_q)
    params.seq_strides_k = mk_aotensor(seq_strides_k, if_empty_then_like=cu_seqlens_k)
    params.varlen_type = IVARLEN_TYPE[varlen_type]
    return _bwd(params, _bwd_params.kVersion, _stream(), extargs if extargs is not None else attn_options())


def debug_simulate_encoded_softmax(R, dropout_p, philox_seed, philox_offset1, philox_offset2):
    return _debug_mask(mk_aotensor(R), dropout_p, mk_aotensor(philox_seed), mk_aotensor(philox_offset1),
                       philox_offset2, _stream())


def lazy_dq_acc(dq: torch.Tensor):
    """fp32 zero-initialised dQ accumulator shaped like dq, allocated by torch only if the backward
    asks for it (reference: bindings/lazy_tensor/lazy_tensor_template.h:19-58, at::zeros)."""
    like = T4(dq.data_ptr(), tuple(dq.size()), tuple(dq.stride()), cast_dtype(dq.dtype))
    return _p.lazy_tensor.dq_acc_from(like, lambda: torch.zeros(dq.shape, dtype=torch.float32, device=dq.device))


def lazy_delta(L: torch.Tensor):
    """fp32 delta scratch shaped like the logsumexp tensor, allocated by torch when the backward
    acquires it (reference: lazy_tensor_template.h:60-97, at::empty)."""
    like = T2(L.data_ptr(), tuple(L.size()), tuple(L.stride()), cast_dtype(L.dtype))
    return _p.lazy_tensor.delta_from(like, lambda: torch.empty(L.shape, dtype=torch.float32, device=L.device))


def pooled_lazy_delta(L: torch.Tensor):
    """The same from the module's own cudaMalloc pool (no torch allocator involved), bound to the
    current stream."""
    like = T2(L.data_ptr(), tuple(L.size()), tuple(L.stride()), cast_dtype(L.dtype))
    return _p.lazy_tensor.delta(like, L.device.index, torch.cuda.current_stream().cuda_stream)


def pooled_lazy_dq_acc(dq: torch.Tensor):
    like = T4(dq.data_ptr(), tuple(dq.size()), tuple(dq.stride()), cast_dtype(dq.dtype))
    return _p.lazy_tensor.dq_acc(like, dq.device.index, torch.cuda.current_stream().cuda_stream)


def check_stream():
    """Synchronise the current stream and raise if a kernel of this library gave up on a bounded
    wait (its outputs are then incomplete).  The condition is sticky until reset_kernel_status()."""
    err = _p.stream_check(_stream())
    if err != hipError_t.hipSuccess:
        raise RuntimeError(f"aotriton_b200: stream check failed: {err} (kernel status {_p.kernel_status(False):#x})")


def reset_kernel_status():
    return _p.kernel_status(True)


def eager_delta(delta: torch.Tensor):
    """Wrap a caller-owned fp32 tensor shaped like L as the backward's delta scratch."""
    return _p.lazy_tensor.eager_delta(
        T2(delta.data_ptr(), tuple(delta.size()), tuple(delta.stride()), cast_dtype(delta.dtype)))
