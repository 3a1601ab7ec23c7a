"""torch.autograd wrappers over the operator: what a framework's SDPA integration calls.

Follows the reference's test-side wrappers (ROCm/aotriton modules/flash/tests/
attn_torch_function.py:87-270 and varlen_attn_torch_function.py:38-206): the forward allocates O
and the fp32 logsumexp, owns the Philox seed/offset scalars when dropout is on and hands the
values it actually used to the backward; the backward allocates dQ/dK/dV(/dB) and a delta scratch.
"""
from __future__ import annotations

import torch

from . import flash
from .flash import hipError_t

DEFAULT_PHILOX_SEED = 0x1BF52
DEFAULT_PHILOX_OFFSET_1 = 0x1D4000
DEFAULT_PHILOX_OFFSET_2 = 0x000B42


def _check(err, what):
    if err != hipError_t.hipSuccess:
        raise RuntimeError(f"{what} failed: {err}")


def _philox_tensors(device, dropout_p, seed, offset1):
    null = torch.empty([0], device=device, dtype=torch.uint64)
    if dropout_p <= 0.0:
        return null, null, 0, null, null
    mk = lambda v: torch.tensor([v], device=device, dtype=torch.uint64)
    return mk(seed), mk(offset1), DEFAULT_PHILOX_OFFSET_2, mk(0), mk(0)


# Kernel family of the most recent backward (the library keeps it per thread, and autograd runs
# backward on a thread of its own): 1 = general, 2 = tcgen05, 0 = none yet.
last_bwd_family = 0


def _note_bwd_family():
    global last_bwd_family
    from . import cabi
    last_bwd_family = int(cabi.lib().ab200_last_bwd_family())


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, b, causal, sm_scale, dropout_p, return_lse=False,
                philox_seed=DEFAULT_PHILOX_SEED, philox_offset1=DEFAULT_PHILOX_OFFSET_1):
        o = torch.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[3]), device=q.device, dtype=q.dtype)
        M = torch.empty((q.shape[0] * q.shape[1], q.shape[2]), device=q.device, dtype=torch.float32)
        seed, off1, off2, seed_out, off_out = _philox_tensors(q.device, dropout_p, philox_seed, philox_offset1)
        atomic = torch.zeros([1], device=q.device, dtype=torch.int32) if causal else \
            torch.empty([0], device=q.device, dtype=torch.int32)
        _check(flash.attn_fwd(q, k, v, b, sm_scale, M, o, dropout_p, seed, off1, off2, seed_out, off_out,
                              None, causal, atomic), "attn_fwd")
        ctx.save_for_backward(q, k, v, b, o, M)
        ctx.sm_scale, ctx.causal, ctx.dropout_p = sm_scale, causal, dropout_p
        ctx.philox_seed, ctx.philox_offset = seed_out, off_out
        return (o, M) if return_lse else o

    @staticmethod
    def backward(ctx, do, *unused):
        q, k, v, b, o, L = ctx.saved_tensors
        do = do if do.stride(-1) == 1 else do.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        db = torch.empty_like(b) if b is not None else None
        delta = torch.empty_like(L)
        _check(flash.attn_bwd(q, k, v, b, ctx.sm_scale, o, do, dq, dk, dv, db, None, L, flash.eager_delta(delta),
                              ctx.dropout_p, ctx.philox_seed, ctx.philox_offset, 0, ctx.causal), "attn_bwd")
        _note_bwd_family()
        return dq, dk, dv, db, None, None, None, None, None, None


def attention(q, k, v, b=None, causal=False, sm_scale=None, dropout_p=0.0, return_lse=False,
              philox_seed=DEFAULT_PHILOX_SEED, philox_offset1=DEFAULT_PHILOX_OFFSET_1):
    """O = dropout(softmax(Q K^T * sm_scale + b, mask)) V for (B, H, S, D) tensors (any strides with
    unit innermost stride).  `causal` is a bool, a (left, right) window or a flash.CausalType."""
    sm_scale = q.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    return _Attention.apply(q, k, v, b, causal, sm_scale, dropout_p, return_lse, philox_seed, philox_offset1)


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, sm_scale,
                dropout_p, return_lse=False, philox_seed=DEFAULT_PHILOX_SEED,
                philox_offset1=DEFAULT_PHILOX_OFFSET_1):
        # q, k, v: (1, H, total_tokens, D) views of THD storage
        o = torch.empty((1, q.shape[2], q.shape[1], v.shape[3]), device=q.device, dtype=q.dtype).transpose(1, 2)
        M = torch.empty((q.shape[1], q.shape[2]), device=q.device, dtype=torch.float32)
        seed, off1, off2, seed_out, off_out = _philox_tensors(q.device, dropout_p, philox_seed, philox_offset1)
        atomic = torch.empty([0], device=q.device, dtype=torch.int32)
        _check(flash.attn_fwd_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, None, None,
                                     None, sm_scale, M, o, dropout_p, seed, off1, off2, seed_out, off_out, None,
                                     causal, atomic, "compact"), "attn_fwd (varlen)")
        ctx.save_for_backward(q, k, v, o, M, cu_seqlens_q, cu_seqlens_k)
        ctx.max_seqlens = (max_seqlen_q, max_seqlen_k)
        ctx.sm_scale, ctx.causal, ctx.dropout_p = sm_scale, causal, dropout_p
        ctx.philox_seed, ctx.philox_offset = seed_out, off_out
        return (o, M) if return_lse else o

    @staticmethod
    def backward(ctx, do, *unused):
        q, k, v, o, L, cu_q, cu_k = ctx.saved_tensors
        do = do if do.stride(-1) == 1 else do.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty_like(L)
        _check(flash.attn_bwd_varlen(q, k, v, cu_q, cu_k, ctx.max_seqlens[0], ctx.max_seqlens[1], None, None, None,
                                     ctx.sm_scale, o, do, dq, dk, dv, None, None, L, flash.eager_delta(delta),
                                     ctx.dropout_p, ctx.philox_seed, ctx.philox_offset, 0, ctx.causal,
                                     "compact"), "attn_bwd (varlen)")
        _note_bwd_family()
        return (dq, dk, dv) + (None,) * 10


def varlen_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=False,
                     sm_scale=None, dropout_p=0.0, return_lse=False):
    sm_scale = q.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    return _VarlenAttention.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal,
                                  sm_scale, dropout_p, return_lse)
