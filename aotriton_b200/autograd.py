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


# ---------------------------------------------------------------------------------------------
# torch.library custom operators: the form in which a framework's SDPA dispatcher would register
# this library (the reference is wired into PyTorch the same way on ROCm, README.md:71-75; its own
# tests wrap the operator in autograd.Function, tests/attn_torch_function.py:87-270).  The ops are
# opaque to tracing (fake implementations give shapes and dtypes) and carry an autograd formula,
# so torch.compile and torch.export keep them as single nodes.
def _lse_rows(q):
    return q.shape[0] * q.shape[1], q.shape[2]


@torch.library.custom_op("aotriton_b200::attn_fwd", mutates_args=())
def op_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor | None, sm_scale: float,
                dropout_p: float, causal_type: int, window_left: int, window_right: int, philox_seed: int,
                philox_offset1: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (out, logsumexp, philox seed used, philox offset used)."""
    o = torch.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[3]), device=q.device, dtype=q.dtype)
    M = torch.empty(_lse_rows(q), device=q.device, dtype=torch.float32)
    seed, off1, off2, seed_out, off_out = _philox_tensors(q.device, dropout_p, philox_seed, philox_offset1)
    causal = (window_left, window_right) if causal_type == flash.CausalType.WINDOWED else False
    atomic = torch.zeros([1], device=q.device, dtype=torch.int32)
    _check(flash.attn_fwd(q, k, v, bias, sm_scale, M, o, dropout_p, seed, off1, off2, seed_out, off_out, None,
                          causal, atomic), "attn_fwd")
    if dropout_p <= 0.0:
        seed_out = torch.zeros([1], device=q.device, dtype=torch.uint64)
        off_out = torch.zeros([1], device=q.device, dtype=torch.uint64)
    return o, M, seed_out, off_out


@op_attn_fwd.register_fake
def _(q, k, v, bias, sm_scale, dropout_p, causal_type, window_left, window_right, philox_seed, philox_offset1):
    o = q.new_empty((q.shape[0], q.shape[1], q.shape[2], v.shape[3]))
    M = q.new_empty(_lse_rows(q), dtype=torch.float32)
    s = q.new_empty([1], dtype=torch.uint64)
    return o, M, s, q.new_empty([1], dtype=torch.uint64)


@torch.library.custom_op("aotriton_b200::attn_bwd", mutates_args=())
def op_attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
                dout: torch.Tensor, lse: torch.Tensor, philox_seed: torch.Tensor, philox_offset: torch.Tensor,
                sm_scale: float, dropout_p: float, causal_type: int, window_left: int, window_right: int,
                deterministic: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (dq, dk, dv, dbias); dbias is an empty tensor when there is no bias."""
    dout = dout if dout.stride(-1) == 1 else dout.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    db = torch.empty_like(bias) if bias is not None else None
    causal = (window_left, window_right) if causal_type == flash.CausalType.WINDOWED else False
    null = torch.empty([0], device=q.device, dtype=torch.uint64)
    opts = flash.attn_options()
    opts.deterministic = bool(deterministic)
    _check(flash.attn_bwd(q, k, v, bias, sm_scale, out, dout, dq, dk, dv, db, flash.lazy_dq_acc(dq), lse,
                          flash.lazy_delta(lse), dropout_p, philox_seed if dropout_p > 0 else null,
                          philox_offset if dropout_p > 0 else null, 0, causal, opts), "attn_bwd")
    _note_bwd_family()
    return dq, dk, dv, db if db is not None else q.new_empty([0])


@op_attn_bwd.register_fake
def _(q, k, v, bias, out, dout, lse, philox_seed, philox_offset, sm_scale, dropout_p, causal_type, window_left,
      window_right, deterministic):
    return (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
            torch.empty_like(bias) if bias is not None else q.new_empty([0]))


def _op_setup_context(ctx, inputs, output):
    q, k, v, bias, sm_scale, dropout_p, causal_type, wl, wr, _, _ = inputs
    out, lse, seed_out, off_out = output
    ctx.save_for_backward(q, k, v, bias, out, lse, seed_out, off_out)
    ctx.args = (sm_scale, dropout_p, causal_type, wl, wr)


def _op_backward(ctx, dout, dlse, dseed, doff):
    q, k, v, bias, out, lse, seed_out, off_out = ctx.saved_tensors
    sm_scale, dropout_p, causal_type, wl, wr = ctx.args
    dq, dk, dv, db = op_attn_bwd(q, k, v, bias, out, dout, lse, seed_out, off_out, sm_scale, dropout_p, causal_type,
                                 wl, wr, torch.are_deterministic_algorithms_enabled())
    return dq, dk, dv, (db if bias is not None else None), None, None, None, None, None, None, None


op_attn_fwd.register_autograd(_op_backward, setup_context=_op_setup_context)


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None,
                                 enable_gqa=False, philox_seed=DEFAULT_PHILOX_SEED,
                                 philox_offset1=DEFAULT_PHILOX_OFFSET_1):
    """torch.nn.functional.scaled_dot_product_attention's signature over the custom operators.
    attn_mask must be a floating-point additive bias broadcastable to (B, Hq, Sq, Sk) or None (the
    operator has no boolean-mask input; the reference's kernels take an additive bias only, and only
    without causal masking, aot/_common.py:24-27)."""
    if attn_mask is not None:
        if attn_mask.dtype == torch.bool:
            raise ValueError("boolean attn_mask is not supported; pass an additive floating-point bias")
        if is_causal:
            raise ValueError("attn_mask together with is_causal is not supported by the operator")
        attn_mask = attn_mask.to(query.dtype).expand(query.shape[0], query.shape[1], query.shape[2], key.shape[2])
        if attn_mask.stride(-1) != 1:
            attn_mask = attn_mask.contiguous()
    if not enable_gqa and query.shape[1] != key.shape[1]:
        raise ValueError("query and key head counts differ; pass enable_gqa=True")
    scale = query.shape[-1] ** -0.5 if scale is None else scale
    ct, wl, wr = flash.translate_causal(bool(is_causal))
    return op_attn_fwd(query, key, value, attn_mask, float(scale), float(dropout_p), ct, wl, wr, philox_seed,
                       philox_offset1)[0]
