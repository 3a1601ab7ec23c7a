"""fp32/fp64 restatement of the attention forward and backward.  TEST INFRASTRUCTURE ONLY.

Dense matrices, explicit formulas, no tiling -- the arithmetic contract of ROCm/aotriton's
kernels written the slow way:
  forward   modules/flash/kernel/fwd_kernel_inner.py:126-277, fwd_kernel.py:573-620
  window    modules/flash/kernel/masked_load_store.py:43-63
  backward  modules/flash/kernel/bwd_inner_dk_dv.py:117-256, bwd_inner_dq.py:117-205
  delta     modules/flash/kernel/bwd_preprocess.py:118-133
  LSE       modules/flash/tune/sdpa_math.py:16-41
and the test oracle the reference itself uses, torch's math SDPA
(modules/flash/tests/_common_test.py:61-79, 410-454), exposed as `sdpa_math_reference`.

Pinned by: the known-answer test of modules/flash/tests/_core_test_backward.py:333-351
(LSE = 2.79018449783325195 for identity inputs) and by outputs of the reference's own Triton
kernels executed with the Triton interpreter (tests/golden/*.npz, tests/golden/make_golden.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from . import philox

TOP_LEFT = -2147483647
BOTTOM_RIGHT = -2147483646


def parse_window(causal_type: int, window_left: int, window_right: int, seqlen_q: int, seqlen_k: int):
    """(window_left, window_right) in tokens, or None when no window applies."""
    if causal_type == 0:
        return None
    if causal_type == 1 or window_left == TOP_LEFT:
        wl = seqlen_q
    elif causal_type == 2 or window_left == BOTTOM_RIGHT:
        wl = seqlen_q
    else:
        wl = window_left
    if causal_type == 1 or window_right == TOP_LEFT:
        wr = 0
    elif causal_type == 2 or window_right == BOTTOM_RIGHT:
        wr = seqlen_k - seqlen_q
    else:
        wr = window_right
    return wl, wr


def window_mask(seqlen_q: int, seqlen_k: int, causal_type: int = 0, window_left: int = 0,
                window_right: int = 0) -> torch.Tensor:
    """Boolean [Sq, Sk]: True where the score takes part in the softmax."""
    w = parse_window(causal_type, window_left, window_right, seqlen_q, seqlen_k)
    if w is None:
        return torch.ones(seqlen_q, seqlen_k, dtype=torch.bool)
    wl, wr = w
    m = torch.arange(seqlen_q)[:, None]
    n = torch.arange(seqlen_k)[None, :]
    return (n <= m + wr) & (n >= m - wl)


@dataclass
class AttnResult:
    out: torch.Tensor
    lse: torch.Tensor
    dq: torch.Tensor | None = None
    dk: torch.Tensor | None = None
    dv: torch.Tensor | None = None
    db: torch.Tensor | None = None
    delta: torch.Tensor | None = None


def attention(q, k, v, *, sm_scale, bias=None, mask=None, keep=None, dropout_p=0.0, dout=None,
              acc_dtype=torch.float32, round_dtype=None) -> AttnResult:
    """One dense problem: q [B,Hq,Sq,D], k/v [B,Hk,Sk,D*], mask bool [Sq,Sk] (or broadcastable
    to [B,Hq,Sq,Sk]), keep bool [B,Hq,Sq,Sk] dropout keep mask.  Returns fp32/fp64 tensors.

    round_dtype: when given, P and dS are rounded through that dtype before the value
    matmuls, the way the kernels cast them to the input type.
    """
    B, Hq, Sq, _ = q.shape
    Hk, Sk = k.shape[1], k.shape[2]
    g = Hq // Hk
    qf, kf, vf = (t.to(acc_dtype) for t in (q, k, v))
    kf = kf.repeat_interleave(g, dim=1)
    vf = vf.repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sm_scale
    if bias is not None:
        s = s + bias.to(acc_dtype)
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    mx = s.amax(dim=-1, keepdim=True)
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)      # rows with no valid key
    e = torch.exp(s - mx)
    l = e.sum(dim=-1, keepdim=True)
    dead = l == 0
    p = torch.where(dead, torch.zeros_like(e), e / torch.where(dead, torch.ones_like(l), l))
    lse = torch.where(dead, torch.full_like(l, float("inf")), mx + torch.log(torch.where(dead, torch.ones_like(l), l)))
    scale = 1.0 / (1.0 - dropout_p) if dropout_p > 0 else 1.0
    pd = p
    if keep is not None and dropout_p > 0:
        pd = torch.where(keep, p * scale, torch.zeros_like(p))

    def rnd(x):
        return x.to(round_dtype).to(acc_dtype) if round_dtype is not None else x

    out = torch.matmul(rnd(pd), vf)
    res = AttnResult(out=out, lse=lse.squeeze(-1))
    if dout is None:
        return res
    do = dout.to(acc_dtype)
    # delta uses the output as stored (rounded to the io dtype) like the kernels do
    o_stored = out.to(q.dtype).to(acc_dtype)
    delta = (o_stored * do).sum(dim=-1, keepdim=True)
    dp = torch.matmul(do, vf.transpose(-1, -2))
    if keep is not None and dropout_p > 0:
        dp = torch.where(keep, dp * scale, torch.zeros_like(dp))
    ds = p * (dp - delta)
    dv_full = torch.matmul(rnd(pd).transpose(-1, -2), do)
    dk_full = torch.matmul(rnd(ds).transpose(-1, -2), qf) * sm_scale
    dq = torch.matmul(rnd(ds), kf) * sm_scale
    res.dq = dq
    res.dk = dk_full.reshape(B, Hk, g, Sk, -1).sum(dim=2)
    res.dv = dv_full.reshape(B, Hk, g, Sk, -1).sum(dim=2)
    res.db = ds
    res.delta = delta.squeeze(-1)
    return res


def sdpa_math_reference(q, k, v, *, sm_scale, bias=None, mask=None, keep=None, dropout_p=0.0, dout=None,
                        acc_dtype=torch.float32):
    """The reference's own test oracle: aten math SDPA + autograd (_common_test.py:61-79, 436-454).
    mask/bias are merged into one additive attn_mask, as the reference does for windows."""
    B, Hq, Sq, _ = q.shape
    Sk = k.shape[2]
    qf, kf, vf = (t.detach().to(acc_dtype).requires_grad_(dout is not None) for t in (q, k, v))
    attn = None
    bf = None
    if bias is not None:
        bf = bias.detach().to(acc_dtype).requires_grad_(dout is not None)
        attn = bf
    if mask is not None:
        add = torch.zeros(Sq, Sk, dtype=acc_dtype).masked_fill(~mask, float("-inf"))
        attn = add if attn is None else attn + add
    dm = keep if (keep is not None and dropout_p > 0) else None
    out, _ = torch.ops.aten._scaled_dot_product_attention_math(
        qf, kf, vf, attn_mask=attn, dropout_p=dropout_p if dm is not None else 0.0, is_causal=False,
        dropout_mask=dm, scale=sm_scale, enable_gqa=(q.shape[1] != k.shape[1]))
    if dout is None:
        return AttnResult(out=out.detach(), lse=None)
    out.backward(dout.to(acc_dtype))
    return AttnResult(out=out.detach(), lse=None, dq=qf.grad, dk=kf.grad, dv=vf.grad,
                      db=bf.grad if bf is not None else None)


def keep_masks(seed, offset_base, batch, num_head_q, max_sq, max_sk, dropout_p, seqlens=None,
               head_offset=0, num_head_total=None) -> torch.Tensor:
    """Keep mask [batch, Hq, max_sq, max_sk] (dense) from the Philox oracle."""
    ht = num_head_total or num_head_q
    out = np.zeros((batch, num_head_q, max_sq, max_sk), dtype=bool)
    for z in range(batch):
        for h in range(num_head_q):
            out[z, h] = philox.keep_mask(seed, offset_base, z, h + head_offset, ht, max_sq, max_sk,
                                         max_sq, max_sk, dropout_p)
    return torch.from_numpy(out)


def attention_varlen(q, k, v, cu_q, cu_k, *, sm_scale, causal_type=0, window_left=0, window_right=0,
                     dropout_p=0.0, seed=0, offset_base=0, max_sq=None, max_sk=None, dout=None,
                     acc_dtype=torch.float32, round_dtype=None, fn=attention):
    """Compact varlen: q [1,Hq,Tq,D], k/v [1,Hk,Tk,D]; cu_* python lists.  Returns AttnResult with
    packed tensors; lse/delta shaped [Hq, Tq] (the (H, total) layout of fwd_kernel_inner.py:30-43)."""
    Hq = q.shape[1]
    n = len(cu_q) - 1
    lens_q = [cu_q[i + 1] - cu_q[i] for i in range(n)]
    lens_k = [cu_k[i + 1] - cu_k[i] for i in range(n)]
    max_sq = max_sq or max(lens_q)
    max_sk = max_sk or max(lens_k)
    out = torch.zeros(q.shape[:3] + (v.shape[3],), dtype=acc_dtype)
    lse = torch.zeros(Hq, q.shape[2], dtype=acc_dtype)
    grads = dout is not None
    dq = torch.zeros(q.shape, dtype=acc_dtype) if grads else None
    dk = torch.zeros(k.shape, dtype=acc_dtype) if grads else None
    dv = torch.zeros(v.shape, dtype=acc_dtype) if grads else None
    delta = torch.zeros_like(lse) if grads else None
    for z in range(n):
        a, b = cu_q[z], cu_q[z + 1]
        c, d = cu_k[z], cu_k[z + 1]
        if b == a:
            continue
        mask = window_mask(b - a, d - c, causal_type, window_left, window_right)
        keep = None
        if dropout_p > 0:
            km = np.stack([philox.keep_mask(seed, offset_base, z, h, Hq, max_sq, max_sk, b - a, d - c, dropout_p)
                           for h in range(Hq)])
            keep = torch.from_numpy(km)[None]
        r = fn(q[:, :, a:b], k[:, :, c:d], v[:, :, c:d], sm_scale=sm_scale, mask=mask, keep=keep,
               dropout_p=dropout_p, dout=None if dout is None else dout[:, :, a:b], acc_dtype=acc_dtype,
               **({"round_dtype": round_dtype} if fn is attention else {}))
        out[:, :, a:b] = r.out
        if r.lse is not None:
            lse[:, a:b] = r.lse[0]
        if grads:
            dq[:, :, a:b] = r.dq
            dk[:, :, c:d] = r.dk
            dv[:, :, c:d] = r.dv
            if r.delta is not None:
                delta[:, a:b] = r.delta[0]
    return AttnResult(out=out, lse=lse, dq=dq, dk=dk, dv=dv, delta=delta)
