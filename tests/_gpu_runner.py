"""Drive the library through its C-ABI from CPU-resident test inputs (GPU tests only)."""
from __future__ import annotations

import torch

from aotriton_b200 import cabi

# "fused": automatic choice with the fused backward requested and a dQ accumulator supplied, so that the backward takes the fused
# (atomic-dQ) form where it applies
FAMILY = {"auto": 0, "general": 1, "sm100": 2, "fused": 3}


def dev(t):
    return None if t is None else t.cuda()


def run_fwd_bwd(q, k, v, do=None, *, sm_scale, bias=None, causal_type=0, window_left=0, window_right=0,
                dropout_p=0.0, seed=None, offset1=None, offset2=0, cu_q=None, cu_k=None, max_sq=0, max_sk=0,
                family="auto", want_dbias=False, lse_null=False, varlen_type=0, seq_strides_q=None,
                seq_strides_k=None, keep_layout=None):
    """Inputs are CPU tensors in logical (B,H,S,D) order (any strides).  Returns a dict of CPU tensors:
    out, lse, and with `do` also dq, dk, dv, delta (and db).  Raises on a non-zero return code."""
    old = cabi.lib().ab200_set_kernel_family(FAMILY[family])
    try:
        qd, kd, vd, bd, dod = dev(q), dev(k), dev(v), dev(bias), dev(do)
        if keep_layout is not None:      # re-create a permuted storage on the device
            qd, kd, vd, dod = (keep_layout(t) if t is not None else None for t in (qd, kd, vd, dod))
        B, Hq, Sq, _ = q.shape
        Dv = v.shape[3]
        out = torch.full((B, Hq, Sq, Dv), float("nan"), dtype=q.dtype, device="cuda")
        if keep_layout is not None:
            out = keep_layout(out)
        prob = dict(sm_scale=sm_scale, causal_type=causal_type, window_left=window_left, window_right=window_right,
                    dropout_p=dropout_p, philox_offset2=offset2)
        seed_t = off_t = None
        if dropout_p > 0:
            seed_t = torch.tensor([seed], dtype=torch.uint64, device="cuda")
            off_t = torch.tensor([offset1], dtype=torch.uint64, device="cuda")
            prob.update(philox_seed=seed_t, philox_offset1=off_t)
        if cu_q is not None:
            cuq = torch.tensor(cu_q, dtype=torch.int32, device="cuda")
            cuk = torch.tensor(cu_k, dtype=torch.int32, device="cuda")
            prob.update(cu_seqlens_q=cuq, cu_seqlens_k=cuk, max_seqlen_q=max_sq, max_seqlen_k=max_sk,
                        varlen_type=varlen_type)
            if seq_strides_q is not None:
                prob.update(seq_strides_q=torch.tensor(seq_strides_q, dtype=torch.int32, device="cuda"),
                            seq_strides_k=torch.tensor(seq_strides_k, dtype=torch.int32, device="cuda"))
            if varlen_type == cabi.VARLEN_PADDED:
                lse_shape = (len(cu_q) - 1) * Hq, max_sq
            else:
                total = seq_strides_q[-1] if seq_strides_q is not None else cu_q[-1]
                lse_shape = (Hq, total)
        else:
            lse_shape = (B * Hq, Sq)
        lse = None if lse_null else torch.full(lse_shape, float("nan"), dtype=torch.float32, device="cuda")
        seed_out = torch.zeros(1, dtype=torch.uint64, device="cuda") if dropout_p > 0 else None
        off_out = torch.zeros(1, dtype=torch.uint64, device="cuda") if dropout_p > 0 else None
        err = cabi.attn_fwd(qd, kd, vd, out, lse, bias=bd, philox_seed_output=seed_out,
                            philox_offset_output=off_out, **prob)
        if err != 0:
            raise RuntimeError(f"ab200_attn_fwd returned {err}")
        res = {"out": out.cpu(), "lse": None if lse is None else lse.cpu(),
               "fwd_family": cabi.lib().ab200_last_fwd_family()}
        if dropout_p > 0:
            res["seed_out"], res["off_out"] = int(seed_out.cpu().item()), int(off_out.cpu().item())
        if do is not None:
            dq = torch.full_like(qd, float("nan")); dk = torch.full_like(kd, float("nan"))
            dv = torch.full_like(vd, float("nan"))
            db = torch.full_like(bd, float("nan")) if (want_dbias and bd is not None) else None
            delta = torch.full(lse_shape, float("nan"), dtype=torch.float32, device="cuda")
            bprob = dict(prob)
            if family == "fused":      # zero-filled fp32, contiguous in dq's logical (B, H, S, D) order
                bprob["dq_acc"] = torch.zeros(tuple(qd.shape), dtype=torch.float32, device="cuda")
            if dropout_p > 0:   # the backward consumes what the forward reported (offset2 already folded in)
                bprob.update(philox_seed=seed_out, philox_offset1=off_out, philox_offset2=0)
            err = cabi.attn_bwd(qd, kd, vd, out, dod, dq, dk, dv, lse, delta, bias=bd, dbias=db, **bprob)
            if err != 0:
                raise RuntimeError(f"ab200_attn_bwd returned {err}")
            res.update(dq=dq.cpu(), dk=dk.cpu(), dv=dv.cpu(), delta=delta.cpu(),
                       bwd_family=cabi.lib().ab200_last_bwd_family())
            if db is not None:
                res["db"] = db.cpu()
        torch.cuda.synchronize()
        return res
    finally:
        cabi.lib().ab200_set_kernel_family(old)
