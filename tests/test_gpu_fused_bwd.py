"""GPU: the fused backward (dK, dV and atomically accumulated dQ in one kernel, then a conversion
kernel) against the two-kernel backward and the oracle, at sizes with several key blocks per
sequence, GQA groups, windows, ragged ends, dropout and every varlen flavour; the deterministic
option; and run-to-run determinism of the two-kernel form.

Tolerances: atol = rtol = 2e-2 (bf16) / 1e-2 (fp16) against the oracle; the two forms against each
other within the same tolerance (their dQ sums differ in order and in where they round)."""
import numpy as np
import pytest
import torch

from oracle import attention as A
from _util import ATOL, close, randn_inputs

pytestmark = pytest.mark.gpu
TL, BR = A.TOP_LEFT, A.BOTTOM_RIGHT


def _bwd(q, k, v, out, do, lse, *, fused, deterministic=False, **prob):
    from aotriton_b200 import cabi
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
    delta = torch.empty_like(lse)
    acc = torch.zeros(tuple(q.shape), dtype=torch.float32, device="cuda") if fused else None
    old = cabi.lib().ab200_set_kernel_family(3 if fused else 2)      # 3: fused backward where it applies
    try:
        err = cabi.attn_bwd(q, k, v, out, do, dq, dk, dv, lse, delta, dq_acc=acc, deterministic=deterministic, **prob)
    finally:
        cabi.lib().ab200_set_kernel_family(old)
    assert err == 0, err
    torch.cuda.synchronize()
    return dq, dk, dv, cabi.lib().ab200_last_bwd_family()


CASES = [
    # dtype, B, Hq, Hk, Sq, Sk, D, causal(type, wl, wr), dropout
    (torch.bfloat16, 2, 4, 4, 512, 512, 128, (3, TL, TL), 0.0),
    (torch.bfloat16, 1, 8, 2, 700, 700, 128, (3, 200, 0), 0.0),
    (torch.float16, 1, 4, 1, 333, 461, 128, (3, BR, BR), 0.0),
    (torch.float16, 2, 2, 2, 257, 129, 128, (0, 0, 0), 0.25),
    (torch.float16, 1, 2, 2, 300, 300, 72, (0, 0, 0), 0.0),
    (torch.bfloat16, 1, 2, 1, 130, 390, 96, (3, TL, TL), 0.1),
    (torch.bfloat16, 1, 1, 1, 1, 1, 128, (3, TL, TL), 0.0),
    (torch.bfloat16, 1, 2, 2, 300, 100, 128, (3, BR, BR), 0.0),      # a tile of dead rows beside a live one
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{str(c[0])[6:]}-B{c[1]}H{c[2]}:{c[3]}-S{c[4]}x{c[5]}-D{c[6]}-c{c[7][0]}-p{c[8]}")
def test_fused_backward_dense(case):
    from aotriton_b200 import cabi
    dt, B, Hq, Hk, Sq, Sk, D, (ct, wl, wr), p = case
    q, k, v, do = randn_inputs((B, Hq, Sq, D), (B, Hk, Sk, D), (B, Hk, Sk, D), dt, seed=Sq + Sk + D)
    sm = D ** -0.5
    seed, off = 99, 7
    keep = A.keep_masks(seed, off, B, Hq, Sq, Sk, p) if p > 0 else None
    ref = A.attention(q, k, v, sm_scale=sm, mask=A.window_mask(Sq, Sk, ct, wl, wr), keep=keep, dropout_p=p, dout=do)
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    prob = dict(sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr)
    if p > 0:
        prob.update(dropout_p=p, philox_seed=torch.tensor([seed], dtype=torch.uint64, device="cuda"),
                    philox_offset1=torch.tensor([off], dtype=torch.uint64, device="cuda"))
    out = torch.empty_like(qd)
    lse = torch.empty(B * Hq, Sq, dtype=torch.float32, device="cuda")
    assert cabi.attn_fwd(qd, kd, vd, out, lse, **prob) == 0
    split = _bwd(qd, kd, vd, out, dod, lse, fused=False, **prob)
    fused = _bwd(qd, kd, vd, out, dod, lse, fused=True, **prob)
    assert split[3] == 2 and fused[3] == 3, (split[3], fused[3])
    for n, s_, f_, want in zip(("dq", "dk", "dv"), split, fused, (ref.dq, ref.dk, ref.dv)):
        ok, err = close(f_.float().cpu(), want, ATOL[dt])
        assert ok, f"fused {n} vs oracle: {err}"
        ok, err = close(f_.float().cpu(), s_.float().cpu(), ATOL[dt])
        assert ok, f"fused {n} vs two-kernel form: {err}"
    # deterministic calls keep the two-kernel form even when an accumulator is offered
    det = _bwd(qd, kd, vd, out, dod, lse, fused=True, deterministic=True, **prob)
    assert det[3] == 2
    for s_, d_ in zip(split[:3], det[:3]):
        assert torch.equal(s_, d_), "the two-kernel form is not reproducible run to run"
    assert cabi.lib().ab200_kernel_status(0) == 0


@pytest.mark.parametrize("varlen", ["compact", "padded", "strided"])
def test_fused_backward_varlen(varlen):
    from aotriton_b200 import cabi
    dt, Hq, Hk, D, p = torch.float16, 4, 2, 128, 0.1
    lens = [70, 300, 1, 129, 256]
    cu_l = [0] + list(np.cumsum(lens))
    smax = max(lens)
    g = torch.Generator().manual_seed(3)
    seed_t = torch.tensor([5], dtype=torch.uint64, device="cuda")
    off_t = torch.tensor([11], dtype=torch.uint64, device="cuda")
    cu = torch.tensor(cu_l, dtype=torch.int32, device="cuda")
    prob = dict(sm_scale=D ** -0.5, causal_type=3, window_left=TL, window_right=TL, dropout_p=p, philox_seed=seed_t,
                philox_offset1=off_t, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=smax, max_seqlen_k=smax)
    if varlen == "padded":
        n = len(lens)
        q, k, v, do = (t.cuda() for t in randn_inputs((n, Hq, smax, D), (n, Hk, smax, D), (n, Hk, smax, D), dt, seed=2))
        prob["varlen_type"] = cabi.VARLEN_PADDED
        lse_shape = (n * Hq, smax)
        span = lambda z: (z, slice(0, lens[z]))
    else:
        starts = cu_l if varlen == "compact" else [0, 80, 400, 416, 560, 830]
        T = starts[-1]
        mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).cuda().transpose(1, 2)
        q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
        if varlen == "strided":
            ss = torch.tensor(starts, dtype=torch.int32, device="cuda")
            prob.update(varlen_type=cabi.VARLEN_STRIDED, seq_strides_q=ss, seq_strides_k=ss)
        lse_shape = (Hq, T)
        span = lambda z: (0, slice(starts[z], starts[z] + lens[z]))
    out = torch.empty_like(q)
    lse = torch.empty(lse_shape, dtype=torch.float32, device="cuda")
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
    split = _bwd(q, k, v, out, do, lse, fused=False, **prob)
    fused = _bwd(q, k, v, out, do, lse, fused=True, **prob)
    assert split[3] == 2 and fused[3] == 3
    for z in range(len(lens)):
        b, sl = span(z)
        for n_, s_, f_ in zip(("dq", "dk", "dv"), split, fused):
            a_, b_ = f_[b:b + 1, :, sl].float().cpu(), s_[b:b + 1, :, sl].float().cpu()
            assert not torch.isnan(a_).any(), f"{varlen} z={z} {n_}: NaN"
            ok, err = close(a_, b_, ATOL[dt])
            assert ok, f"{varlen} z={z} {n_}: fused differs from the two-kernel form by {err}"
    assert cabi.lib().ab200_kernel_status(0) == 0


def test_fused_backward_through_the_operator_api():
    """attn_bwd of the C++ API acquires DQ_ACC from the caller's allocator only when it will use it."""
    from aotriton_b200 import flash, cabi
    from aotriton_b200.flash import hipError_t
    dt, B, H, S, D = torch.bfloat16, 1, 2, 384, 128
    q, k, v, do = (t.cuda() for t in randn_inputs((B, H, S, D), (B, H, S, D), (B, H, S, D), dt, seed=10))
    sm = D ** -0.5
    o = torch.empty_like(q)
    L = torch.empty(B * H, S, dtype=torch.float32, device="cuda")
    null = torch.empty(0, dtype=torch.uint64, device="cuda")
    atomic = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert flash.attn_fwd(q, k, v, None, sm, L, o, 0.0, null, null, 0, null, null, None, True, atomic) == hipError_t.hipSuccess
    made = []

    def run(deterministic):
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
        opts = flash.attn_options()
        opts.deterministic = deterministic
        opts.force_backend_index = 2          # fused backward where it applies
        like = flash.T4(dq.data_ptr(), tuple(dq.size()), tuple(dq.stride()), flash.cast_dtype(dq.dtype))

        def factory():
            made.append(deterministic)
            return torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
        acc = flash._p.lazy_tensor.dq_acc_from(like, factory)
        err = flash.attn_bwd(q, k, v, None, sm, o, do, dq, dk, dv, None, acc, L, flash.lazy_delta(L), 0.0, null, null,
                             0, True, opts)
        assert err == hipError_t.hipSuccess
        torch.cuda.synchronize()
        return dq, dk, dv

    fused = run(False)
    assert made == [False], "the accumulator was not acquired for the fused form"
    det = run(True)
    assert made == [False], "a deterministic call must not acquire the accumulator"
    for f_, d_ in zip(fused, det):
        ok, err = close(f_.float().cpu(), d_.float().cpu(), ATOL[dt])
        assert ok, err
    assert cabi.lib().ab200_kernel_status(0) == 0
