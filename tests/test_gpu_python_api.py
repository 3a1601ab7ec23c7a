"""GPU: the Python surfaces above the C-ABI, each against the CPU oracle -- the autograd wrappers
(dense with bias + dBias + dropout, compact varlen), the torch.library custom operators behind an
F.scaled_dot_product_attention-shaped call, lazy delta / dQ-accumulator tensors that the backward
acquires through the allocator callback, and the four v2-named positional entry points.

Tolerances: atol = rtol = 2e-2 (bf16) / 1e-2 (fp16); LSE 1e-3.
"""
import numpy as np
import pytest
import torch

from oracle import attention as A
from _util import ATOL, LSE_ATOL, close, randn_inputs

pytestmark = pytest.mark.gpu
TL = A.TOP_LEFT


def _cmp(tag, got, want, tol):
    ok, err = close(got.float().cpu(), want.float().cpu(), tol)
    assert ok, f"{tag}: max err {err}"


def test_autograd_dense_bias_dropout():
    from aotriton_b200 import autograd
    dt, B, H, Sq, Sk, D, p = torch.float16, 2, 3, 130, 200, 64, 0.2
    q, k, v, do = randn_inputs((B, H, Sq, D), (B, H, Sk, D), (B, H, Sk, D), dt, seed=4)
    bias = torch.randn(B, H, Sq, Sk, generator=torch.Generator().manual_seed(5)).to(dt)
    keep = A.keep_masks(autograd.DEFAULT_PHILOX_SEED, autograd.DEFAULT_PHILOX_OFFSET_1 +
                        autograd.DEFAULT_PHILOX_OFFSET_2, B, H, Sq, Sk, p)
    ref = A.attention(q, k, v, sm_scale=D ** -0.5, bias=bias, keep=keep, dropout_p=p, dout=do)
    qd, kd, vd, bd = (t.cuda().requires_grad_() for t in (q, k, v, bias))
    out, lse = autograd.attention(qd, kd, vd, bd, causal=False, dropout_p=p, return_lse=True)
    out.backward(do.cuda())
    for n, got, want in (("out", out, ref.out), ("dq", qd.grad, ref.dq), ("dk", kd.grad, ref.dk),
                         ("dv", vd.grad, ref.dv), ("db", bd.grad, ref.db)):
        _cmp("autograd dense " + n, got, want, ATOL[dt])
    _cmp("autograd dense lse", lse.reshape(B, H, Sq), ref.lse, LSE_ATOL)
    assert autograd.last_bwd_family == 2


def test_autograd_compact_varlen_dropout():
    from aotriton_b200 import autograd
    dt, Hq, Hk, D, p = torch.bfloat16, 4, 2, 128, 0.1
    lens = [33, 128, 200, 1]
    cu = [0] + list(np.cumsum(lens))
    T = cu[-1]
    g = torch.Generator().manual_seed(6)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    base = autograd.DEFAULT_PHILOX_OFFSET_1 + autograd.DEFAULT_PHILOX_OFFSET_2
    ref = A.attention_varlen(q, k, v, cu, cu, sm_scale=D ** -0.5, causal_type=3, window_left=TL, window_right=TL,
                             dropout_p=p, seed=autograd.DEFAULT_PHILOX_SEED, offset_base=base, max_sq=max(lens),
                             max_sk=max(lens), dout=do)
    thd = lambda t: t.cuda().transpose(1, 2).contiguous().transpose(1, 2).requires_grad_()
    qd, kd, vd = thd(q), thd(k), thd(v)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    out, lse = autograd.varlen_attention(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), causal=True, dropout_p=p,
                                         return_lse=True)
    out.backward(do.cuda())
    for n, got, want in (("out", out, ref.out), ("dq", qd.grad, ref.dq), ("dk", kd.grad, ref.dk),
                         ("dv", vd.grad, ref.dv)):
        _cmp("autograd varlen " + n, got, want, ATOL[dt])
    _cmp("autograd varlen lse", lse, ref.lse, LSE_ATOL)
    assert autograd.last_bwd_family == 2


@pytest.mark.parametrize("deterministic", [False, True])
def test_custom_op_sdpa_signature(deterministic):
    """F.scaled_dot_product_attention-shaped call over torch.ops.aotriton_b200.*, GQA + causal."""
    from aotriton_b200 import autograd
    dt, B, Hq, Hk, S, D = torch.bfloat16, 2, 8, 2, 384, 128
    q, k, v, do = randn_inputs((B, Hq, S, D), (B, Hk, S, D), (B, Hk, S, D), dt, seed=8)
    ref = A.attention(q, k, v, sm_scale=D ** -0.5, mask=A.window_mask(S, S, 3, TL, TL), dout=do)
    qd, kd, vd = (t.cuda().requires_grad_() for t in (q, k, v))
    prev = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(deterministic)
    try:
        out = autograd.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=True)
        out.backward(do.cuda())
    finally:
        torch.use_deterministic_algorithms(prev)
    for n, got, want in (("out", out, ref.out), ("dq", qd.grad, ref.dq), ("dk", kd.grad, ref.dk),
                         ("dv", vd.grad, ref.dv)):
        _cmp(f"custom op (deterministic={deterministic}) " + n, got, want, ATOL[dt])
    torch.library.opcheck(torch.ops.aotriton_b200.attn_fwd.default,
                          (qd.detach(), kd.detach(), vd.detach(), None, D ** -0.5, 0.0, 3, TL, TL, 1, 2),
                          test_utils=("test_schema", "test_faketensor"))


def test_lazy_tensors_are_acquired_through_the_callback():
    """attn_bwd with non-eager delta (torch allocator and the module's own pool): same gradients as
    with an eager delta; a lazy tensor serves one call only."""
    from aotriton_b200 import flash
    from aotriton_b200.flash import hipError_t
    dt, B, H, S, D = torch.float16, 1, 2, 256, 64
    q, k, v, do = (t.cuda() for t in randn_inputs((B, H, S, D), (B, H, S, D), (B, H, S, D), dt, seed=10))
    sm = D ** -0.5
    o = torch.empty_like(q)
    L = torch.empty(B * H, S, dtype=torch.float32, device="cuda")
    null = torch.empty(0, dtype=torch.uint64, device="cuda")
    atomic = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert flash.attn_fwd(q, k, v, None, sm, L, o, 0.0, null, null, 0, null, null, None, True, atomic) == hipError_t.hipSuccess

    def bwd(delta, dq_acc=None):
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
        err = flash.attn_bwd(q, k, v, None, sm, o, do, dq, dk, dv, None, dq_acc, L, delta, 0.0, null, null, 0, True)
        torch.cuda.synchronize()
        return err, (dq, dk, dv)

    err, want = bwd(flash.eager_delta(torch.empty_like(L)))
    assert err == hipError_t.hipSuccess
    for make in (flash.lazy_delta, flash.pooled_lazy_delta):
        lazy = make(L)
        err, got = bwd(lazy, flash.lazy_dq_acc(want[0]))
        assert err == hipError_t.hipSuccess
        for g, w in zip(got, want):
            assert torch.equal(g, w)
        err, _ = bwd(lazy)             # already disposed by the first call
        assert err == hipError_t.hipErrorInvalidValue


def test_v2_named_entry_points():
    """aotriton::v2::flash::attn_fwd / attn_bwd / *_compact_varlen through pyaotriton, positional."""
    from aotriton_b200 import flash, load_pyaotriton
    from aotriton_b200.flash import hipError_t, mk_aotensor, T0, T1, T2, T4, DType, Stream
    v2 = load_pyaotriton().v2.flash
    dt, B, Hq, Hk, S, D = torch.float16, 2, 4, 2, 160, 64
    q, k, v, do = randn_inputs((B, Hq, S, D), (B, Hk, S, D), (B, Hk, S, D), dt, seed=12)
    sm = D ** -0.5
    ref = A.attention(q, k, v, sm_scale=sm, mask=A.window_mask(S, S, 3, TL, TL), dout=do)
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o = torch.full_like(qd, float("nan"))
    L = torch.empty(B * Hq, S, dtype=torch.float32, device="cuda")
    delta = torch.empty_like(L)
    stream = Stream(torch.cuda.current_stream().cuda_stream)
    n4 = T4(0, [0] * 4, [0] * 4, DType.kFloat16)
    n0 = T0(0, DType.kUInt64)
    err = v2.attn_fwd(mk_aotensor(qd), mk_aotensor(kd), mk_aotensor(vd), n4, sm, mk_aotensor(L), mk_aotensor(o), 0.0,
                      n0, n0, 0, n0, n0, n4, True, TL, TL, stream)
    assert err == hipError_t.hipSuccess
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
    err = v2.attn_bwd(mk_aotensor(qd), mk_aotensor(kd), mk_aotensor(vd), n4, sm, mk_aotensor(o), mk_aotensor(dod),
                      mk_aotensor(dq), mk_aotensor(dk), mk_aotensor(dv), n4, mk_aotensor(L), mk_aotensor(delta), 0.0,
                      n0, n0, 0, True, TL, TL, stream)
    assert err == hipError_t.hipSuccess
    torch.cuda.synchronize()
    for n, got, want in (("out", o, ref.out), ("dq", dq, ref.dq), ("dk", dk, ref.dk), ("dv", dv, ref.dv)):
        _cmp("v2 dense " + n, got, want, ATOL[dt])

    # compact varlen
    lens = [50, 129, 7]
    cu = [0] + list(np.cumsum(lens))
    T = cu[-1]
    g = torch.Generator().manual_seed(13)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    ref = A.attention_varlen(q, k, v, cu, cu, sm_scale=sm, causal_type=0, window_left=0, window_right=0,
                             dropout_p=0.0, seed=0, offset_base=0, max_sq=max(lens), max_sk=max(lens), dout=do)
    thd = lambda t: t.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    qd, kd, vd, dod = thd(q), thd(k), thd(v), thd(do)
    o = torch.full_like(qd, float("nan"))
    L = torch.empty(Hq, T, dtype=torch.float32, device="cuda")
    delta = torch.empty_like(L)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    err = v2.attn_fwd_compact_varlen(mk_aotensor(qd), mk_aotensor(kd), mk_aotensor(vd), n4, mk_aotensor(cu_t),
                                     mk_aotensor(cu_t), max(lens), max(lens), sm, mk_aotensor(L), mk_aotensor(o), 0.0,
                                     n0, n0, 0, n0, n0, n4, False, 0, 0, stream)
    assert err == hipError_t.hipSuccess
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
    err = v2.attn_bwd_compact_varlen(mk_aotensor(qd), mk_aotensor(kd), mk_aotensor(vd), mk_aotensor(cu_t),
                                     mk_aotensor(cu_t), max(lens), max(lens), n4, sm, mk_aotensor(o), mk_aotensor(dod),
                                     mk_aotensor(dq), mk_aotensor(dk), mk_aotensor(dv), n4, mk_aotensor(L),
                                     mk_aotensor(delta), 0.0, n0, n0, 0, False, 0, 0, stream)
    assert err == hipError_t.hipSuccess
    torch.cuda.synchronize()
    for n, got, want in (("out", o, ref.out), ("dq", dq, ref.dq), ("dk", dk, ref.dk), ("dv", dv, ref.dv)):
        _cmp("v2 varlen " + n, got, want, ATOL[dt])


def test_full_size_device_reference_agrees_with_the_oracle():
    """The full-size configuration tests compare against a dense fp32 evaluation on the device; this
    ties that evaluation to oracle.attention on a case small enough for the oracle (GQA group, causal
    mask, dropout, bias), so the full-size tests inherit the oracle's pin."""
    from test_gpu_full_configs import _dev_reference
    G, S, D, p = 2, 96, 32, 0.3
    g = torch.Generator().manual_seed(14)
    q, do = torch.randn(1, G, S, D, generator=g), torch.randn(1, G, S, D, generator=g)
    k, v = torch.randn(1, 1, S, D, generator=g), torch.randn(1, 1, S, D, generator=g)
    bias = torch.randn(1, G, S, S, generator=g)
    keep = A.keep_masks(3, 9, 1, G, S, S, p)
    ref = A.attention(q, k, v, sm_scale=0.2, bias=bias, keep=keep, dropout_p=p, dout=do)
    r = _dev_reference(q[0].cuda(), k[0, 0].cuda(), v[0, 0].cuda(), do[0].cuda(), sm=0.2, keep=keep[0].cuda(), p=p,
                       bias=bias[0].cuda())
    for n in ("out", "dq"):
        _cmp("device reference " + n, r[n], getattr(ref, n)[0], 1e-4)
    for n in ("dk", "dv"):
        _cmp("device reference " + n, r[n], getattr(ref, n)[0, 0], 1e-4)
    _cmp("device reference db", r["db"], ref.db[0], 1e-4)
    _cmp("device reference lse", r["lse"], ref.lse[0], 1e-5)
    mask = A.window_mask(S, S, 3, TL, TL)
    ref = A.attention(q, k, v, sm_scale=0.2, mask=mask, dout=do)
    r = _dev_reference(q[0].cuda(), k[0, 0].cuda(), v[0, 0].cuda(), do[0].cuda(), sm=0.2, mask=mask.cuda())
    for n in ("out", "dq"):
        _cmp("device reference causal " + n, r[n], getattr(ref, n)[0], 1e-4)
    _cmp("device reference causal dk", r["dk"], ref.dk[0, 0], 1e-4)
