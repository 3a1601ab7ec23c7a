"""CPU: the host side of the launch path on a pretended sm_100 device (no GPU involved).

The library routes every CUDA call of that path through one table.  With the table in its
pretend-a-device mode the whole host logic runs here: argument checks, the choice of kernel variant,
how many kernels each operator call launches, and -- with a failure injected into any one of the
calls -- that the injected code comes back to the caller, nothing is launched after it, and lazy
tensors are still released.  Nothing in this file touches a device or makes one fault.
"""
import ctypes as C

import pytest

from aotriton_b200 import cabi

CALLS = dict(get_device=0, set_device=1, stream_device=2, device_attr=3, func_attr=4, symbol=5, memset=6, launch=7,
             encode=8, sync=9)


@pytest.fixture
def fake():
    L = cabi.lib()
    L.ab200_debug_host_calls(1, -1, 0, 0)
    try:
        yield L
    finally:
        L.ab200_debug_host_calls(0, -1, 0, 0)
        L.ab200_set_kernel_family(0)


def _view(ptr, shape, strides=None):
    v = cabi.View4()
    v.ptr = ptr
    st = strides or [shape[1] * shape[2] * shape[3], shape[2] * shape[3], shape[3], 1]
    for i in range(4):
        v.size[i], v.stride[i] = shape[i], st[i]
    return v


def _problem(dtype=cabi.DTYPE_BF16, B=2, Hq=4, Hk=2, S=256, D=128):
    p = cabi.Problem()
    p.dtype, p.batch, p.num_head_q, p.num_head_k = dtype, B, Hq, Hk
    p.max_seqlen_q = p.max_seqlen_k = S
    p.head_dim_qk = p.head_dim_vo = D
    p.sm_scale = D ** -0.5
    return p


def _fwd_args(**kw):
    a = cabi.FwdArgs()
    a.prob = _problem(**kw)
    pr = a.prob
    a.q = _view(0x10000000, (pr.batch, pr.num_head_q, pr.max_seqlen_q, pr.head_dim_qk))
    a.k = _view(0x20000000, (pr.batch, pr.num_head_k, pr.max_seqlen_k, pr.head_dim_qk))
    a.v = _view(0x30000000, (pr.batch, pr.num_head_k, pr.max_seqlen_k, pr.head_dim_vo))
    a.out = _view(0x40000000, (pr.batch, pr.num_head_q, pr.max_seqlen_q, pr.head_dim_vo))
    a.lse = 0x50000000
    return a


def _bwd_args(**kw):
    a = cabi.BwdArgs()
    a.prob = _problem(**kw)
    pr = a.prob
    qs = (pr.batch, pr.num_head_q, pr.max_seqlen_q, pr.head_dim_qk)
    ks = (pr.batch, pr.num_head_k, pr.max_seqlen_k, pr.head_dim_qk)
    a.q, a.out, a.dout, a.dq = (_view(0x10000000 + i * 0x1000000, qs) for i in range(4))
    a.k, a.v, a.dk, a.dv = (_view(0x20000000 + i * 0x1000000, ks) for i in range(4))
    a.lse, a.delta = 0x50000000, 0x51000000
    return a


def test_launch_counts_and_variants(fake):
    L = fake
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_fwd(C.byref(_fwd_args()), None) == 0
    assert L.ab200_launch_count() - n0 == 1 and L.ab200_last_fwd_family() == 2
    assert L.ab200_debug_host_call_count(CALLS["encode"]) == 3          # Q, K, V tile maps
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_bwd(C.byref(_bwd_args()), None) == 0
    assert L.ab200_launch_count() - n0 == 3 and L.ab200_last_bwd_family() == 2      # preprocess, dK/dV, dQ
    # fp32 and odd head dims go to the general kernels; forcing tcgen05 on them is refused before any launch
    assert L.ab200_attn_fwd(C.byref(_fwd_args(dtype=cabi.DTYPE_FP32, D=64)), None) == 0 and L.ab200_last_fwd_family() == 1
    L.ab200_set_kernel_family(2)
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_fwd(C.byref(_fwd_args(D=44)), None) == 801
    assert L.ab200_launch_count() == n0
    # fused backward: only on request (family 3), with an accumulator, not for deterministic calls
    a = _bwd_args()
    a.dq_acc = 0x60000000
    L.ab200_set_kernel_family(0)
    assert L.ab200_bwd_uses_dq_acc(C.byref(a), None) == 0
    L.ab200_set_kernel_family(3)
    assert L.ab200_bwd_uses_dq_acc(C.byref(a), None) == 1
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_bwd(C.byref(a), None) == 0
    assert L.ab200_launch_count() - n0 == 3 and L.ab200_last_bwd_family() == 3      # preprocess, fused, conversion
    a.deterministic = 1
    assert L.ab200_bwd_uses_dq_acc(C.byref(a), None) == 0
    assert L.ab200_attn_bwd(C.byref(a), None) == 0 and L.ab200_last_bwd_family() == 2


def test_wide_heads_launch_one_kernel_per_gradient(fake):
    """Head dims above 128: forward on its 256-wide instantiation, backward as preprocess + dV + dK + dQ;
    no fused form; a launch failure in the middle stops the call there."""
    L = fake
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_fwd(C.byref(_fwd_args(D=256)), None) == 0
    assert L.ab200_launch_count() - n0 == 1 and L.ab200_last_fwd_family() == 2
    n0, e0 = L.ab200_launch_count(), L.ab200_debug_host_call_count(CALLS["encode"])
    assert L.ab200_attn_bwd(C.byref(_bwd_args(D=192)), None) == 0
    assert L.ab200_launch_count() - n0 == 4 and L.ab200_last_bwd_family() == 2
    assert L.ab200_debug_host_call_count(CALLS["encode"]) - e0 == 8     # four tile maps for dV + dK, four for dQ
    a = _bwd_args(D=256)
    a.dq_acc = 0x60000000
    L.ab200_set_kernel_family(3)
    assert L.ab200_bwd_uses_dq_acc(C.byref(a), None) == 0
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_bwd(C.byref(a), None) == 0
    assert L.ab200_launch_count() - n0 == 4 and L.ab200_last_bwd_family() == 2
    L.ab200_set_kernel_family(0)
    L.ab200_debug_host_calls(1, CALLS["launch"], 719, 2)      # the third launch (dK) fails
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_bwd(C.byref(_bwd_args(D=256)), None) == 719
    assert L.ab200_launch_count() - n0 == 2


@pytest.mark.parametrize("call,code", [("func_attr", 1), ("symbol", 13), ("encode", 1), ("launch", 719),
                                       ("device_attr", 101)])
def test_injected_failures_come_back_and_stop_the_call(fake, call, code):
    L = fake
    L.ab200_debug_host_calls(1, CALLS[call], code, 0)
    n0 = L.ab200_launch_count()
    err = L.ab200_attn_fwd(C.byref(_fwd_args()), None)
    assert err != 0 and L.ab200_launch_count() == n0
    if call in ("func_attr", "symbol", "launch"):
        assert err == code
    elif call == "device_attr":
        assert err == 209          # the device cannot be identified: hipErrorNoBinaryForGpu
    # the backward stops at the failing stage: with the second launch failing, exactly one kernel ran
    L.ab200_debug_host_calls(1, CALLS["launch"], 719, 1)
    n0 = L.ab200_launch_count()
    assert L.ab200_attn_bwd(C.byref(_bwd_args()), None) == 719
    assert L.ab200_launch_count() - n0 == 1


def test_operator_api_releases_lazy_tensors_when_a_launch_fails(fake):
    """attn_bwd of the C++ API must free D and DQ_ACC whatever happens (attn_bwd.cc:157-158)."""
    from aotriton_b200 import load_pyaotriton
    p = load_pyaotriton()
    T4, T2, DType = p.T4, p.T2, p.DType
    shape, strides = [2, 4, 256, 128], [4 * 256 * 128, 256 * 128, 128, 1]
    kshape, kstrides = [2, 2, 256, 128], [2 * 256 * 128, 256 * 128, 128, 1]
    mk = lambda ptr, sh, st: T4(ptr, sh, st, DType.kBFloat16)
    params = p.v3.flash.attn_bwd_params()
    params.Q, params.Out, params.DO, params.DQ = (mk(0x10000000 + i * 0x1000000, shape, strides) for i in range(4))
    params.K, params.V, params.DK, params.DV = (mk(0x20000000 + i * 0x1000000, kshape, kstrides) for i in range(4))
    params.Sm_scale = 0.1
    params.dropout_p = 0.0
    params.causal_type, params.varlen_type, params.window_left, params.window_right = 0, 0, 0, 0
    L2 = T2(0x50000000, [8, 256], [256, 1], DType.kFloat32)
    params.L = L2
    events = []

    class FakeTensor:
        def __init__(self, name):
            self.name = name
            events.append(("made", name))

        def data_ptr(self):
            return 0x70000000

        def __del__(self):
            events.append(("freed", self.name))

    params.D = p.lazy_tensor.delta_from(L2, lambda: FakeTensor("delta"))
    params.DQ_ACC = p.lazy_tensor.dq_acc_from(params.DQ, lambda: FakeTensor("dq_acc"))
    opts = p.v3.flash.attn_options()
    opts.force_backend_index = 2                      # fused backward: both lazy tensors are acquired
    fake.ab200_debug_host_calls(1, CALLS["launch"], 719, 1)
    err = p.v3.flash.attn_bwd(params, p.v3.flash.attn_bwd_params.kVersion, p.Stream(), opts)
    assert err == p.hipError_t.hipErrorLaunchFailure
    import gc
    gc.collect()
    assert ("made", "delta") in events and ("made", "dq_acc") in events
    assert ("freed", "delta") in events and ("freed", "dq_acc") in events
    # wrong struct version: refused before anything is acquired
    events.clear()
    params.D = p.lazy_tensor.delta_from(L2, lambda: FakeTensor("delta2"))
    assert p.v3.flash.attn_bwd(params, 1, p.Stream(), opts) == p.hipError_t.hipErrorInvalidSymbol
    assert ("made", "delta2") not in events


def test_selection_table():
    L = cabi.lib()
    sel = lambda *a: L.ab200_select_variant(*a)
    A, DB, FU, FG, FT = (cabi.SELECT_ALIGNED, cabi.SELECT_DBIAS, cabi.SELECT_FUSED_REQUESTED, cabi.SELECT_FORCE_GENERAL,
                         cabi.SELECT_FORCE_TCGEN05)
    unpack = lambda r: (r & 0xff, r >> 8)
    assert unpack(sel(0, cabi.DTYPE_BF16, 128, 128, A)) == (2, 128)
    assert unpack(sel(0, cabi.DTYPE_FP16, 72, 72, A)) == (2, 128)
    assert unpack(sel(0, cabi.DTYPE_FP16, 40, 64, A)) == (2, 64)
    assert unpack(sel(0, cabi.DTYPE_FP16, 256, 256, A)) == (2, 256)
    assert unpack(sel(1, cabi.DTYPE_FP16, 256, 256, A)) == (2, 256)
    assert unpack(sel(1, cabi.DTYPE_FP16, 256, 256, A | FU)) == (2, 256)     # the fused form is 128-wide only
    assert unpack(sel(1, cabi.DTYPE_FP16, 264, 264, A)) == (1, 0)
    assert unpack(sel(0, cabi.DTYPE_FP32, 64, 64, A)) == (1, 0)
    assert unpack(sel(0, cabi.DTYPE_BF16, 128, 128, 0)) == (1, 0)            # unaligned tensors
    assert unpack(sel(0, cabi.DTYPE_BF16, 100, 100, A)) == (1, 0)            # head dim not a multiple of 8
    assert unpack(sel(0, cabi.DTYPE_BF16, 128, 128, A | FG)) == (1, 0)
    assert sel(0, cabi.DTYPE_FP32, 64, 64, A | FT) == -801
    assert sel(0, cabi.DTYPE_BF16, 520, 520, A) == -801                      # beyond the largest head dim
    assert unpack(sel(1, cabi.DTYPE_BF16, 128, 128, A | FU)) == (3, 128)
    assert unpack(sel(1, cabi.DTYPE_BF16, 128, 128, A | FU | DB)) == (2, 128)
    assert unpack(sel(1, cabi.DTYPE_BF16, 64, 64, A | FU)) == (2, 64)
    assert sel(2, cabi.DTYPE_BF16, 64, 64, A) == -1 and sel(0, 7, 64, 64, A) == -801
