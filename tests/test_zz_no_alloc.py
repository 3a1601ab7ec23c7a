"""GPU: the backward entry point that brings its own delta scratch.

Some hosts cannot give the backward a delta buffer: runtimes that committed all device memory to a
fixed plan before the first step, and foreign-language callers that have no device allocator to
put behind the LazyTensor callback.  `ab200_attn_bwd_static_scratch` serves them from an array
inside the library.  This test calls it through the C-ABI twice in a row (the array is shared by
all calls, so the second call starts from the first call's leftovers) and checks dQ, dK, dV against
the ordinary entry point on the same inputs, and that an oversized problem is refused.

Collected last on purpose (file name), so that a run stopping at the first failure has already
run every other test; it must also pass alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

from _util import ATOL, close, randn_inputs

pytestmark = pytest.mark.gpu


def _backward(stage, q, k, v, out, do, lse, delta, **prob):
    from aotriton_b200 import cabi
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
    err = cabi.attn_bwd(q, k, v, out, do, dq, dk, dv, lse, delta, stage=stage, **prob)
    assert err == 0, f"{stage}: error {err}"
    torch.cuda.synchronize()
    return dq, dk, dv


@pytest.mark.parametrize("dt,B,Hq,Hk,S,D,causal", [
    (torch.bfloat16, 2, 4, 2, 384, 128, True),      # tcgen05 kernels
    (torch.float32, 1, 2, 2, 100, 40, False),       # general kernels
])
def test_static_scratch_matches_caller_scratch_twice(dt, B, Hq, Hk, S, D, causal):
    from aotriton_b200 import cabi
    q, k, v, do = (t.cuda() for t in randn_inputs((B, Hq, S, D), (B, Hk, S, D), (B, Hk, S, D), dt, seed=17))
    prob = dict(sm_scale=D ** -0.5)
    if causal:
        prob.update(causal_type=3, window_left=cabi.WINDOW_TOP_LEFT, window_right=cabi.WINDOW_TOP_LEFT)
    out = torch.empty_like(q)
    lse = torch.empty(B * Hq, S, dtype=torch.float32, device="cuda")
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
    delta = torch.empty_like(lse)
    want = _backward("all", q, k, v, out, do, lse, delta, **prob)
    for call in range(2):
        # delta=None: the entry point must not need a caller buffer at all
        got = _backward("static_scratch", q, k, v, out, do, lse, None, **prob)
        for name, g, w in zip(("dq", "dk", "dv"), got, want):
            ok, err = close(g.float().cpu(), w.float().cpu(), ATOL[dt])
            assert ok, f"call {call}: {name} differs from ab200_attn_bwd by {err}"
    assert cabi.lib().ab200_kernel_status(0) == 0


def test_static_scratch_compact_varlen_and_no_allocation():
    """Token-packed varlen (delta laid out as heads x packed tokens), and proof that the entry point
    takes no device memory: free memory reported by the driver is the same before and after."""
    import numpy as np
    from aotriton_b200 import cabi
    dt, Hq, Hk, D = torch.float16, 4, 2, 64
    lens = [100, 37, 260]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
    T = int(sum(lens))
    g = torch.Generator().manual_seed(23)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).cuda().transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    prob = dict(sm_scale=D ** -0.5, causal_type=3, window_left=cabi.WINDOW_TOP_LEFT, window_right=cabi.WINDOW_TOP_LEFT,
                cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    out = torch.empty_like(q)
    lse = torch.empty(Hq, T, dtype=torch.float32, device="cuda")
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
    want = _backward("all", q, k, v, out, do, lse, torch.empty_like(lse), **prob)
    # Outputs and their snapshots are allocated up front, so that nothing inside the measured window
    # goes through torch's allocator either.
    outs = [torch.empty_like(t) for t in (q, k, v)]
    snaps = [[torch.empty_like(t) for t in (q, k, v)] for _ in range(2)]
    assert cabi.attn_bwd(q, k, v, out, do, *outs, lse, None, stage="static_scratch", **prob) == 0   # symbol look-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for call in range(2):
        for t in outs:
            t.fill_(float("nan"))
        assert cabi.attn_bwd(q, k, v, out, do, *outs, lse, None, stage="static_scratch", **prob) == 0
        for dst, src in zip(snaps[call], outs):
            dst.copy_(src)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device memory changed by {free_before - free_after} bytes"
    for call in range(2):
        for name, g_, w in zip(("dq", "dk", "dv"), snaps[call], want):
            ok, err = close(g_.float().cpu(), w.float().cpu(), ATOL[dt])
            assert ok, f"varlen call {call}: {name} differs from ab200_attn_bwd by {err}"
    # a packed call that does not declare its token count cannot be bounded and is refused
    a = cabi.make_bwd_args(q, k, v, out, do, *want, lse, None, **prob)
    a.q.size[2] = 0
    before = cabi.lib().ab200_launch_count()
    assert cabi.lib().ab200_attn_bwd_static_scratch(C.byref(a), None) == 1
    assert cabi.lib().ab200_launch_count() == before


def test_static_scratch_refuses_problems_beyond_its_array():
    from aotriton_b200 import cabi
    # batch * heads * seqlen = 2 * 64 * 16384 rows > 2**20: rejected on the host, nothing launched
    a = cabi.BwdArgs()
    a.prob.dtype = cabi.DTYPE_BF16
    a.prob.batch, a.prob.num_head_q, a.prob.num_head_k = 2, 64, 8
    a.prob.max_seqlen_q = a.prob.max_seqlen_k = 16384
    a.prob.head_dim_qk = a.prob.head_dim_vo = 128
    for view in (a.dq, a.dk, a.dv):
        view.ptr = 0x1000
    before = cabi.lib().ab200_launch_count()
    assert cabi.lib().ab200_attn_bwd_static_scratch(C.byref(a), None) == 1
    assert cabi.lib().ab200_launch_count() == before
    assert 2 * 64 * 16384 > cabi.STATIC_DELTA_FLOATS
