"""GPU: the corners a plain parity sweep does not reach, all through the C-ABI on one device.

  * a dropout problem cut into the batch x kv-head segments a multi-GPU run would use (world sizes
    2, 4, 8, run one after another on this device) must reproduce the unsharded result bit for bit,
    which exercises the kernels' philox_offset2 / philox_head_offset / philox_num_head_q handling;
  * padded, compact and strided varlen whose padding and gap rows hold NaN or inf must give the same
    finite results as with benign padding (the reference zero-fills loads beyond a sequence's end,
    modules/flash/kernel/masked_load_store.py:214-307);
  * a bounded wait that runs out: the kernel returns, the status word names the wait, the entry
    points refuse further work until the word is reset, and a normal launch then succeeds.

Tolerances: bit-exact where stated, otherwise atol = rtol = 2e-2 (bf16) / 1e-2 (fp16), LSE 1e-3.
"""
import numpy as np
import pytest
import torch

from oracle import attention as A
from _util import ATOL, LSE_ATOL, close, randn_inputs

pytestmark = pytest.mark.gpu
TL = A.TOP_LEFT
FAMILY = {"general": 1, "sm100": 2}


class _Family:
    def __init__(self, name):
        self.code = FAMILY[name]

    def __enter__(self):
        from aotriton_b200 import cabi
        self.old = cabi.lib().ab200_set_kernel_family(self.code)

    def __exit__(self, *exc):
        from aotriton_b200 import cabi
        cabi.lib().ab200_set_kernel_family(self.old)


def _fwd_bwd(q, k, v, do, lse_shape, **prob):
    """Device tensors (views allowed) in, NaN-prefilled device outputs back."""
    from aotriton_b200 import cabi
    out = torch.full_like(q, float("nan"))
    lse = torch.full(lse_shape, float("nan"), dtype=torch.float32, device="cuda")
    delta = torch.full(lse_shape, float("nan"), dtype=torch.float32, device="cuda")
    seed_out = torch.zeros(1, dtype=torch.uint64, device="cuda")
    off_out = torch.zeros(1, dtype=torch.uint64, device="cuda")
    err = cabi.attn_fwd(q, k, v, out, lse, philox_seed_output=seed_out, philox_offset_output=off_out, **prob)
    assert err == 0, f"attn_fwd returned {err}"
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
    err = cabi.attn_bwd(q, k, v, out, do, dq, dk, dv, lse, delta, **prob)
    assert err == 0, f"attn_bwd returned {err}"
    torch.cuda.synchronize()
    return dict(out=out, lse=lse, dq=dq, dk=dk, dv=dv)


# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("family", ["general", "sm100"])
def test_sharded_dense_dropout_is_bit_identical(family):
    from aotriton_b200 import cabi, sharding
    dt, B, Hq, Hk, S, D, p = torch.bfloat16, 3, 8, 4, 200, 64, 0.25
    G = Hq // Hk
    q, k, v, do = (t.cuda() for t in randn_inputs((B, Hq, S, D), (B, Hk, S, D), (B, Hk, S, D), dt, seed=31))
    seed = torch.tensor([77], dtype=torch.uint64, device="cuda")
    off1 = torch.tensor([1234], dtype=torch.uint64, device="cuda")
    prob = dict(sm_scale=D ** -0.5, causal_type=3, window_left=TL, window_right=TL, dropout_p=p, philox_seed=seed,
                philox_offset1=off1)
    with _Family(family):
        full = _fwd_bwd(q, k, v, do, (B * Hq, S), philox_offset2=5, **prob)
        assert not any(torch.isnan(t.float()).any() for t in full.values())
        for world in (2, 4, 8):
            got = {n: torch.full_like(t, float("nan")) for n, t in full.items()}
            for rank in range(world):
                for seg in sharding.partition_dense(B, Hk, world, rank):
                    adj = sharding.philox_adjustment(seg, G, Hq, S, S)
                    qs, ks = sharding.slice_dense(seg, G, q, k)
                    dos, vs = sharding.slice_dense(seg, G, do, v)
                    nh = qs.shape[1]
                    r = _fwd_bwd(qs, ks, vs, dos, (nh, S), philox_offset2=5 + adj["philox_offset2_add"],
                                 philox_head_offset=adj["philox_head_offset"],
                                 philox_num_head_q=adj["philox_num_head_q"], **prob)
                    sharding.slice_dense(seg, G, got["out"]).copy_(r["out"])
                    sharding.slice_dense(seg, G, got["dq"]).copy_(r["dq"])
                    _, dks = sharding.slice_dense(seg, G, got["dq"], got["dk"]); dks.copy_(r["dk"])
                    _, dvs = sharding.slice_dense(seg, G, got["dq"], got["dv"]); dvs.copy_(r["dv"])
                    sharding.slice_lse_dense(seg, G, got["lse"], Hq).copy_(r["lse"])
            for n in full:
                assert torch.equal(got[n].view(torch.int16 if got[n].dtype == dt else torch.int32),
                                   full[n].view(torch.int16 if full[n].dtype == dt else torch.int32)), \
                    f"world {world}: {n} of the shards differs from the unsharded run"
    assert cabi.lib().ab200_kernel_status(0) == 0


@pytest.mark.parametrize("family", ["general", "sm100"])
def test_sharded_varlen_dropout_is_bit_identical(family):
    """Varlen problems are split over kv heads only; the q-head index of the Philox counter stays global."""
    from aotriton_b200 import cabi, sharding
    dt, Hq, Hk, D, p = torch.float16, 8, 4, 128, 0.1
    G = Hq // Hk
    lens = [70, 130, 1, 257]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
    T, smax = int(sum(lens)), max(lens)
    g = torch.Generator().manual_seed(12)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).cuda().transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    seed = torch.tensor([42], dtype=torch.uint64, device="cuda")
    off1 = torch.tensor([0], dtype=torch.uint64, device="cuda")
    prob = dict(sm_scale=D ** -0.5, causal_type=3, window_left=TL, window_right=TL, dropout_p=p, philox_seed=seed,
                philox_offset1=off1, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=smax, max_seqlen_k=smax)
    with _Family(family):
        full = _fwd_bwd(q, k, v, do, (Hq, T), **prob)
        for world in (2, 4):
            got = {n: torch.full_like(t, float("nan")) for n, t in full.items()}
            for rank in range(world):
                for seg in sharding.partition_varlen(Hk, world, rank):
                    hs = slice(seg.hk_lo * G, seg.hk_hi * G)
                    ks_ = slice(seg.hk_lo, seg.hk_hi)
                    r = _fwd_bwd(q[:, hs], k[:, ks_], v[:, ks_], do[:, hs], ((seg.hk_hi - seg.hk_lo) * G, T),
                                 philox_head_offset=seg.hk_lo * G, philox_num_head_q=Hq, **prob)
                    got["out"][:, hs] = r["out"]; got["dq"][:, hs] = r["dq"]
                    got["dk"][:, ks_] = r["dk"]; got["dv"][:, ks_] = r["dv"]
                    got["lse"][hs] = r["lse"]
            for n in full:
                assert torch.equal(torch.nan_to_num(got[n].float()), torch.nan_to_num(full[n].float())), \
                    f"world {world}: {n} of the shards differs from the unsharded run"
    assert cabi.lib().ab200_kernel_status(0) == 0


# ----------------------------------------------------------------------------------------------
def _valid_equal(tag, a, b, dt):
    assert not torch.isnan(a.float()).any() and not torch.isinf(a.float()).any(), f"{tag}: non-finite values"
    ok, err = close(a.float().cpu(), b.float().cpu(), ATOL[dt])
    assert ok, f"{tag}: differs from the run with benign padding by {err}"


@pytest.mark.parametrize("family", ["general", "sm100"])
@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_padded_varlen_ignores_nonfinite_padding(family, poison, D):
    from aotriton_b200 import cabi
    dt, Hq, Hk = torch.float16, 4, 2
    lens = [40, 17, 150, 128]
    S = 256
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
    base = [t.cuda() for t in randn_inputs((4, Hq, S, D), (4, Hk, S, D), (4, Hk, S, D), dt, seed=3)]
    prob = dict(sm_scale=D ** -0.5, causal_type=3, window_left=TL, window_right=TL, cu_seqlens_q=cu, cu_seqlens_k=cu,
                max_seqlen_q=S, max_seqlen_k=S, varlen_type=cabi.VARLEN_PADDED)
    with _Family(family):
        clean = _fwd_bwd(*base, (4 * Hq, S), **prob)
        bad = [t.clone() for t in base]
        for t in bad:
            for z, L in enumerate(lens):
                t[z, :, L:] = poison
        dirty = _fwd_bwd(*bad, (4 * Hq, S), **prob)
    for z, L in enumerate(lens):
        for n in ("out", "dq", "dk", "dv"):
            _valid_equal(f"padded z={z} {n}", dirty[n][z, :, :L], clean[n][z, :, :L], dt)
        ok, err = close(dirty["lse"].reshape(4, Hq, S)[z, :, :L].cpu(), clean["lse"].reshape(4, Hq, S)[z, :, :L].cpu(),
                        LSE_ATOL)
        assert ok, f"padded z={z} lse {err}"
    # and the benign run itself against the oracle, one sequence
    z, L = 2, lens[2]
    q, k, v, do = (t.cpu() for t in base)
    ref = A.attention(q[z:z + 1, :, :L], k[z:z + 1, :, :L], v[z:z + 1, :, :L], sm_scale=D ** -0.5,
                      mask=A.window_mask(L, L, 3, TL, TL), dout=do[z:z + 1, :, :L])
    for n in ("out", "dq", "dk", "dv"):
        ok, err = close(clean[n][z:z + 1, :, :L].float().cpu(), getattr(ref, n), ATOL[dt])
        assert ok, f"padded z={z} {n} vs oracle {err}"


@pytest.mark.parametrize("family", ["general", "sm100"])
@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
@pytest.mark.parametrize("D", [128, 192])
def test_compact_and_strided_varlen_ignore_nonfinite_neighbours(family, poison, D):
    """Compact: one whole sequence holds non-finite tokens; its neighbours, whose last partial blocks
    reach into it, must be unaffected.  Strided: the gaps between sequences hold non-finite values."""
    from aotriton_b200 import cabi
    dt, Hq, Hk = torch.bfloat16, 2, 2
    lens = [100, 60, 135, 5]
    cu_l = [0] + list(np.cumsum(lens))
    T = cu_l[-1]
    g = torch.Generator().manual_seed(9)
    mk = lambda H, n: torch.randn(1, n, H, D, generator=g).to(dt).cuda().transpose(1, 2)
    base = [mk(Hq, T), mk(Hk, T), mk(Hk, T), mk(Hq, T)]
    cu = torch.tensor(cu_l, dtype=torch.int32, device="cuda")
    prob = dict(sm_scale=D ** -0.5, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    with _Family(family):
        clean = _fwd_bwd(*base, (Hq, T), **prob)
        bad = [t.clone() for t in base]
        for t in bad:
            t[:, :, cu_l[1]:cu_l[2]] = poison          # sequence 1 is poisoned
        dirty = _fwd_bwd(*bad, (Hq, T), **prob)
    for z in (0, 2, 3):
        a, b = cu_l[z], cu_l[z + 1]
        for n in ("out", "dq", "dk", "dv"):
            _valid_equal(f"compact z={z} {n}", dirty[n][:, :, a:b], clean[n][:, :, a:b], dt)
    # strided: sequences at offsets with gaps, gaps poisoned
    starts = [0, 112, 200, 352, 368]      # last entry = rows of the storage (row length of LSE)
    Ts = starts[-1]
    base = [mk(Hq, Ts), mk(Hk, Ts), mk(Hk, Ts), mk(Hq, Ts)]
    ss = torch.tensor(starts, dtype=torch.int32, device="cuda")
    prob = dict(sm_scale=D ** -0.5, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens),
                varlen_type=cabi.VARLEN_STRIDED, seq_strides_q=ss, seq_strides_k=ss, causal_type=3, window_left=TL,
                window_right=TL)
    with _Family(family):
        clean = _fwd_bwd(*base, (Hq, Ts), **prob)
        bad = [t.clone() for t in base]
        for t in bad:
            for z, L in enumerate(lens):
                t[:, :, starts[z] + L:starts[z + 1]] = poison
        dirty = _fwd_bwd(*bad, (Hq, Ts), **prob)
    for z, L in enumerate(lens):
        a = starts[z]
        for n in ("out", "dq", "dk", "dv"):
            _valid_equal(f"strided z={z} {n}", dirty[n][:, :, a:a + L], clean[n][:, :, a:a + L], dt)
    assert cabi.lib().ab200_kernel_status(0) == 0


# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which,lo,hi,D", [(1, 0x100, 0x1000, 128), (2, 0x1000, 0x2000, 128), (3, 0x2000, 0x3000, 128),
                                           (2, 0x3000, 0x4000, 256), (3, 0x3000, 0x4000, 256)])
def test_bounded_wait_runs_out_cleanly(which, lo, hi, D):
    """One copy is left out on a one-tile problem with a wait limit of about a million cycles: the
    role waiting longest gives up, the kernel drains and returns, and the status word names a wait
    of the right kernel (forward 0x1xx-0x9xx, dK/dV 0x1xxx, dQ 0x2xxx, the kernels for head dims
    above 128 0x3xxx)."""
    from aotriton_b200 import cabi
    L = cabi.lib()
    dt, S = torch.bfloat16, 128
    q, k, v, do = (t.cuda() for t in randn_inputs((1, 1, S, D), (1, 1, S, D), (1, 1, S, D), dt, seed=1))
    out = torch.empty_like(q)
    lse = torch.empty(1, S, dtype=torch.float32, device="cuda")
    delta = torch.empty_like(lse)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    prob = dict(sm_scale=D ** -0.5)
    assert L.ab200_kernel_status(1) == 0
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
    torch.cuda.synchronize()
    want = out.clone()
    stream = torch.cuda.current_stream().cuda_stream
    old = L.ab200_set_kernel_family(2)
    L.ab200_debug_bounded_wait_test(which, 1000)
    try:
        if which == 1:
            assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
        else:
            stage = {2: "dkdv", 3: "dq"}[which]
            assert cabi.attn_bwd(q, k, v, out, do, dq, dk, dv, lse, delta, stage="preprocess", **prob) == 0
            assert cabi.attn_bwd(q, k, v, out, do, dq, dk, dv, lse, delta, stage=stage, **prob) == 0
    finally:
        L.ab200_debug_bounded_wait_test(0, 0)
        L.ab200_set_kernel_family(old)
    assert L.ab200_stream_check(stream) == 719                # hipErrorLaunchFailure
    code = L.ab200_kernel_status(0)
    assert lo <= code < hi, hex(code)
    # the failure is sticky: launches are refused until the word is reset
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 719
    assert L.ab200_kernel_status(1) == code
    assert L.ab200_kernel_status(0) == 0
    assert L.ab200_stream_check(stream) == 0
    out.fill_(float("nan"))
    assert cabi.attn_fwd(q, k, v, out, lse, **prob) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, want)
