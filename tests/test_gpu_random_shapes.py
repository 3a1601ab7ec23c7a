"""Seeded random sweep of shapes and features through the automatic kernel choice and through the
general kernels, against the oracle.

The hand-picked cases of test_gpu_parity.py sit on the block boundaries someone thought of; this sweep
draws sequence lengths, head dims (multiples of 8 up to 256, so both the 128-wide kernels and the
one-accumulator kernels for wider heads are hit), GQA groups, windows, dropout and bias at random, so
that ragged last blocks, windows that miss whole blocks, single-block problems and dead rows meet every
kernel.  Tolerances as in test_gpu_parity.py (atol = rtol = 2e-2 bf16, 1e-2 fp16; LSE 1e-3).
"""
import os
import random

import pytest
import torch

from oracle import attention as A
from _util import ATOL, LSE_ATOL, FUDGE, close, randn_inputs, expected_family, reference_rule

pytestmark = pytest.mark.gpu

# AB200_SWEEP_FACTOR=N runs N times as many seeds, AB200_SWEEP_OFFSET=K starts them at K (an occasional
# long sweep over other cases; the defaults keep the suite short and fixed)
SWEEP = max(1, int(os.environ.get("AB200_SWEEP_FACTOR", "1")))
OFFSET = int(os.environ.get("AB200_SWEEP_OFFSET", "0"))

TL, BR = A.TOP_LEFT, A.BOTTOM_RIGHT


def _draw(seed: int):
    r = random.Random(seed)
    dt = r.choice([torch.float16, torch.bfloat16])
    B, Hk, G = r.choice([1, 2]), r.choice([1, 2]), r.choice([1, 1, 2, 3])
    Sq = r.choice([1, 7, 63, 64, 65, 127, 128, 129, 200, 257, 384, r.randint(1, 400)])
    Sk = r.choice([1, 5, 63, 64, 65, 127, 128, 129, 191, 300, 385, r.randint(1, 400)])
    wide = r.random() < 0.6
    D = 8 * r.randint(17, 32) if wide else 8 * r.randint(1, 16)
    Dv = D if r.random() < 0.7 else (8 * r.randint(1, 32))
    kind = r.choice(["none", "tl", "br", "window", "window"])
    if kind == "none":
        causal = (0, 0, 0)
    elif kind == "tl":
        causal = (3, TL, TL)
    elif kind == "br":
        causal = (3, BR, BR)
    else:
        causal = (3, r.randint(0, 300), r.randint(0, 300))
    p = r.choice([0.0, 0.0, 0.3])
    bias = r.random() < 0.3
    bshd = r.random() < 0.3      # (B, S, H, D) storage behind the logical (B, H, S, D) views
    return dt, B, Hk * G, Hk, Sq, Sk, D, Dv, causal, p, bias, bshd


@pytest.mark.parametrize("family", ["auto", "general", "fused"])
@pytest.mark.parametrize("seed", range(OFFSET, OFFSET + 96 * SWEEP))
def test_random_shape_vs_oracle(seed, family):
    from _gpu_runner import run_fwd_bwd
    dt, B, Hq, Hk, Sq, Sk, D, Dv, (ct, wl, wr), p, use_bias, bshd = _draw(seed)
    q, k, v, do = randn_inputs((B, Hq, Sq, D), (B, Hk, Sk, D), (B, Hk, Sk, Dv), dt, seed=1000 + seed)
    bias = None
    if use_bias:
        g = torch.Generator().manual_seed(seed)
        Skp = (Sk + 7) // 8 * 8
        bias = torch.randn(B, Hq, Sq, Skp, generator=g).to(dt)[..., :Sk]
    sm = D ** -0.5
    sd, off1, off2 = 0x1BF52, 0x1D4000, 0xB42
    mask = A.window_mask(Sq, Sk, ct, wl, wr)
    keep = A.keep_masks(sd, off1 + off2, B, Hq, Sq, Sk, p) if p > 0 else None
    ref = A.attention(q, k, v, sm_scale=sm, bias=bias, mask=mask, keep=keep, dropout_p=p, dout=do)
    res = run_fwd_bwd(q, k, v, do, sm_scale=sm, bias=bias, causal_type=ct, window_left=wl, window_right=wr,
                      dropout_p=p, seed=sd, offset1=off1, offset2=off2, family=family, want_dbias=use_bias,
                      keep_layout=(lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)) if bshd else None)
    tag = (f"seed {seed}/{family}: {dt} B{B} H{Hq}:{Hk} S{Sq}x{Sk} D{D}x{Dv} causal{(ct, wl, wr)} p{p} bias{use_bias} "
           f"bshd{bshd}")
    for which in ("fwd", "bwd"):
        want = 1 if family == "general" else expected_family(dt, D, Dv, which, family == "fused", use_bias)
        assert res[which + "_family"] == want, f"{tag}: {which} ran on family {res[which + '_family']}, expected {want}"
    lp = None
    for key in ("out", "dq", "dk", "dv"):
        ok, err = close(res[key].float(), getattr(ref, key), ATOL[dt])
        if not ok and Sk > 1:
            # Shapes with few keys and many queries (or the reverse) sum hundreds of 16-bit-rounded
            # probabilities into one gradient element, which no flat tolerance fits; the reference suite's own
            # criterion applies there: error relative to that of a math SDPA in the input dtype
            # (modules/flash/tests/_common_test.py:460-495).
            if lp is None:
                lp = A.sdpa_math_reference(q, k, v, sm_scale=sm, bias=bias, mask=mask, keep=keep, dropout_p=p, dout=do,
                                           acc_dtype=dt)
            ok, err, tol = reference_rule(res[key].float(), getattr(ref, key), getattr(lp, key).float(), FUDGE[key])
            assert ok, f"{tag}: {key} err {err} beyond the flat tolerance and the reference rule's {tol}"
        assert ok, f"{tag}: {key} max err {err}"
    ok, err = close(res["lse"].reshape(-1), ref.lse.reshape(-1).float(), LSE_ATOL)
    assert ok, f"{tag}: lse max err {err}"
    if use_bias:
        # dB = dS = P (dP - delta) per element, not a sum: it carries delta's error in full where P is near 1,
        # and delta = rowsum(O dO) is taken from the 16-bit O (error ~ 2^-9 |O||dO| sqrt(D), which the other
        # tests also allow for with 4 x the flat tolerance on delta)
        ok, err = close(res["db"].float(), ref.db, ATOL[dt] * 4, ATOL[dt])
        assert ok, f"{tag}: db max err {err}"


@pytest.mark.parametrize("family", ["auto", "general"])
@pytest.mark.parametrize("seed", range(OFFSET, OFFSET + 24 * SWEEP))
def test_random_compact_varlen_vs_oracle(seed, family):
    """Token-packed sequences of random lengths (empty ones included) in THD storage."""
    import numpy as np
    from _gpu_runner import run_fwd_bwd
    r = random.Random(5000 + seed)
    dt = r.choice([torch.float16, torch.bfloat16])
    Hk, G = r.choice([1, 2]), r.choice([1, 2])
    Hq = Hk * G
    D = 8 * r.randint(1, 32)
    lens = [r.choice([0, 1, 5, 63, 64, 65, 127, 128, 129, 200, r.randint(1, 260)]) for _ in range(r.randint(2, 6))]
    if max(lens) == 0:
        lens[0] = 17
    cu = [0] + list(np.cumsum(lens))
    T = int(cu[-1])
    p = r.choice([0.0, 0.2])
    ct, wl, wr = r.choice([(0, 0, 0), (3, TL, TL), (3, BR, BR), (3, r.randint(0, 200), r.randint(0, 200))])
    g = torch.Generator().manual_seed(seed)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    sm = D ** -0.5
    ref = A.attention_varlen(q, k, v, cu, cu, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr,
                             dropout_p=p, seed=42, offset_base=0, max_sq=max(lens), max_sk=max(lens), dout=do)
    thd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    res = run_fwd_bwd(q, k, v, do, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr, dropout_p=p,
                      seed=42, offset1=0, offset2=0, cu_q=cu, cu_k=cu, max_sq=max(lens), max_sk=max(lens),
                      family=family, keep_layout=thd)
    tag = f"varlen seed {seed}/{family}: {dt} H{Hq}:{Hk} lens{lens} D{D} causal{(ct, wl, wr)} p{p}"
    for which in ("fwd", "bwd"):
        want = 1 if family == "general" else expected_family(dt, D, D, which)
        assert res[which + "_family"] == want, f"{tag}: {which} ran on family {res[which + '_family']}"
    for key in ("out", "dq", "dk", "dv"):
        ok, err = close(res[key].float(), getattr(ref, key), ATOL[dt])
        assert ok, f"{tag}: {key} max err {err}"


@pytest.mark.parametrize("family", ["auto", "general"])
@pytest.mark.parametrize("seed", range(OFFSET, OFFSET + 16 * SWEEP))
def test_random_padded_and_strided_varlen_vs_oracle(seed, family):
    """Padded varlen (rank-4 tensors, lengths from cu_seqlens) and strided varlen (THD storage with gaps,
    offsets from seq_strides) with random lengths, head dims and windows; each sequence against the dense
    oracle on its own slice."""
    import numpy as np
    from aotriton_b200 import cabi
    from _gpu_runner import run_fwd_bwd
    r = random.Random(9000 + seed)
    dt = r.choice([torch.float16, torch.bfloat16])
    Hk, G = r.choice([1, 2]), r.choice([1, 2])
    Hq = Hk * G
    D = 8 * r.randint(1, 32)
    lens = [r.choice([1, 17, 63, 64, 65, 128, 129, 150, r.randint(1, 200)]) for _ in range(r.randint(2, 4))]
    nseq, S = len(lens), max(lens)
    cu = [0] + list(np.cumsum(lens))
    ct, wl, wr = r.choice([(0, 0, 0), (3, TL, TL), (3, BR, BR), (3, r.randint(0, 150), r.randint(0, 150))])
    sm = D ** -0.5
    tag = f"seed {seed}/{family}: {dt} H{Hq}:{Hk} lens{lens} D{D} causal{(ct, wl, wr)}"

    def check(got, ref, what, L):
        for key in ("out", "dq", "dk", "dv"):
            ok, err = close(got[key].float(), getattr(ref, key), ATOL[dt])
            assert ok, f"{tag}: {what} {key} max err {err}"

    # padded
    q, k, v, do = randn_inputs((nseq, Hq, S, D), (nseq, Hk, S, D), (nseq, Hk, S, D), dt, seed=seed)
    res = run_fwd_bwd(q, k, v, do, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr, cu_q=cu, cu_k=cu,
                      max_sq=S, max_sk=S, family=family, varlen_type=cabi.VARLEN_PADDED)
    for which in ("fwd", "bwd"):
        want = 1 if family == "general" else expected_family(dt, D, D, which)
        assert res[which + "_family"] == want, f"{tag}: padded {which} ran on family {res[which + '_family']}"
    for z, L in enumerate(lens):
        ref = A.attention(q[z:z + 1, :, :L], k[z:z + 1, :, :L], v[z:z + 1, :, :L], sm_scale=sm,
                          mask=A.window_mask(L, L, ct, wl, wr), dout=do[z:z + 1, :, :L])
        check({n: res[n][z:z + 1, :, :L] for n in ("out", "dq", "dk", "dv")}, ref, f"padded z={z}", L)
    # strided: random gaps between the sequences
    starts = [0]
    for L in lens:
        starts.append(starts[-1] + L + r.choice([0, 3, 16, 40]))
    T = starts[-1]
    g = torch.Generator().manual_seed(seed)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    thd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    res = run_fwd_bwd(q, k, v, do, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr, cu_q=cu, cu_k=cu,
                      max_sq=S, max_sk=S, family=family, varlen_type=cabi.VARLEN_STRIDED, seq_strides_q=starts,
                      seq_strides_k=starts, keep_layout=thd)
    for z, L in enumerate(lens):
        a = starts[z]
        ref = A.attention(q[:, :, a:a + L], k[:, :, a:a + L], v[:, :, a:a + L], sm_scale=sm,
                          mask=A.window_mask(L, L, ct, wl, wr), dout=do[:, :, a:a + L])
        check({n: res[n][:, :, a:a + L] for n in ("out", "dq", "dk", "dv")}, ref, f"strided z={z}", L)
