"""GPU parity tests: the CUDA kernels, called through the C-ABI, against the CPU oracle, the golden
vectors produced by the reference's own kernels, and the reference test-suite's acceptance rule.

Tolerances (written here on purpose): O, dQ, dK, dV, dB within atol = rtol = 2e-2 for bf16, 1e-2 for
fp16, 1e-4 for fp32; LSE within 1e-3; dropout keep masks bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import attention as A
from oracle import philox
from _util import ATOL, LSE_ATOL, FUDGE, load_golden, close, reference_rule, randn_inputs, expected_family

pytestmark = pytest.mark.gpu

FAMILIES = ["general", "auto", "fused"]
TL, BR = A.TOP_LEFT, A.BOTTOM_RIGHT


def _runner():
    from _gpu_runner import run_fwd_bwd
    return run_fwd_bwd


def _check_family(res, family, dt, d_qk, d_vo, tag, dbias=False):
    """The automatic choice must land on the tcgen05 kernels exactly when the shape is in their range
    (a stride or alignment regression would otherwise fall back silently and still pass parity)."""
    want = {"general": 1, "sm100": 2}.get(family)
    for which in ("fwd", "bwd"):
        if which + "_family" not in res:
            continue
        w = want if want is not None else expected_family(dt, d_qk, d_vo, which, family == "fused", dbias)
        assert res[which + "_family"] == w, f"{tag}: {which} ran on family {res[which + '_family']}, expected {w}"


def _check(res, ref, dt, tag, keys=("out", "dq", "dk", "dv"), lse=True, scale=1.0):
    for key in keys:
        ok, err = close(res[key].float(), getattr(ref, key), ATOL[dt] * scale)
        assert ok, f"{tag}:{key} max err {err}"
    if lse and res.get("lse") is not None:
        ok, err = close(res["lse"].reshape(-1), ref.lse.reshape(-1).float(), LSE_ATOL)
        assert ok, f"{tag}:lse max err {err}"


@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("name", ["dense_causal_fp16", "gqa_swa_fp16", "bias_padded_d24_fp16",
                                  "noncausal_gqa_fp16_d32", "bottom_right_fp32"])
def test_golden_dense(name, family):
    """Same inputs as the reference's kernels were run on; compare with what they produced."""
    g = load_golden(name)
    dt = g["dtype"]
    B, Hq, Hk, Sq, Sk, D, Dv = (int(x) for x in g["dims"])
    res = _runner()(g["q"], g["k"], g["v"], g["do"], sm_scale=g["sm_scale"], bias=g.get("b"),
                    causal_type=g["causal_type"], window_left=g["window_left"], window_right=g["window_right"],
                    family=family, want_dbias="b" in g)
    _check_family(res, family, dt, D, Dv, name, dbias="b" in g)
    for key, gk in (("out", "o"), ("dq", "dq"), ("dk", "dk"), ("dv", "dv")):
        ok, err = close(res[key].float(), g[gk].float(), ATOL[dt])
        assert ok, f"{name}:{key} max err {err}"
    ok, err = close(res["lse"], g["lse"], 2e-3 if "b" in g else LSE_ATOL)
    assert ok, f"{name}:lse {err}"
    ok, err = close(res["delta"], g["delta"], ATOL[dt] * 4)
    assert ok, f"{name}:delta {err}"
    if "b" in g:
        ok, err = close(res["db"].float(), g["db"].float(), ATOL[dt])
        assert ok, f"{name}:db {err}"


@pytest.mark.parametrize("family", FAMILIES)
def test_golden_varlen(family):
    g = load_golden("varlen_causal_fp16")
    cu_q, cu_k = g["cu_q"].tolist(), g["cu_k"].tolist()
    lens = np.diff(g["cu_q"])
    thd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)     # (1,H,T,D) view of THD storage
    res = _runner()(g["q"], g["k"], g["v"], g["do"], sm_scale=g["sm_scale"], causal_type=g["causal_type"],
                    window_left=g["window_left"], window_right=g["window_right"], cu_q=cu_q, cu_k=cu_k,
                    max_sq=int(lens.max()), max_sk=int(lens.max()), family=family, keep_layout=thd)
    _check_family(res, family, g["dtype"], g["q"].shape[3], g["v"].shape[3], "golden varlen")
    for key, gk in (("out", "o"), ("dq", "dq"), ("dk", "dk"), ("dv", "dv")):
        ok, err = close(res[key].float(), g[gk].float(), ATOL[g["dtype"]])
        assert ok, f"{key} max err {err}"
    ok, err = close(res["lse"], g["lse"], LSE_ATOL)
    assert ok, f"lse {err}"


CASES = [
    # dtype, B, Hq, Hk, Sq, Sk, D, Dv, causal(type, wl, wr), dropout, bias
    (torch.float16, 2, 4, 4, 128, 128, 64, 64, (0, 0, 0), 0.0, False),
    (torch.bfloat16, 1, 4, 2, 200, 200, 128, 128, (3, TL, TL), 0.0, False),
    (torch.bfloat16, 2, 8, 2, 256, 256, 128, 128, (3, 64, 0), 0.0, False),
    (torch.float16, 1, 4, 1, 177, 263, 128, 128, (3, BR, BR), 0.0, False),
    (torch.float16, 3, 5, 5, 11, 31, 8, 8, (0, 0, 0), 0.5, False),
    (torch.bfloat16, 3, 10, 2, 523, 337, 64, 64, (3, TL, TL), 0.5, False),
    (torch.float16, 2, 2, 2, 96, 160, 72, 72, (0, 0, 0), 0.2, True),
    (torch.float16, 1, 2, 2, 130, 130, 256, 256, (0, 0, 0), 0.2, True),
    (torch.float32, 2, 4, 4, 128, 128, 64, 64, (0, 0, 0), 0.0, False),
    (torch.float16, 1, 2, 2, 64, 64, 184, 184, (3, TL, TL), 0.0, False),
    (torch.bfloat16, 1, 2, 1, 100, 100, 24, 152, (0, 0, 0), 0.0, False),
    (torch.float16, 1, 2, 2, 300, 300, 128, 128, (3, 5, 7), 0.1, False),
    (torch.bfloat16, 1, 1, 1, 1, 1, 128, 128, (3, TL, TL), 0.0, False),
    (torch.float16, 1, 3, 3, 129, 1, 32, 32, (0, 0, 0), 0.0, False),
    # a whole 128-row tile of dead rows beside a live one (bottom-right causal, Sq > Sk)
    (torch.bfloat16, 1, 2, 2, 300, 100, 128, 128, (3, BR, BR), 0.0, False),
    # sliding window over several key blocks: the two query tiles of a CTA reach different blocks
    (torch.float16, 1, 2, 1, 700, 700, 64, 64, (3, 130, 20), 0.0, False),
    # head dims above 128 (the backward's one-accumulator kernels): GQA with a window over several
    # 64-row blocks and ragged ends; bottom-right causal with dead rows and dropout; unequal head dims
    (torch.bfloat16, 2, 4, 2, 300, 420, 192, 192, (3, 100, 30), 0.0, False),
    (torch.float16, 1, 2, 2, 257, 129, 256, 256, (3, BR, BR), 0.1, False),
    (torch.bfloat16, 1, 2, 1, 384, 384, 256, 136, (3, TL, TL), 0.0, False),
    (torch.float16, 1, 3, 3, 200, 333, 160, 160, (0, 0, 0), 0.3, True),
]


@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{str(c[0])[6:]}-B{c[1]}H{c[2]}:{c[3]}-S{c[4]}x{c[5]}-D{c[6]}x{c[7]}-c{c[8][0]}-p{c[9]}-b{int(c[10])}")
@pytest.mark.parametrize("dist", ["randn", "rand"])
def test_dense_vs_oracle(case, family, dist):
    dt, B, Hq, Hk, Sq, Sk, D, Dv, (ct, wl, wr), p, use_bias = case
    q, k, v, do = randn_inputs((B, Hq, Sq, D), (B, Hk, Sk, D), (B, Hk, Sk, Dv), dt, seed=hash((Sq, Sk, D)) % 1000,
                               dist=dist)
    bias = None
    if use_bias:
        g = torch.Generator().manual_seed(5)
        # last dim over-allocated to a multiple of 8 then sliced, as the reference tests do
        Skp = (Sk + 7) // 8 * 8
        bias = torch.randn(B, Hq, Sq, Skp, generator=g).to(dt)[..., :Sk]
    sm = 1.0 / (D ** 0.5)
    seed, off1, off2 = 0x1BF52, 0x1D4000, 0xB42
    mask = A.window_mask(Sq, Sk, ct, wl, wr)
    keep = A.keep_masks(seed, off1 + off2, B, Hq, Sq, Sk, p) if p > 0 else None
    ref = A.attention(q, k, v, sm_scale=sm, bias=bias, mask=mask, keep=keep, dropout_p=p, dout=do)
    res = _runner()(q, k, v, do, sm_scale=sm, bias=bias, causal_type=ct, window_left=wl, window_right=wr,
                    dropout_p=p, seed=seed, offset1=off1, offset2=off2, family=family, want_dbias=use_bias)
    tag = f"{case}/{family}/{dist}"
    _check_family(res, family, dt, D, Dv, tag, dbias=use_bias)
    # Flat tolerances scale with the size of the reference values for unnormalised N(0,1) gradients.
    _check(res, ref, dt, tag)
    if use_bias:
        ok, err = close(res["db"].float(), ref.db, ATOL[dt])
        assert ok, f"{tag}:db {err}"
    ok, err = close(res["delta"].reshape(-1), ref.delta.reshape(-1), ATOL[dt] * 4)
    assert ok, f"{tag}:delta {err}"
    if p > 0:
        assert res["seed_out"] == seed and res["off_out"] == off1 + off2
    # The reference suite's own criterion: error relative to the error of a same-dtype math SDPA
    # (computed on the host in the input dtype, the way _common_test.py:345-349 builds its
    # low-precision reference).  Skipped for Sk == 1, where the softmax is exactly 1, both
    # references agree to the last bit and the rule degenerates to an absolute 1e-5.
    if dt != torch.float32 and Sk > 1:
        lp = A.sdpa_math_reference(q, k, v, sm_scale=sm, bias=bias, mask=mask, keep=keep, dropout_p=p, dout=do,
                                   acc_dtype=dt)
        for n in ("out", "dq", "dk", "dv"):
            ok, err, tol = reference_rule(res[n].float(), getattr(ref, n), getattr(lp, n).float(), FUDGE[n])
            assert ok, f"{tag}:{n} reference rule err {err} > tol {tol}"


@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("dt,D,Hq,Hk,p,causal", [
    (torch.float16, 128, 4, 2, 0.1, True),
    (torch.bfloat16, 64, 2, 2, 0.0, False),
    (torch.float16, 32, 3, 3, 0.5, True),
    (torch.bfloat16, 256, 4, 2, 0.1, True),
    (torch.float16, 192, 2, 2, 0.0, False),
])
def test_compact_varlen_vs_oracle(family, dt, D, Hq, Hk, p, causal):
    lens = [4, 8, 63, 64, 128, 143, 0, 200, 1]
    cu = [0] + list(np.cumsum(lens))
    T = cu[-1]
    g = torch.Generator().manual_seed(11)
    mk = lambda H: torch.randn(1, T, H, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    sm = D ** -0.5
    ct, wl, wr = (3, TL, TL) if causal else (0, 0, 0)
    ref = A.attention_varlen(q, k, v, cu, cu, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr,
                             dropout_p=p, seed=42, offset_base=0, max_sq=max(lens), max_sk=max(lens), dout=do)
    thd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    res = _runner()(q, k, v, do, sm_scale=sm, causal_type=ct, window_left=wl, window_right=wr, dropout_p=p,
                    seed=42, offset1=0, offset2=0, cu_q=cu, cu_k=cu, max_sq=max(lens), max_sk=max(lens),
                    family=family, keep_layout=thd)
    _check_family(res, family, dt, D, D, "compact varlen")
    _check(res, ref, dt, f"varlen/{family}")
    ok, err = close(res["delta"], ref.delta, ATOL[dt] * 4)
    assert ok, f"delta {err}"


@pytest.mark.parametrize("family", FAMILIES)
def test_padded_and_strided_varlen(family):
    """Padded varlen: rank-4 tensors padded to max length, lengths from cu_seqlens.  Strided varlen:
    THD storage with gaps, token offsets from seq_strides."""
    from aotriton_b200 import cabi
    dt, Hq, D = torch.float16, 2, 64
    lens = [40, 17, 64]
    cu = [0] + list(np.cumsum(lens))
    S = max(lens)
    q, k, v, do = randn_inputs((3, Hq, S, D), (3, Hq, S, D), (3, Hq, S, D), dt, seed=3)
    sm = D ** -0.5
    res = _runner()(q, k, v, do, sm_scale=sm, causal_type=3, window_left=TL, window_right=TL, cu_q=cu, cu_k=cu,
                    max_sq=S, max_sk=S, family=family, varlen_type=cabi.VARLEN_PADDED)
    _check_family(res, family, dt, D, D, "padded varlen")
    for z, L in enumerate(lens):
        ref = A.attention(q[z:z + 1, :, :L], k[z:z + 1, :, :L], v[z:z + 1, :, :L], sm_scale=sm,
                          mask=A.window_mask(L, L, 3, TL, TL), dout=do[z:z + 1, :, :L])
        for key in ("out", "dq", "dk", "dv"):
            ok, err = close(res[key][z:z + 1, :, :L].float(), getattr(ref, key), ATOL[dt])
            assert ok, f"padded z={z} {key} {err}"
        ok, err = close(res["lse"].reshape(3, Hq, S)[z, :, :L], ref.lse[0], LSE_ATOL)
        assert ok, f"padded z={z} lse {err}"
    # strided: sequences start at offsets with gaps
    starts = [0, 48, 80, 150]   # last entry = total storage rows (row length of LSE)
    T = starts[-1]
    g = torch.Generator().manual_seed(9)
    mk = lambda: torch.randn(1, T, Hq, D, generator=g).to(dt).transpose(1, 2)
    q, k, v, do = mk(), mk(), mk(), mk()
    thd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    res = _runner()(q, k, v, do, sm_scale=sm, cu_q=cu, cu_k=cu, max_sq=S, max_sk=S, family=family,
                    varlen_type=cabi.VARLEN_STRIDED, seq_strides_q=starts, seq_strides_k=starts, keep_layout=thd)
    _check_family(res, family, dt, D, D, "strided varlen")
    for z, L in enumerate(lens):
        a = starts[z]
        ref = A.attention(q[:, :, a:a + L], k[:, :, a:a + L], v[:, :, a:a + L], sm_scale=sm, dout=do[:, :, a:a + L])
        for key in ("out", "dq", "dk", "dv"):
            ok, err = close(res[key][:, :, a:a + L].float(), getattr(ref, key), ATOL[dt])
            assert ok, f"strided z={z} {key} {err}"
        ok, err = close(res["lse"][:, a:a + L], ref.lse[0], LSE_ATOL)
        assert ok, f"strided z={z} lse {err}"


@pytest.mark.parametrize("family", FAMILIES)
def test_bshd_layout(family):
    """(B,S,H,D) storage passed as a permuted view."""
    dt = torch.bfloat16
    q, k, v, do = randn_inputs((2, 4, 192, 128), (2, 2, 192, 128), (2, 2, 192, 128), dt, seed=21)
    sm = 128 ** -0.5
    ref = A.attention(q, k, v, sm_scale=sm, mask=A.window_mask(192, 192, 3, TL, TL), dout=do)
    bshd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    res = _runner()(q, k, v, do, sm_scale=sm, causal_type=3, window_left=TL, window_right=TL, family=family,
                    keep_layout=bshd)
    _check_family(res, family, dt, 128, 128, "bshd")
    _check(res, ref, dt, f"bshd/{family}")


@pytest.mark.parametrize("family", FAMILIES)
def test_lse_known_answer_and_null_lse(family):
    # Q = K = V = I16, scale 1/4: every LSE is 2.79018449783325195 (reference known-answer test)
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        eye = torch.eye(16, dtype=dt).reshape(1, 1, 16, 16)
        res = _runner()(eye, eye, eye, None, sm_scale=0.25, family=family)
        assert torch.allclose(res["lse"], torch.full_like(res["lse"], 2.79018449783325195), atol=1e-5)
        res2 = _runner()(eye, eye, eye, None, sm_scale=0.25, family=family, lse_null=True)
        assert torch.equal(res["out"], res2["out"])


@pytest.mark.parametrize("family", FAMILIES)
def test_large_bf16_values_no_nan(family):
    # all-133120.0 bf16 inputs must not produce NaN (reference test_large_bf16_nan_values)
    x = torch.full((1, 1, 256, 128), 133120.0, dtype=torch.bfloat16)
    res = _runner()(x, x, x, None, sm_scale=128 ** -0.5, causal_type=3, window_left=TL, window_right=TL,
                    family=family)
    assert not torch.isnan(res["out"].float()).any() and not torch.isnan(res["lse"]).any()
    assert torch.allclose(res["out"].float(), torch.full_like(res["out"].float(), 133120.0))


@pytest.mark.parametrize("family", FAMILIES)
def test_fully_masked_rows_and_zero_scale(family):
    # bottom-right causal with Sq > Sk: the first Sq-Sk rows see no key -> O = 0, LSE = +inf, zero grads
    dt = torch.float16
    q, k, v, do = randn_inputs((1, 2, 160, 64), (1, 2, 96, 64), (1, 2, 96, 64), dt, seed=2)
    res = _runner()(q, k, v, do, sm_scale=0.125, causal_type=3, window_left=BR, window_right=BR, family=family)
    dead = 160 - 96
    assert torch.all(res["out"][:, :, :dead] == 0)
    assert torch.all(torch.isinf(res["lse"].reshape(1, 2, 160)[:, :, :dead]))
    assert torch.all(res["dq"][:, :, :dead] == 0)
    ref = A.attention(q, k, v, sm_scale=0.125, mask=A.window_mask(160, 96, 3, BR, BR), dout=do)
    _check(res, ref, dt, f"dead-rows/{family}")
    # sm_scale == 0 with masking: uniform attention over the unmasked keys, no NaN
    res = _runner()(q, k, v, do, sm_scale=0.0, causal_type=3, window_left=TL, window_right=TL, family=family)
    ref = A.attention(q, k, v, sm_scale=0.0, mask=A.window_mask(160, 96, 3, TL, TL), dout=do)
    _check(res, ref, dt, f"zero-scale/{family}")


def test_dropout_mask_bit_exact_debug_kernel():
    """debug_simulate_encoded_softmax against the integer oracle, element for element."""
    from aotriton_b200 import cabi
    for (B, H, Sq, Sk, p, seed, off1, off2, dt) in [
        (2, 3, 77, 131, 0.1, 42, 0, 0, torch.float16),
        (1, 2, 64, 64, 0.5, 0x1BF52, 0x1D4000, 0xB42, torch.bfloat16),
        (1, 1, 33, 1026, 0.2, 0xDEADBEEFCAFEF00D, (1 << 33) + 5, 3, torch.float32),
    ]:
        r = torch.zeros(B, H, Sq, Sk, dtype=dt, device="cuda")
        st = torch.from_numpy(np.array([seed], dtype=np.uint64)).cuda()
        ot = torch.from_numpy(np.array([off1], dtype=np.uint64)).cuda()
        assert cabi.debug_simulate_encoded_softmax(r, p, st, ot, off2) == 0
        got = (r.cpu().float() > 0)
        assert torch.all(r.cpu().float().abs() == 0.5)
        want = A.keep_masks(seed, off1 + off2, B, H, Sq, Sk, p)
        assert torch.equal(got, want)


@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("dt,D", [(torch.float16, 128), (torch.bfloat16, 64)])
def test_dropout_mask_bit_exact_through_forward(family, dt, D):
    """With V = identity (Sk <= D) the output is the dropped probability matrix itself, so its zero
    pattern is the keep mask the forward kernel used -- compared bit for bit with the oracle."""
    B, H, Sq, Sk, p = 2, 3, 150, D, 0.3
    g = torch.Generator().manual_seed(8)
    q = (torch.randn(B, H, Sq, D, generator=g) * 0.1).to(dt)
    k = (torch.randn(B, H, Sk, D, generator=g) * 0.1).to(dt)
    v = torch.eye(D, dtype=dt).reshape(1, 1, D, D).expand(B, H, D, D).contiguous()
    res = _runner()(q, k, v, None, sm_scale=1.0, dropout_p=p, seed=123, offset1=1000, offset2=7, family=family)
    want = A.keep_masks(123, 1007, B, H, Sq, Sk, p)
    assert torch.equal(res["out"].float() != 0, want)


def test_error_codes_on_device():
    from aotriton_b200 import cabi
    q = torch.zeros(1, 1, 16, 16, dtype=torch.float16, device="cuda")
    assert cabi.lib().ab200_check_gpu(None) == 0
    assert cabi.lib().ab200_multiprocessor_count(None) > 0
    out = torch.zeros_like(q)
    assert cabi.attn_fwd(q, q, q, out, None, sm_scale=1.0) == 0
    # a shape outside the tcgen05 kernels' range is refused, not silently rerouted, when they are forced
    cabi.lib().ab200_set_kernel_family(2)
    try:
        q8 = torch.zeros(1, 1, 16, 8, dtype=torch.float32, device="cuda")
        assert cabi.attn_fwd(q8, q8, q8, torch.zeros_like(q8), None, sm_scale=1.0) == 801
    finally:
        cabi.lib().ab200_set_kernel_family(0)
    torch.cuda.synchronize()
