"""CPU: the oracle against (a) the reference's known-answer test, (b) outputs of the
reference's own Triton kernels (tests/golden/*.npz) and (c) the reference's test oracle
(torch math SDPA + autograd)."""
import numpy as np
import pytest
import torch

from oracle import attention as A
from oracle import philox
from _util import GOLDEN, load_golden, close

DENSE = ["dense_causal_fp16", "gqa_swa_fp16", "bias_padded_d24_fp16", "noncausal_gqa_fp16_d32", "bottom_right_fp32"]


def test_lse_known_answer():
    # modules/flash/tests/_core_test_backward.py:333-351
    q = torch.eye(16).reshape(1, 1, 16, 16)
    r = A.attention(q, q, q, sm_scale=0.25)
    assert torch.allclose(r.lse, torch.full_like(r.lse, 2.79018449783325195), atol=1e-6)


def test_philox_matches_reference_fast_dropout_mask():
    z = np.load(GOLDEN / "philox_keep.npz")
    for i, (seed, base, x, y, stride, M, N) in enumerate(z["meta"].tolist()):
        p = float(z["p"][i])
        # fast_dropout_mask(seed, thr, base, x, y, M, N, stride): offset = base + (x+m)*stride + (y+n)//4
        m = np.arange(M, dtype=np.uint64)[:, None]
        c = np.arange(N // 4, dtype=np.uint64)[None, :]
        offs = np.uint64(base) + (np.uint64(x) + m) * np.uint64(stride) + np.uint64(y // 4) + c
        w = philox.philox4x32_10(seed, offs)[..., [0, 2, 1, 3]].reshape(M, N)
        keep = w.view(np.int32) > np.int32(philox.dropout_threshold(p))
        assert np.array_equal(keep.astype(np.int32), z[f"keep{i}"]), f"case {i}"


def test_dropout_threshold_values():
    assert philox.dropout_threshold(0.1) == -1717986944
    assert philox.dropout_threshold(0.2) == -1288490240
    assert philox.dropout_threshold(0.5) == 0


def test_keep_mask_layout():
    # keep_mask is the per-(z,h) rectangle of the same counter scheme
    full = philox.keep_mask(42, 7, 1, 2, 4, 24, 40, 24, 40, 0.3)
    stride = 10
    base = 7 + (1 * 4 + 2) * 24 * stride
    w = philox.philox4x32_10(42, np.array([base + 5 * stride + 3], dtype=np.uint64))[0]
    thr = philox.dropout_threshold(0.3)
    exp = [np.int32(w[j]) > thr for j in (0, 2, 1, 3)]
    assert list(full[5, 12:16]) == exp


@pytest.mark.parametrize("name", DENSE)
def test_oracle_vs_reference_kernels_dense(name):
    g = load_golden(name)
    dt = g["dtype"]
    B, Hq, Hk, Sq, Sk, D, Dv = (int(x) for x in g["dims"])
    mask = A.window_mask(Sq, Sk, g["causal_type"], g["window_left"], g["window_right"])
    r = A.attention(g["q"], g["k"], g["v"], sm_scale=g["sm_scale"], bias=g.get("b"), mask=mask, dout=g["do"],
                    round_dtype=dt)
    tol = {torch.float16: 4e-3, torch.bfloat16: 3e-2, torch.float32: 2e-5}[dt]
    for key, val in (("o", r.out), ("dq", r.dq), ("dk", r.dk), ("dv", r.dv)):
        ok, err = close(val, g[key].float(), tol)
        assert ok, f"{name}:{key} err={err}"
    # With bias the reference multiplies bias by log2(e) in the bias dtype (fwd_kernel_inner.py:187),
    # which costs it up to ~1e-3 in LSE against exact arithmetic.
    lse_tol = 2e-3 if "b" in g else (1e-4 if dt != torch.bfloat16 else 1e-3)
    ok, err = close(r.lse.reshape(B * Hq, Sq), g["lse"], lse_tol)
    assert ok, f"{name}:lse err={err}"
    ok, err = close(r.delta.reshape(B * Hq, Sq), g["delta"], tol * 4)
    assert ok, f"{name}:delta err={err}"
    if "db" in g:
        ok, err = close(r.db, g["db"].float(), tol)
        assert ok, f"{name}:db err={err}"


def test_oracle_vs_reference_kernels_varlen():
    g = load_golden("varlen_causal_fp16")
    cu_q, cu_k = g["cu_q"].tolist(), g["cu_k"].tolist()
    r = A.attention_varlen(g["q"], g["k"], g["v"], cu_q, cu_k, sm_scale=g["sm_scale"],
                           causal_type=g["causal_type"], window_left=g["window_left"],
                           window_right=g["window_right"], dout=g["do"], round_dtype=g["dtype"])
    for key, val in (("o", r.out), ("dq", r.dq), ("dk", r.dk), ("dv", r.dv)):
        ok, err = close(val, g[key].float(), 4e-3)
        assert ok, f"{key} err={err}"
    ok, err = close(r.lse, g["lse"], 1e-4)
    assert ok, f"lse err={err}"


@pytest.mark.parametrize("dropout_p", [0.0, 0.3])
def test_oracle_vs_math_sdpa(dropout_p):
    torch.manual_seed(0)
    B, Hq, Hk, S, D = 2, 4, 2, 40, 16
    q = torch.randn(B, Hq, S, D); k = torch.randn(B, Hk, S, D); v = torch.randn(B, Hk, S, D)
    do = torch.randn(B, Hq, S, D)
    mask = A.window_mask(S, S, 3, 12, 3)
    keep = A.keep_masks(42, 1000, B, Hq, S, S, dropout_p) if dropout_p else None
    a = A.attention(q, k, v, sm_scale=0.3, mask=mask, keep=keep, dropout_p=dropout_p, dout=do)
    b = A.sdpa_math_reference(q, k, v, sm_scale=0.3, mask=mask, keep=keep, dropout_p=dropout_p, dout=do)
    for n in ("out", "dq", "dk", "dv"):
        assert torch.allclose(getattr(a, n), getattr(b, n), atol=1e-5), n


def test_config1_cpu_plumbing():
    """First benchmark configuration: fp32 B=2 H=4 S=128 D=64, N(0,1) from seed 0, on the host."""
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(2, 4, 128, 64, generator=g) for _ in range(4))
    sm = 1.0 / 8.0
    a = A.attention(q, k, v, sm_scale=sm, dout=do)
    b = A.sdpa_math_reference(q, k, v, sm_scale=sm, dout=do)
    for n in ("out", "dq", "dk", "dv"):
        assert torch.allclose(getattr(a, n), getattr(b, n), atol=2e-5), n
    lse = torch.logsumexp(torch.matmul(q, k.transpose(-1, -2)) * sm, dim=-1)
    assert torch.allclose(a.lse, lse, atol=1e-5)
    assert a.delta.shape == (2, 4, 128)
