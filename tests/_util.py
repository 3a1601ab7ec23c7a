"""Shared helpers of the test-suite: golden-vector loading, tolerances, input generation."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
TORCH_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}

# Flat acceptance tolerances of the build target (O, dQ, dK, dV, dB per dtype; LSE separately).
ATOL = {torch.bfloat16: 2e-2, torch.float16: 1e-2, torch.float32: 1e-4}
LSE_ATOL = 1e-3


def load_golden(name: str) -> dict:
    z = np.load(GOLDEN / f"{name}.npz")
    dt = TORCH_DT[str(z["dtype"])]
    out = {"dtype": dt, "sm_scale": float(z["sm_scale"])}
    for key in z.files:
        if key in ("dtype", "sm_scale"):
            continue
        a = z[key]
        if key in ("q", "k", "v", "do", "o", "dq", "dk", "dv", "b", "db"):
            t = torch.from_numpy(a)
            out[key] = t.view(torch.bfloat16) if dt == torch.bfloat16 else t
        elif key in ("lse", "delta"):
            out[key] = torch.from_numpy(a)
        else:
            out[key] = a
    out["causal_type"], out["window_left"], out["window_right"] = (int(x) for x in z["causal"])
    return out


def close(actual: torch.Tensor, expected: torch.Tensor, atol: float, rtol: float | None = None) -> tuple[bool, float]:
    """allclose with rtol defaulting to atol; returns (ok, max abs error).  NaN anywhere fails."""
    rtol = atol if rtol is None else rtol
    a, e = actual.double(), expected.double()
    if torch.isnan(a).any():
        return False, float("nan")
    finite = torch.isfinite(e)
    if not torch.equal(torch.isfinite(a), finite):
        return False, float("inf")
    if not torch.equal(a[~finite], e[~finite]):
        return False, float("inf")
    err = (a[finite] - e[finite]).abs()
    ok = bool((err <= atol + rtol * e[finite].abs()).all())
    return ok, float(err.max()) if err.numel() else 0.0


def reference_rule(actual, ref_hp, ref_lp, fudge: float) -> tuple[bool, float, float]:
    """The reference test-suite's own criterion (modules/flash/tests/_common_test.py:460-495):
    max|x - ref_hp| <= max(1e-5, fudge * max|ref_hp - ref_lp|)."""
    ref_err = float((ref_hp.double() - ref_lp.double()).abs().max())
    tol = max(1e-5, fudge * ref_err)
    err = float((actual.double() - ref_hp.double()).abs().max())
    return err <= tol, err, tol


FUDGE = {"out": 3.0, "dq": 148.0, "dk": 48.0, "dv": 36.0, "db": 17.0}


def randn_inputs(shape_q, shape_k, shape_v, dtype, seed, device="cpu", dist="randn"):
    g = torch.Generator().manual_seed(seed)
    f = torch.randn if dist == "randn" else torch.rand
    q = f(shape_q, generator=g, dtype=torch.float32).to(dtype)
    k = f(shape_k, generator=g, dtype=torch.float32).to(dtype)
    v = f(shape_v, generator=g, dtype=torch.float32).to(dtype)
    do = f(shape_q[:-1] + (shape_v[-1],), generator=g, dtype=torch.float32).to(dtype)
    return tuple(t.to(device) for t in (q, k, v, do))


def expected_family(dtype, d_qk: int, d_vo: int, which: str = "fwd", fused: bool = False, dbias: bool = False) -> int:
    """Kernel family the automatic choice must take for freshly allocated (16-byte aligned, unit inner
    stride) tensors: 2 = tcgen05 whenever the shape is inside those kernels' range, 1 = general; the
    backward reports 3 when it ran the fused form (dQ accumulator given, head dim above 64, no dBias)."""
    if dtype not in (torch.float16, torch.bfloat16):
        return 1
    if d_qk > 256 or d_vo > 256 or d_qk % 8 or d_vo % 8:
        return 1
    # the fused form exists for the 128-wide instantiation only
    if which == "bwd" and fused and not dbias and 64 < max(d_qk, d_vo) <= 128:
        return 3
    return 2
