"""CPU: host-side behaviour of the operator API that needs no device -- error codes, argument
validation order, Python surface of pyaotriton, the sharding arithmetic."""
import numpy as np
import pytest
import torch

from aotriton_b200 import cabi, sharding, load_pyaotriton


def _views(p, dtype=None, D=64, S=32):
    dtype = dtype or p.DType.kFloat16
    t4 = p.T4(0x1000, [1, 2, S, D], [2 * S * D, S * D, D, 1], dtype)
    return t4


def test_python_surface():
    p = load_pyaotriton()
    for name in ("T0", "T1", "T2", "T4", "DType", "Stream", "hipError_t", "HipMemory", "get_name_suffix",
                 "hipGetLastError", "hipDeviceSynchronize"):
        assert hasattr(p, name), name
    assert p.v3.flash.attn_fwd_params.kVersion == 3 and p.v3.flash.attn_bwd_params.kVersion == 6
    for name in ("dq_acc", "delta", "eager_delta", "eager_null_dq_acc", "LT2", "LT4"):
        assert hasattr(p.lazy_tensor, name)
    t = _views(p)
    assert t.size(2) == 32 and t.stride(1) == 32 * 64 and t.dtype == p.DType.kFloat16 and t.data_ptr == 0x1000
    prm = p.v3.flash.attn_fwd_params()
    prm.Q = t
    prm.causal_type = 3
    prm.window_left = -2147483647
    assert prm.Q.size(3) == 64 and prm.causal_type == 3 and prm.window_left == -2147483647
    opt = p.v3.flash.attn_options()
    assert opt.force_backend_index == -1 and opt.deterministic is False


def test_version_mismatch_is_invalid_symbol():
    p = load_pyaotriton()
    E = p.hipError_t
    assert p.v3.flash.attn_fwd(p.v3.flash.attn_fwd_params(), 2) == E.hipErrorInvalidSymbol
    assert p.v3.flash.attn_bwd(p.v3.flash.attn_bwd_params(), 5) == E.hipErrorInvalidSymbol


def test_argument_validation_without_device():
    p = load_pyaotriton()
    E = p.hipError_t
    prm = p.v3.flash.attn_fwd_params()
    prm.Sm_scale = 1.0
    prm.dropout_p = 0.0
    prm.causal_type = 0
    prm.window_left = prm.window_right = 0
    prm.philox_offset2 = 0
    # all tensors null -> element type unknown -> rejected before any device query
    assert p.v3.flash.attn_fwd(prm, 3) == E.hipErrorNotSupported
    big = p.T4(0x1000, [1, 1, 16, 1024], [16384, 16384, 1024, 1], p.DType.kFloat16)
    prm.Q = prm.K = prm.V = prm.Out = big
    assert p.v3.flash.attn_fwd(prm, 3) == E.hipErrorNotSupported          # head dim > 512
    ok = _views(p)
    prm.Q = prm.K = prm.V = prm.Out = ok
    prm.causal_type = 7
    assert p.v3.flash.attn_fwd(prm, 3) == E.hipErrorNotSupported          # unknown causal type
    prm.causal_type = 0
    i8 = _views(p, p.DType.kInt8)
    prm.Q = i8
    assert p.v3.flash.attn_fwd(prm, 3) == E.hipErrorNotSupported          # unsupported element type
    prm.Q = ok
    # valid description but no B200 in this process -> the arch gate answers, nothing is launched
    if not torch.cuda.is_available():
        assert p.v3.flash.attn_fwd(prm, 3) == E.hipErrorNoBinaryForGpu
        assert p.v2.flash.check_gpu(p.Stream()) == E.hipErrorNoBinaryForGpu


def test_backward_releases_lazy_tensors_on_error():
    p = load_pyaotriton()
    prm = p.v3.flash.attn_bwd_params()
    like = p.T2(0, [4, 8], [8, 1], p.DType.kFloat32)
    prm.D = p.lazy_tensor.delta(like, 0)
    prm.Sm_scale = 1.0
    prm.dropout_p = 0.0
    prm.causal_type = 0
    prm.window_left = prm.window_right = 0
    prm.philox_offset2 = 0
    # No device: acquire fails to allocate -> invalid value; dispose must still run exactly once
    # (a second call on the same params object must not double free).
    r1 = p.v3.flash.attn_bwd(prm, 6)
    r2 = p.v3.flash.attn_bwd(prm, 6)
    assert r1 != p.hipError_t.hipSuccess and r2 != p.hipError_t.hipSuccess


def test_cabi_rejects_null_and_bad_strides():
    a = cabi.FwdArgs()
    assert cabi.lib().ab200_attn_fwd(None, None) == 1
    a.prob.dtype = cabi.DTYPE_FP16
    a.prob.batch, a.prob.num_head_q, a.prob.num_head_k = 1, 4, 3           # Hq % Hk != 0
    a.prob.max_seqlen_q = a.prob.max_seqlen_k = 16
    a.prob.head_dim_qk = a.prob.head_dim_vo = 64
    assert cabi.lib().ab200_attn_fwd(a, None) == 1
    a.prob.num_head_k = 2
    assert cabi.lib().ab200_attn_fwd(a, None) == 1                          # null q/k/v/out
    for v in (a.q, a.k, a.v, a.out):
        v.ptr = 0x1000
        v.stride[0], v.stride[1], v.stride[2], v.stride[3] = 4096, 1024, 64, 2
        v.size[0], v.size[1], v.size[2], v.size[3] = 1, 4, 16, 64
    assert cabi.lib().ab200_attn_fwd(a, None) == 1                          # innermost stride must be 1
    a.prob.dropout_p = 1.5
    assert cabi.lib().ab200_attn_fwd(a, None) == 1


def test_kernel_family_switch_is_per_thread_and_restorable():
    L = cabi.lib()
    old = L.ab200_set_kernel_family(1)
    assert L.ab200_set_kernel_family(old) == 1
    assert L.ab200_set_kernel_family(99) == old      # out of range: unchanged
    import threading
    seen = []
    L.ab200_set_kernel_family(2)
    t = threading.Thread(target=lambda: seen.append(L.ab200_set_kernel_family(0)))
    t.start(); t.join()
    assert seen == [0]                               # the other thread still had the default
    L.ab200_set_kernel_family(old)


@pytest.mark.parametrize("batch,hk,world", [(4, 32, 8), (1, 8, 8), (1, 8, 4), (3, 5, 4), (2, 3, 8), (8, 16, 2)])
def test_dense_partition_covers_every_unit_once(batch, hk, world):
    seen = np.zeros((batch, hk), dtype=int)
    sizes = []
    for r in range(world):
        n = 0
        for s in sharding.partition_dense(batch, hk, world, r):
            seen[s.b, s.hk_lo:s.hk_hi] += 1
            n += s.hk_hi - s.hk_lo
        sizes.append(n)
    assert (seen == 1).all()
    assert max(sizes) - min(sizes) <= 1


def test_varlen_partition_and_philox_adjustment():
    parts = [sharding.partition_varlen(8, 4, r) for r in range(4)]
    assert [(p[0].hk_lo, p[0].hk_hi) for p in parts] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    adj = sharding.philox_adjustment(sharding.Segment(2, 3, 5), group=4, num_head_q=32, max_seqlen_q=100,
                                     max_seqlen_k=50)
    assert adj == dict(philox_offset2_add=2 * 32 * 100 * 13, philox_head_offset=12, philox_num_head_q=32)


def test_custom_ops_trace_without_a_device():
    """The torch.library operators carry fake implementations and an autograd formula, so a tracer sees
    shapes and dtypes without any kernel (and without a GPU)."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode
    from aotriton_b200 import autograd
    with FakeTensorMode():
        q = torch.empty(2, 8, 128, 64, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 2, 128, 64, dtype=torch.bfloat16, device="cuda")
        v = torch.empty(2, 2, 128, 96, dtype=torch.bfloat16, device="cuda")
        o = autograd.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        assert o.shape == (2, 8, 128, 96) and o.dtype == torch.bfloat16 and o.device.type == "cuda"
    # forward and backward through the registered autograd formula, on meta tensors
    q, k, v = (torch.empty(s, dtype=torch.bfloat16, device="meta", requires_grad=True)
               for s in ((2, 8, 128, 64), (2, 2, 128, 64), (2, 2, 128, 96)))
    o = autograd.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    o.sum().backward()
    assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape
    for bad in (dict(attn_mask=torch.zeros(1, dtype=torch.bool)), dict(attn_mask=torch.zeros(1), is_causal=True)):
        try:
            autograd.scaled_dot_product_attention(torch.zeros(1, 1, 4, 8), torch.zeros(1, 1, 4, 8),
                                                  torch.zeros(1, 1, 4, 8), **bad)
            raise AssertionError("accepted an unsupported mask")
        except ValueError:
            pass


def test_bench_traffic_table_equals_the_profile_summary():
    """roofline.traffic comes from one table in bench.py; it must quote the committed ncu summary."""
    import importlib.util
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("bench_module", root / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    text = (root / "profiles" / "tcgen05_kernels_dense_causal_bf16_B2_H32_S4096_D128.md").read_text()
    numbers = {float(x) for x in re.findall(r"(\d+\.\d+)\s*MB", text)}
    for kern, (rd, wr) in bench.C2_DRAM_TRAFFIC_B2.items():
        assert rd / 1e6 in numbers and wr / 1e6 in numbers, (kern, rd, wr, sorted(numbers))
