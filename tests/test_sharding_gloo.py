"""CPU, two gloo ranks: the batch x head partition used for multi-GPU runs.  Each rank computes
its shard with the oracle (standing in for the device kernels), the shards are gathered, and the
result must equal the unsharded computation -- including the dropout mask, which depends on the
shard's position through philox_offset2 / philox_head_offset / philox_num_head_q."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    from aotriton_b200 import sharding
    from oracle import attention as A
    from oracle import philox
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                      # same full problem on every rank
        B, Hq, Hk, S, D, p = 3, 6, 3, 40, 16, 0.25
        G = Hq // Hk
        q = torch.randn(B, Hq, S, D); k = torch.randn(B, Hk, S, D); v = torch.randn(B, Hk, S, D)
        do = torch.randn(B, Hq, S, D)
        seed, base = 77, 1234
        mask = A.window_mask(S, S, 3, A.TOP_LEFT, A.TOP_LEFT)
        out = torch.zeros(B, Hq, S, D); dk = torch.zeros(B, Hk, S, D)
        for seg in sharding.partition_dense(B, Hk, world, rank):
            adj = sharding.philox_adjustment(seg, G, Hq, S, S)
            qs, ks = sharding.slice_dense(seg, G, q, k)
            dos, vs = sharding.slice_dense(seg, G, do, v)
            nh = qs.shape[1]
            # keep mask of the shard exactly as a kernel given the adjusted Philox fields would draw it:
            # batch index restarts at 0, heads are offset, the host offset carries the batch position
            keep = torch.stack([torch.from_numpy(philox.keep_mask(
                seed, base + adj["philox_offset2_add"], 0, h + adj["philox_head_offset"],
                adj["philox_num_head_q"], S, S, S, S, p)) for h in range(nh)])[None]
            r = A.attention(qs, ks, vs, sm_scale=0.25, mask=mask, keep=keep, dropout_p=p, dout=dos)
            sharding.slice_dense(seg, G, out).copy_(r.out)
            _, dks = sharding.slice_dense(seg, G, do, dk)
            dks.copy_(r.dk)
        dist.all_reduce(out)                      # shards are disjoint, zeros elsewhere
        dist.all_reduce(dk)
        if rank == 0:
            keep_full = A.keep_masks(seed, base, B, Hq, S, S, p)
            ref = A.attention(q, k, v, sm_scale=0.25, mask=mask, keep=keep_full, dropout_p=p, dout=do)
            results.put((float((out - ref.out).abs().max()), float((dk - ref.dk).abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_partition_reproduces_unsharded_result():
    ctx = mp.get_context("spawn")
    results = ctx.SimpleQueue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(150)
        assert pr.exitcode == 0
    err_out, err_dk = results.get()
    assert err_out < 1e-5 and err_dk < 1e-5
