"""CPU: the GPU lease that gives every pytest-xdist worker a device of its own
(aotriton_b200/testing/gpu_lease.py; reference: python/pytest-gpu-lease/tests)."""
import multiprocessing as mp
import os
import time

from aotriton_b200.testing.gpu_lease import Lease


def _hold(directory, pool, first, hold_s, out):
    lease = Lease(directory, pool, first=first, timeout=20)
    out.put((os.getpid(), lease.gpu, time.monotonic()))
    time.sleep(hold_s)
    out.put((os.getpid(), -1 - lease.gpu, time.monotonic()))
    lease.release()


def test_leases_are_exclusive_and_wait_for_a_free_gpu(tmp_path):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    pool, workers = 2, 4
    procs = [ctx.Process(target=_hold, args=(tmp_path, pool, w, 0.4, out)) for w in range(workers)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    events = sorted((out.get() for _ in range(2 * workers)), key=lambda e: e[2])
    held = {}
    for pid, code, _ in events:
        if code >= 0:
            assert code < pool and code not in held.values(), f"GPU {code} handed out twice: {events}"
            held[pid] = code
        else:
            assert held.pop(pid) == -1 - code
    assert not held


def test_uncontended_workers_map_to_their_own_index(tmp_path):
    leases = [Lease(tmp_path, 4, first=i, wait=False) for i in range(4)]
    assert [l.gpu for l in leases] == [0, 1, 2, 3]
    try:
        Lease(tmp_path, 4, first=0, wait=False)
        raise AssertionError("a fifth lease on four GPUs must not succeed")
    except TimeoutError:
        pass
    leases[2].release()
    assert Lease(tmp_path, 4, first=0, wait=False).gpu == 2       # the freed one; a crashed holder frees it the same way
    for l in leases:
        l.release()


def test_fixture_modes(pytester=None):
    # pin and not-distributed modes need no lock directory at all
    from aotriton_b200.testing import gpu_lease

    class Cfg:
        pass
    assert gpu_lease._worker(Cfg()) == ("master", 0, 0)
    c = Cfg()
    c.workerinput = {"workerid": "gw5", "workercount": 8}
    assert gpu_lease._worker(c) == ("gw5", 5, 8)
    os.environ["GPU_LEASE_POOL"] = "3"
    try:
        assert gpu_lease._pool_size(8) == 3
    finally:
        del os.environ["GPU_LEASE_POOL"]
