"""pytest plugin: one GPU per pytest-xdist worker on a multi-GPU box.

Counterpart of the reference's `pytest-gpu-lease` (python/pytest-gpu-lease/pytest_gpu_lease/
plugin.py:124-175): running the GPU suite with `pytest -n 8 -p aotriton_b200.testing.gpu_lease`
puts every worker on a GPU of its own, so an 8-GPU node runs eight test processes side by side
without two of them sharing a device.

Mechanism (different from the reference's byte-range locks on one file): a lease directory holds
one lock file per GPU ordinal; a worker takes `flock(LOCK_EX | LOCK_NB)` on the first file it can
get, starting from its own worker number so that an uncontended run maps worker i to GPU i, and
keeps the descriptor open for its whole session.  The kernel drops the lock when the process
ends, however it ends, so a crashed worker never strands a GPU.  When every GPU is taken the
worker waits and retries: there is deliberately no way to put two workers on one device.

Environment:
  GPU_LEASE_PIN=<n>     every worker uses GPU n, nothing is locked (reruns, bisecting a device)
  GPU_LEASE_POOL=<k>    number of GPUs to hand out (default: torch.cuda.device_count(), or the
                        xdist worker count when torch sees no device)
  GPU_LEASE_DIR=<path>  lease directory (default: a directory shared by the workers of the run)

Fixtures: `gpu_id` (int), `gpu_device` ("cuda:<n>"), and the autouse `_bind_leased_gpu`, which makes
the leased GPU torch's current device for tests marked `gpu`.
"""
from __future__ import annotations

import fcntl
import os
import sys
import time
from pathlib import Path

import pytest

RETRY_SECONDS = 0.05


class Lease:
    """An exclusive claim on one GPU ordinal, held through an open, flock'ed file."""

    def __init__(self, directory: Path, pool: int, first: int = 0, wait: bool = True, timeout: float | None = None):
        self.gpu = None
        self._fd = None
        directory.mkdir(parents=True, exist_ok=True)
        deadline = None if timeout is None else time.monotonic() + timeout
        while self.gpu is None:
            for k in range(pool):
                n = (first + k) % pool
                fd = os.open(directory / f"gpu{n}.lock", os.O_RDWR | os.O_CREAT, 0o644)
                try:
                    fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                except OSError:
                    os.close(fd)
                    continue
                self.gpu, self._fd = n, fd
                break
            if self.gpu is None:
                if not wait or (deadline is not None and time.monotonic() > deadline):
                    raise TimeoutError(f"no free GPU among {pool} in {directory}")
                time.sleep(RETRY_SECONDS)

    def release(self):
        if self._fd is not None:
            fcntl.flock(self._fd, fcntl.LOCK_UN)
            os.close(self._fd)
            self._fd = None


def _worker(config) -> tuple[str, int, int]:
    """(label, worker index, worker count); ("master", 0, 0) when the run is not distributed."""
    wi = getattr(config, "workerinput", None)
    if wi is None:
        return "master", 0, 0
    label = wi["workerid"]
    digits = "".join(ch for ch in label if ch.isdigit())
    return label, int(digits or 0), int(wi["workercount"])


def _pool_size(nworkers: int) -> int:
    env = os.getenv("GPU_LEASE_POOL")
    if env is not None:
        return max(1, int(env))
    try:
        import torch
        n = torch.cuda.device_count()
    except Exception:
        n = 0
    return n if n > 0 else max(1, nworkers)


def _say(config, text: str) -> None:
    # session fixtures run under output capture; write past it so that the assignment shows at once
    capman = config.pluginmanager.getplugin("capturemanager")
    suspend = getattr(capman, "global_and_fixture_disabled", None)
    if suspend is None:
        print(text, file=sys.stderr, flush=True)
        return
    with suspend():
        print(text, file=sys.stderr, flush=True)


@pytest.fixture(scope="session")
def gpu_id(request, tmp_path_factory):
    """Ordinal of the GPU this worker owns for its whole session."""
    label, index, nworkers = _worker(request.config)
    pin = os.getenv("GPU_LEASE_PIN")
    if pin is not None:
        _say(request.config, f"[gpu-lease] {label}: GPU {int(pin)} (pinned, no lease)")
        yield int(pin)
        return
    if nworkers == 0:
        _say(request.config, f"[gpu-lease] {label}: GPU 0 (not distributed, no lease)")
        yield 0
        return
    directory = Path(os.getenv("GPU_LEASE_DIR") or tmp_path_factory.getbasetemp().parent / "gpu-lease")
    lease = Lease(directory, _pool_size(nworkers), first=index)
    _say(request.config, f"[gpu-lease] {label}: GPU {lease.gpu} (lease in {directory})")
    try:
        yield lease.gpu
    finally:
        lease.release()


@pytest.fixture(scope="session")
def gpu_device(gpu_id) -> str:
    return f"cuda:{gpu_id}"


@pytest.fixture(autouse=True)
def _bind_leased_gpu(request):
    """Tests marked `gpu` run with the leased GPU as torch's current device (only under xdist or a
    pin: a plain run keeps whatever device is current and takes no lease)."""
    if "gpu" not in request.keywords:
        return
    if getattr(request.config, "workerinput", None) is None and os.getenv("GPU_LEASE_PIN") is None:
        return
    import torch
    if torch.cuda.is_available():
        torch.cuda.set_device(request.getfixturevalue("gpu_id"))
