"""Failure detection and host-side fault injection.

The reference has neither: its CUDA / NCCL error checks abort the process
(lib/kernels/include/kernels/device.h:88-110, lib/kernels/include/kernels/nccl.h:9-20).  Here

* device-side waits on peers are bounded; when one runs out the kernel writes a code to a status word and
  returns, and :meth:`DistContext.check_status` turns it into :class:`CommTimeoutError` on the host;
* ranks publish heartbeats through the ``torch.distributed`` store; :class:`HeartbeatMonitor` reports ranks whose
  heartbeat is older than a deadline, so survivors learn of a lost rank *before* their next launch;
* :class:`FaultInjector` makes failures on the host only (raise, stall, drop a heartbeat, corrupt a file) --
  nothing here ever faults, traps or hangs a GPU.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


class CommTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer expired."""


class RankFailure(RuntimeError):
    """One or more ranks stopped publishing heartbeats."""

    def __init__(self, ranks: List[int]):
        super().__init__(f"ranks {ranks} are not responding")
        self.ranks = ranks


class InjectedFault(RuntimeError):
    """Raised by FaultInjector at a configured point."""


class HeartbeatMonitor:
    """Heartbeats over a key-value store (``torch.distributed.TCPStore`` / ``HashStore`` / any object with
    ``set(key, value)`` and ``get(key)``).  ``beat()`` is called once per step; ``dead_ranks()`` lists ranks whose
    last beat is older than ``timeout_s`` (or that never beat after ``grace_s``)."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 10.0, grace_s: float = 30.0, prefix: str = "hb"):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.timeout_s, self.grace_s, self.prefix = timeout_s, grace_s, prefix
        self.start = time.time()
        self.suppressed = False  # set by the fault injector to emulate a silent rank

    def beat(self, step: int = 0):
        if self.suppressed:
            return
        self.store.set(f"{self.prefix}/{self.rank}", f"{time.time():.6f}:{step}")

    def last_beat(self, rank: int) -> Optional[float]:
        key = f"{self.prefix}/{rank}"
        try:
            # TCPStore.get blocks until the key exists; ask first where the store can say
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            v = self.store.get(key)
        except Exception:
            return None
        if isinstance(v, bytes):
            v = v.decode()
        try:
            return float(str(v).split(":")[0])
        except ValueError:
            return None

    def dead_ranks(self, now: Optional[float] = None) -> List[int]:
        now = time.time() if now is None else now
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            t = self.last_beat(r)
            if t is None:
                if now - self.start > self.grace_s:
                    dead.append(r)
            elif now - t > self.timeout_s:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)


class DictStore:
    """In-process store with the TCPStore surface used here; lets the monitor be tested without sockets."""

    def __init__(self):
        self._d: Dict[str, str] = {}
        self._lock = threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = v

    def get(self, k):
        with self._lock:
            if k not in self._d:
                raise KeyError(k)
            return self._d[k]


@dataclass
class FaultInjector:
    """Host-side fault plan: ``{"step": n, "kind": ...}`` entries fire when ``maybe_fail(step)`` reaches them.

    kinds: ``raise`` (throw InjectedFault), ``stall`` (sleep ``seconds``), ``exit`` (leave the process between
    steps with status ``code``), ``silence`` (stop heartbeats), ``corrupt`` (flip bytes of ``path``)."""
    plan: List[dict] = field(default_factory=list)
    rank: int = 0
    monitor: Optional[HeartbeatMonitor] = None
    fired: List[dict] = field(default_factory=list)

    def maybe_fail(self, step: int):
        for f in self.plan:
            if f.get("step") != step or f.get("rank", self.rank) != self.rank or f in self.fired:
                continue
            self.fired.append(f)
            kind = f.get("kind", "raise")
            if kind == "raise":
                raise InjectedFault(f"injected fault at step {step} on rank {self.rank}")
            if kind == "stall":
                time.sleep(float(f.get("seconds", 1.0)))
            elif kind == "exit":
                os._exit(int(f.get("code", 17)))
            elif kind == "silence" and self.monitor is not None:
                self.monitor.suppressed = True
            elif kind == "corrupt":
                corrupt_file(f["path"], int(f.get("offset", 64)), int(f.get("nbytes", 16)))


def corrupt_file(path: str, offset: int = 64, nbytes: int = 16):
    size = os.path.getsize(path)
    offset = min(offset, max(size - nbytes, 0))
    with open(path, "r+b") as fh:
        fh.seek(offset)
        data = bytearray(fh.read(nbytes))
        for i in range(len(data)):
            data[i] ^= 0xFF
        fh.seek(offset)
        fh.write(bytes(data))


def run_with_recovery(step_fn: Callable[[int], None], num_steps: int, *, save_fn: Callable[[int], None],
                      restore_fn: Callable[[], int], checkpoint_every: int = 1, max_restarts: int = 3,
                      recoverable=(InjectedFault, CommTimeoutError, RankFailure)) -> dict:
    """Drive ``step_fn`` for ``num_steps`` steps; on a recoverable failure restore the last checkpoint and continue.
    Returns ``{"restarts": n, "steps_run": total step invocations}``."""
    restarts, runs, step = 0, 0, 0
    while step < num_steps:
        try:
            step_fn(step)
            runs += 1
            step += 1
            if step % checkpoint_every == 0:
                save_fn(step)
        except recoverable:
            restarts += 1
            if restarts > max_restarts:
                raise
            step = restore_fn()
    return {"restarts": restarts, "steps_run": runs}


class CollectiveWatchdog:
    """Bounds the library collectives (NCCL on GPUs, gloo on the host) the way the device-side waits bound the
    peer-memory kernels: the process group is created with a short timeout and asynchronous error handling, a
    collective that a peer never joins then raises instead of blocking for the default half hour, and the failure
    is turned into ``RankFailure`` after the communicator has been aborted so that no later call can block on it.

        wd = CollectiveWatchdog(timeout_s=5)
        wd.init_process_group("nccl", rank=r, world_size=w, device_id=dev)   # or wd.adopt(existing default group)
        wd.run(dist.all_reduce, t)                                            # raises RankFailure on a dead peer
    """

    def __init__(self, timeout_s: float = 30.0, monitor: Optional[HeartbeatMonitor] = None):
        self.timeout_s = float(timeout_s)
        self.monitor = monitor
        self.aborted = False

    def init_process_group(self, backend: str, **kw):
        import datetime

        import torch.distributed as dist
        if backend == "nccl":
            # surface a collective that timed out or failed as an exception in the calling thread
            os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # a rank that dies while bound to a multicast object faults its peers
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=self.timeout_s), **kw)
        return self

    def abort(self):
        """Tear the communicator down without waiting for outstanding collectives."""
        import torch.distributed as dist
        if self.aborted or not dist.is_initialized():
            return
        self.aborted = True
        try:
            pg = dist.distributed_c10d._get_default_group()
            for dev in ("cuda", "cpu"):
                try:
                    be = pg._get_backend(__import__("torch").device(dev))
                except Exception:
                    continue
                ab = getattr(be, "abort", None) or getattr(be, "_abort", None)
                if ab is not None:
                    ab()
        except Exception:
            pass

    def run(self, fn: Callable, *args, **kw):
        """Run one collective; a timeout or communicator error becomes RankFailure naming the ranks the heartbeat
        monitor (if any) holds for dead."""
        try:
            out = fn(*args, **kw)
            work = out if hasattr(out, "wait") else None
            if work is not None:
                work.wait()
            return out
        except InjectedFault:
            raise
        except Exception as e:  # torch raises RuntimeError / DistBackendError with backend-specific text
            dead = self.monitor.dead_ranks() if self.monitor is not None else []
            self.abort()
            raise RankFailure(dead) from e
