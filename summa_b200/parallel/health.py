"""Failure detection for multi-rank jobs: heartbeats, a pre-launch guard, a collective watchdog
and the host view of the kernels' bounded waits.

The reference recovers by crash-consistent restart (single-writer lock, sealed generations, a
relaunch supervisor; `summa-train/src/trainer.rs:36-95`, `summa-train/scripts/relaunch.sh:1-140`)
and has no multi-rank runtime. With fused kernels that wait on peers' flags, a rank that has gone
away must be noticed on the HOST before the survivors launch the next kernel:

  * `Heartbeat`: every rank bumps a counter (a file per rank in a shared directory, or a key in a
    `torch.distributed` store) from a daemon thread; `dead_ranks()` lists peers whose counter has
    not moved for `timeout` seconds.
  * `guard(step)`: called between steps, before any launch; raises `RankFailure` naming the dead
    ranks, so no kernel is started that would wait for them.
  * `watched_collective(fn, timeout)`: runs a collective on a helper thread and raises `RankFailure`
    if it does not finish in time (the stand-in for the NCCL watchdog / communicator abort; with a
    process group created with a short timeout the collective itself errors out as well).
  * `device_wait_status()`: reads (and clears) the device error word; bit 2 means a kernel's
    bounded peer-flag wait ran out. The kernel has returned and the context is still usable.

Recovery is the reference's: leave the step loop, let the supervisor relaunch with `--resume` from
the last sealed generation (optimizer state is stored whole, so the rank count may change).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], what: str):
        super().__init__(f"{what}: rank(s) {ranks}")
        self.ranks = ranks


class _FileBackend:
    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    def put(self, rank: int, value: int) -> None:
        tmp = os.path.join(self.dir, f".hb-{rank}.tmp")
        with open(tmp, "w") as f:
            f.write(str(value))
        os.replace(tmp, os.path.join(self.dir, f"hb-{rank}"))

    def get(self, rank: int) -> Optional[int]:
        try:
            with open(os.path.join(self.dir, f"hb-{rank}")) as f:
                return int(f.read().strip() or 0)
        except (OSError, ValueError):
            return None


class _StoreBackend:
    def __init__(self, store, prefix: str = "summa_hb"):
        self.store, self.prefix = store, prefix

    def put(self, rank: int, value: int) -> None:
        self.store.set(f"{self.prefix}/{rank}", str(value))

    def get(self, rank: int) -> Optional[int]:
        try:
            if not self.store.check([f"{self.prefix}/{rank}"]):
                return None
            return int(self.store.get(f"{self.prefix}/{rank}").decode())
        except Exception:
            return None


class Heartbeat:
    def __init__(self, rank: int, world: int, directory: Optional[str] = None, store=None, interval: float = 0.2,
                 timeout: float = 2.0):
        if (directory is None) == (store is None):
            raise ValueError("give exactly one of `directory` and `store`")
        self.rank, self.world, self.interval, self.timeout = rank, world, interval, timeout
        self.backend = _FileBackend(directory) if directory is not None else _StoreBackend(store)
        self._beat = 0
        self._stop = threading.Event()
        self._seen = {r: (None, time.monotonic()) for r in range(world)}    # rank -> (last value, when it changed)
        self._thread: Optional[threading.Thread] = None
        self.left = False

    # ---- own pulse
    def start(self) -> "Heartbeat":
        self.backend.put(self.rank, self._beat)
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            self._beat += 1
            try:
                self.backend.put(self.rank, self._beat)
            except Exception:
                pass

    def leave(self) -> None:
        """Orderly departure between steps: the pulse stops and the counter is set to -1, which
        peers treat as gone at their next `guard`, without waiting for the timeout."""
        self.stop()
        self.left = True
        try:
            self.backend.put(self.rank, -1)
        except Exception:
            pass

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)

    # ---- peers
    def dead_ranks(self) -> List[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self.backend.get(r)
            last, when = self._seen[r]
            if v == -1:
                dead.append(r)
                continue
            if v is not None and v != last:
                self._seen[r] = (v, now)
            elif now - when > self.timeout:
                dead.append(r)
        return dead

    def guard(self, step: int = -1) -> None:
        """Call between steps, before launching anything that waits on a peer."""
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead, f"peer heartbeat lost before step {step}")


def watched_collective(fn: Callable[[], object], timeout: float, what: str = "collective"):
    """Runs `fn` (a blocking collective) on a helper thread; `RankFailure` if it has not returned
    after `timeout` seconds or if it raised (a process group with a short timeout raises by itself)."""
    box = {}

    def run():
        try:
            box["value"] = fn()
        except BaseException as e:      # the collective's own timeout / abort
            box["error"] = e

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(timeout)
    if t.is_alive():
        raise RankFailure([], f"{what} did not finish within {timeout:.1f} s")
    if "error" in box:
        raise RankFailure([], f"{what} failed ({type(box['error']).__name__}: {box['error']})")
    return box.get("value")


def device_wait_status() -> dict:
    """Host view of the kernels' bounded waits (reads and clears the device error word)."""
    from ..ops import native
    word = native.read_error_flag()
    return {"word": word, "mbarrier_timeout": bool(word & 1), "peer_wait_timeout": bool(word & 2),
            "bad_argument": bool(word & 4)}
