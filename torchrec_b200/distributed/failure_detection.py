"""Host-side failure detection for one-process-per-GPU jobs.

Three pieces, all on the host, none of which touches a device:

* ``Heartbeat`` -- every rank bumps a counter in the rendezvous store from a daemon thread; ``silent_ranks`` lists peers whose
  counter has not moved for ``max_silence_s``.
* ``FailureBoard`` -- a rank that catches an exception in its step posts it to the store *before* it leaves; peers call
  ``raise_if_peer_failed`` before their next launch and leave between steps too, with no collective in flight.
* ``guarded_step`` -- wraps a step with both, and turns a collective that ran into the process group's timeout into the same
  ``PeerFailure`` error.

Device-side waits of this framework (peer barrier, GEMM pipeline barriers) are time-bounded and report through an error word that
the host reads (``PeerGroup.check_error``, ``gemm_error_status``); ``raise_on_device_status`` folds those into the same path.

The reference has no counterpart besides the elastic-launch ``@record`` wrapper of its examples and the pipeline's
``PipelineState`` (``torchrec/distributed/train_pipeline/types.py:91``).
"""
from __future__ import annotations

import threading
import time
from typing import Any, Callable, Dict, List, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    """Another rank failed or went silent; ``ranks`` lists them, ``reasons`` what they reported."""

    def __init__(self, ranks: List[int], reasons: Optional[Dict[int, str]] = None) -> None:
        self.ranks = ranks
        self.reasons = reasons or {}
        super().__init__(f"peer ranks {ranks} failed: {self.reasons}" if self.reasons else f"peer ranks {ranks} are silent")


class Heartbeat:
    def __init__(self, store: dist.Store, rank: int, world_size: int, interval_s: float = 0.5, prefix: str = "trb_hb") -> None:
        self._store, self._rank, self._world, self._interval, self._prefix = store, rank, world_size, interval_s, prefix
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_seen: Dict[int, tuple] = {}

    def _key(self, rank: int) -> str:
        return f"{self._prefix}/{rank}"

    def start(self) -> "Heartbeat":
        self._store.add(self._key(self._rank), 1)

        def beat() -> None:
            while not self._stop.wait(self._interval):
                if not self._paused.is_set():
                    try:
                        self._store.add(self._key(self._rank), 1)
                    except Exception:
                        return  # the store is gone: the job is being torn down

        self._thread = threading.Thread(target=beat, name="trb-heartbeat", daemon=True)
        self._thread.start()
        return self

    def pause(self) -> None:
        """Stop beating without stopping the thread (what a hung host thread looks like from outside); for tests."""
        self._paused.set()

    def resume(self) -> None:
        self._paused.clear()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self._interval + 1)

    def silent_ranks(self, max_silence_s: float) -> List[int]:
        """Peers whose counter did not change for longer than ``max_silence_s`` (measured on this rank's clock)."""
        now = time.monotonic()
        silent = []
        for r in range(self._world):
            if r == self._rank:
                continue
            try:
                count = int(self._store.add(self._key(r), 0))
            except Exception:
                silent.append(r)
                continue
            seen = self._last_seen.get(r)
            if seen is None or seen[0] != count:
                self._last_seen[r] = (count, now)
            elif now - seen[1] > max_silence_s:
                silent.append(r)
        return silent

    def raise_if_silent(self, max_silence_s: float) -> None:
        s = self.silent_ranks(max_silence_s)
        if s:
            raise PeerFailure(s)


class FailureBoard:
    def __init__(self, store: dist.Store, rank: int, world_size: int, prefix: str = "trb_fail") -> None:
        self._store, self._rank, self._world, self._prefix = store, rank, world_size, prefix
        self._store.add(f"{prefix}/count", 0)

    def post(self, reason: str) -> None:
        self._store.set(f"{self._prefix}/reason/{self._rank}", reason[:1000])
        self._store.add(f"{self._prefix}/flag/{self._rank}", 1)
        self._store.add(f"{self._prefix}/count", 1)

    def failed_ranks(self) -> Dict[int, str]:
        if int(self._store.add(f"{self._prefix}/count", 0)) == 0:
            return {}
        out: Dict[int, str] = {}
        for r in range(self._world):
            if r != self._rank and int(self._store.add(f"{self._prefix}/flag/{r}", 0)) > 0:
                out[r] = self._store.get(f"{self._prefix}/reason/{r}").decode("utf-8", "replace")
        return out

    def raise_if_peer_failed(self) -> None:
        failed = self.failed_ranks()
        if failed:
            raise PeerFailure(sorted(failed), failed)


def raise_on_device_status(status: int, what: str) -> None:
    """Turn the error word of a bounded device-side wait into a host exception (0 = no error)."""
    if status != 0:
        raise RuntimeError(f"{what}: a device-side wait ran out (status {status}); the step's results are invalid")


def guarded_step(step: Callable[[], Any], board: FailureBoard, heartbeat: Optional[Heartbeat] = None, max_silence_s: float = 30.0) -> Any:
    """Check the peers, run ``step``, publish this rank's failure if it raises.  A collective that ran into the process-group
    timeout because a peer left is reported as ``PeerFailure`` when the board or the heartbeat names the peer."""
    board.raise_if_peer_failed()
    if heartbeat is not None:
        heartbeat.raise_if_silent(max_silence_s)
    try:
        return step()
    except PeerFailure:
        raise
    except BaseException as e:
        failed = board.failed_ranks()
        if failed:
            raise PeerFailure(sorted(failed), failed) from e
        board.post(f"{type(e).__name__}: {e}")
        raise


def world_store(pg: Optional[dist.ProcessGroup] = None) -> dist.Store:
    """The rendezvous store of the default process group, namespaced for this module."""
    store = dist.distributed_c10d._get_default_store()
    return dist.PrefixStore("torchrec_b200_failure_detection", store)
