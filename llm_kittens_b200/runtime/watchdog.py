"""Host-side failure detection: a step deadline and peer heartbeats.

The reference's failure handling is crash-and-restart: every error path exits (llmc/cuda_common.h:49-55,
llmc/zero.cuh:36-55) and the launch scripts restart the trainer with ``-y 1`` until the final ``DONE_*`` marker
exists (scripts/run_gpt2_124M.sh:36-63); a rank that hangs inside a collective hangs the job. This module adds
what that scheme lacks, entirely on the host (no kernel is involved, nothing can fault or hang a GPU):

* every rank runs a daemon thread; the training loop calls :meth:`Watchdog.beat` once per step;
* if the own step takes longer than ``deadline_s`` the thread reports it and ends the process with
  :data:`EXIT_RESUME` (75, EX_TEMPFAIL), which :mod:`llm_kittens_b200.cli.supervise` maps to "restart with -y 1";
* with a ``torch.distributed`` key-value store, each beat also publishes ``hb/<rank> = step`` and the thread
  watches the other ranks: a peer whose heartbeat is older than ``deadline_s`` (it crashed, or hangs before its
  next collective) ends this process the same way, instead of leaving it blocked in the next collective.

* :meth:`Watchdog.enter_step` is a bounded host-side rendezvous at a step boundary (``LLMK_WATCHDOG_RENDEZVOUS=1`` in
  the trainers): a peer that left between steps is noticed before this rank launches its next kernel or collective.

The in-kernel waits of the fused communication kernels are bounded separately (status word, see ``ops/_native``);
the watchdog covers what happens between kernels and inside library collectives.
"""
from __future__ import annotations

import os
import sys
import threading
import time
from typing import Callable

EXIT_RESUME = 75


def store_from_env(rank: int, world: int, port_offset: int = 1):
    """A TCPStore beside the process group's rendezvous (MASTER_ADDR, MASTER_PORT + offset), hosted by rank 0."""
    from datetime import timedelta

    import torch.distributed as dist

    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
    return dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=timedelta(seconds=60), wait_for_workers=False)


class Watchdog:
    def __init__(self, rank: int, world: int, deadline_s: float, store=None, poll_s: float | None = None,
                 on_failure: Callable[[str], None] | None = None, clock: Callable[[], float] = time.monotonic):
        self.rank, self.world, self.deadline_s = rank, world, float(deadline_s)
        self.store = store
        self.poll_s = poll_s if poll_s is not None else max(0.05, min(1.0, self.deadline_s / 4))
        self.on_failure = on_failure or self._exit
        self.clock = clock
        self._last_beat = clock()
        self._step = -1
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self.failure: str | None = None
        self._peer_seen: dict[int, tuple[str, float]] = {}   # rank -> (last value, local time it changed)

    # ------------------------------------------------------------------ called by the training loop
    def beat(self, step: int) -> None:
        self._step = step
        self._last_beat = self.clock()
        if self.store is not None:
            try:
                self.store.set(f"hb/{self.rank}", f"{step}")
            except Exception as e:   # the store's host (rank 0) is gone
                self._fail(f"rank {self.rank}: heartbeat store unreachable ({type(e).__name__})")

    def enter_step(self, step: int, timeout_s: float | None = None) -> bool:
        """Host-side rendezvous at a step boundary, to be called when none of this rank's kernels or collectives is in
        flight: publishes ``enter/<rank> = step`` and waits (bounded) until every peer has published a step >= ``step``.
        A peer that left or hangs is thus noticed BEFORE the next kernel or collective is launched. Returns True when
        all peers arrived; otherwise the failure handler runs (default: exit with :data:`EXIT_RESUME`) and False is
        returned."""
        if self.store is None or self.world == 1:
            return True
        timeout_s = self.deadline_s if timeout_s is None else timeout_s
        try:
            self.store.set(f"enter/{self.rank}", str(step))
            t0 = self.clock()
            missing = [r for r in range(self.world) if r != self.rank]
            while True:
                missing = [r for r in missing
                           if not (self.store.check([f"enter/{r}"]) and int(self.store.get(f"enter/{r}").decode()) >= step)]
                if not missing:
                    self._last_beat = self.clock()
                    return True
                if self.clock() - t0 > timeout_s:
                    break
                self._sleep(min(0.01, self.poll_s))
        except Exception as e:
            self._fail(f"rank {self.rank}: heartbeat store unreachable at step {step} ({type(e).__name__})")
            return False
        self._fail(f"rank {self.rank}: rank(s) {missing} did not enter step {step} within {timeout_s:.1f} s")
        return False

    _sleep = staticmethod(time.sleep)

    def start(self) -> None:
        self._last_beat = self.clock()
        now = self.clock()
        for r in range(self.world):
            self._peer_seen[r] = ("", now)
        self._thread = threading.Thread(target=self._run, name="llmk-watchdog", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    # ------------------------------------------------------------------ checks (also callable directly, for tests)
    def check_once(self) -> str | None:
        """One evaluation of the rules; returns the failure text, or None."""
        now = self.clock()
        if now - self._last_beat > self.deadline_s:
            return f"rank {self.rank}: step {self._step} exceeded the deadline of {self.deadline_s:.1f} s"
        if self.store is not None:
            for r in range(self.world):
                if r == self.rank:
                    continue
                try:
                    val = self.store.get(f"hb/{r}").decode() if self.store.check([f"hb/{r}"]) else ""
                except Exception as e:
                    return f"rank {self.rank}: heartbeat store unreachable ({type(e).__name__})"
                last, since = self._peer_seen.get(r, ("", now))
                if val != last:
                    self._peer_seen[r] = (val, now)
                elif now - since > self.deadline_s:
                    return f"rank {self.rank}: no heartbeat from rank {r} for {now - since:.1f} s (last step {last or 'none'})"
        return None

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            msg = self.check_once()
            if msg is not None:
                self._fail(msg)
                return

    def _fail(self, msg: str) -> None:
        if self.failure is None:
            self.failure = msg
            self.on_failure(msg)

    @staticmethod
    def _exit(msg: str) -> None:
        sys.stderr.write(f"[watchdog] {msg}; exiting with code {EXIT_RESUME} so that the run resumes from its last checkpoint\n")
        sys.stderr.flush()
        os._exit(EXIT_RESUME)
