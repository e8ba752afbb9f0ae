"""Host-side failure detection, restart loop and NVTX ranges — no GPU, no kernel: the failures are a step that
never ends (fake clock), a peer that stops publishing heartbeats, and a trainer command that exits early."""
import os
import subprocess
import sys
import textwrap

from llm_kittens_b200.cli import supervise
from llm_kittens_b200.runtime.watchdog import EXIT_RESUME, Watchdog
from llm_kittens_b200.utils import formats, nvtx


class FakeStore:
    def __init__(self):
        self.kv = {}

    def set(self, k, v):
        self.kv[k] = v.encode()

    def get(self, k):
        return self.kv[k]

    def check(self, keys):
        return all(k in self.kv for k in keys)


def test_watchdog_step_deadline_with_fake_clock():
    now = [0.0]
    failures = []
    wd = Watchdog(0, 1, deadline_s=10.0, on_failure=failures.append, clock=lambda: now[0])
    wd.beat(0)
    now[0] = 9.0
    assert wd.check_once() is None
    wd.beat(1)
    now[0] = 18.0
    assert wd.check_once() is None          # 9 s since the last beat
    now[0] = 19.5
    msg = wd.check_once()
    assert msg is not None and "step 1 exceeded the deadline" in msg


def test_watchdog_notices_a_silent_peer():
    now = [0.0]
    store = FakeStore()
    wd = Watchdog(0, 3, deadline_s=5.0, store=store, on_failure=lambda m: None, clock=lambda: now[0])
    wd.start()
    wd.stop()                                # the thread is not needed: the rules are evaluated by hand
    for t in range(1, 5):                    # ranks 1 and 2 beat every second ...
        now[0] = float(t)
        wd.beat(t)
        store.set("hb/1", str(t))
        store.set("hb/2", str(t))
        assert wd.check_once() is None
    for t in range(5, 12):                   # ... then rank 2 stops
        now[0] = float(t)
        wd.beat(t)
        store.set("hb/1", str(t))
        msg = wd.check_once()
        if msg is not None:
            break
    assert msg is not None and "no heartbeat from rank 2" in msg and "last step 4" in msg
    assert 9.0 <= now[0] <= 10.5             # 5 s after its last change at t = 4


def test_watchdog_processes_exit_with_resume_code_when_a_rank_goes_silent(tmp_path):
    """Two real processes and a TCPStore on 127.0.0.1: rank 1 stops after three steps (it sleeps, as a rank stuck
    outside any kernel would); rank 0 keeps stepping and must leave with exit code 75 within a few seconds."""
    script = textwrap.dedent("""
        import os, sys, time
        from llm_kittens_b200.runtime.watchdog import Watchdog, store_from_env
        rank = int(sys.argv[1])
        wd = Watchdog(rank, 2, deadline_s=1.5, store=store_from_env(rank, 2))
        wd.start()
        for step in range(200):
            wd.beat(step)
            time.sleep(0.05)
            if rank == 1 and step == 3:
                time.sleep(4.0)              # silent, but still alive: its own deadline fires as well
        sys.exit(0)
    """)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29650 + os.getpid() % 200),
               PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    procs = [subprocess.Popen([sys.executable, "-c", script, str(r)], env=env, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=60) for p in procs]
    assert procs[0].returncode == EXIT_RESUME, outs[0][1]
    assert "no heartbeat from rank 1" in outs[0][1]
    assert procs[1].returncode == EXIT_RESUME and "exceeded the deadline" in outs[1][1]


def test_supervisor_restarts_with_resume_flag_until_the_final_marker(tmp_path):
    out = str(tmp_path / "log")
    calls = []

    def fake_trainer(argv):
        calls.append(list(argv))
        os.makedirs(out, exist_ok=True)
        if len(calls) == 1:                  # first attempt: a checkpoint at step 10, then the watchdog's exit
            open(formats.checkpoint_paths(out, 10, 0)[2], "w").close()
            return EXIT_RESUME
        if len(calls) == 2:                  # second attempt crashes without progress
            return 1
        open(formats.checkpoint_paths(out, 20, 0)[2], "w").close()
        return 0

    rc = supervise.supervise(["trainer", "-x", "20"], out, final_step=20, max_restarts=5, sleep_s=0.0, run=fake_trainer)
    assert rc == 0 and len(calls) == 3
    assert calls[0] == ["trainer", "-x", "20"]
    assert calls[1][-2:] == ["-y", "1"] and calls[2][-2:] == ["-y", "1"]
    text = open(os.path.join(out, "run.log")).read()
    assert "attempt 0: exit code 75 (resume requested by the watchdog)" in text and "newest checkpoint 10" in text
    assert "attempt 1: exit code 1 (failed)" in text and "attempt 2: exit code 0 (ok)" in text
    # the restarts are bounded
    assert supervise.supervise(["trainer"], str(tmp_path / "never"), 5, max_restarts=2, sleep_s=0.0, run=lambda a: 3) == 3


def test_nvtx_ranges_nest_and_can_be_switched_off():
    nvtx.set_enabled(True)
    try:
        with nvtx.nvtx_range("step"):
            with nvtx.nvtx_range("forward"):
                pass
            with nvtx.nvtx_range("backward_and_reduce"):
                pass
        assert nvtx.recent()[-3:] == [("step", 0), ("forward", 1), ("backward_and_reduce", 1)]
        n = len(nvtx.recent())
        nvtx.set_enabled(False)
        with nvtx.nvtx_range("ignored"):
            pass
        assert len(nvtx.recent()) == n
    finally:
        nvtx.set_enabled(False)


def test_step_rendezvous_notices_a_rank_that_left_before_anything_is_launched():
    now = [0.0]
    store = FakeStore()
    failures = []
    wd = Watchdog(0, 2, deadline_s=2.0, store=store, on_failure=failures.append, clock=lambda: now[0])
    wd._sleep = lambda s: now.__setitem__(0, now[0] + s)      # waiting advances the fake clock
    store.set("enter/1", "3")
    assert wd.enter_step(3) and not failures                  # the peer is already there
    assert wd.enter_step(2) and not failures
    assert not wd.enter_step(4)                               # the peer never publishes step 4
    assert failures and "rank(s) [1] did not enter step 4" in failures[0]
    assert 2.0 <= now[0] <= 2.2
