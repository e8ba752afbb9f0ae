"""Restart loop around a training command: run it until the final checkpoint exists.

Same job as the ``while true; do [ -f DONE_<max> ] && break; mpirun … -y 1; sleep 1; done`` loop of the reference's
launch scripts (scripts/run_gpt2_124M.sh:36-63), as a command:

    python -m llm_kittens_b200.cli.supervise --out log124M --final-step 2000 [--max-restarts 20] -- \\
        python -m torch.distributed.run --nproc-per-node 8 -m llm_kittens_b200.cli.train_gpt2cu ... -o log124M -x 2000

The command is run as given the first time and with ``-y 1`` appended afterwards (resume from the newest checkpoint
with a ``DONE_*`` marker). A run that ends with exit code 0 and the final marker present ends the loop; any other
outcome — a crash, the watchdog's exit code 75 (``runtime/watchdog.py``) — is followed by a restart until
``--max-restarts`` is used up. Launch metadata and every attempt's outcome go to ``<out>/run.log``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time

from ..runtime.watchdog import EXIT_RESUME
from ..utils import formats


def final_marker(out_dir: str, final_step: int) -> str:
    return formats.checkpoint_paths(out_dir, final_step, 0)[2]


def supervise(cmd: list[str], out_dir: str, final_step: int, max_restarts: int = 20, sleep_s: float = 1.0,
              run=subprocess.call) -> int:
    """Returns 0 once the final ``DONE_*`` marker exists, else the last exit code (or 1)."""
    os.makedirs(out_dir, exist_ok=True)
    log = os.path.join(out_dir, "run.log")
    marker = final_marker(out_dir, final_step)
    with open(log, "a") as f:
        f.write(f"supervise: final step {final_step}, command: {' '.join(cmd)}\n")
    rc = 1
    for attempt in range(max_restarts + 1):
        if os.path.exists(marker):
            return 0
        argv = list(cmd) if attempt == 0 and formats.find_max_step(out_dir) < 0 else list(cmd) + ["-y", "1"]
        t0 = time.time()
        rc = run(argv)
        why = "resume requested by the watchdog" if rc == EXIT_RESUME else ("ok" if rc == 0 else "failed")
        with open(log, "a") as f:
            f.write(f"attempt {attempt}: exit code {rc} ({why}) after {time.time() - t0:.1f} s, "
                    f"newest checkpoint {formats.find_max_step(out_dir)}\n")
        if os.path.exists(marker):
            return 0
        time.sleep(sleep_s)
    return rc if rc != 0 else 1


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--" not in argv:
        print(__doc__)
        return 2
    split = argv.index("--")
    ap = argparse.ArgumentParser(prog="llm_kittens_b200.cli.supervise")
    ap.add_argument("--out", required=True, help="the trainer's -o directory")
    ap.add_argument("--final-step", type=int, required=True, help="the trainer's -x value")
    ap.add_argument("--max-restarts", type=int, default=20)
    args = ap.parse_args(argv[:split])
    return supervise(argv[split + 1:], args.out, args.final_step, args.max_restarts)


if __name__ == "__main__":
    sys.exit(main())
