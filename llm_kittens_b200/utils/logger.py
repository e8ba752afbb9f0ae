"""Rank-0 ``main.log`` writer with the line formats that log validators parse
(``s:%d tel:%.4f``, ``s:%d eval:%.4f``, ``s:%d trl:%.4f lr:%.6f norm:%.2f``; reference llmc/logger.h:19-56),
plus the parsers used to validate and compare training logs."""
from __future__ import annotations

import os
import re


def _f32(x: float) -> float:
    """The value as the reference's ``float`` arguments carry it (float32), so both writers print the same digits."""
    import struct

    return struct.unpack("f", struct.pack("f", float(x)))[0]


class Logger:
    """Writes through the C++ host library (``llmk_logger_*``) when it is available, else with Python file I/O; the
    bytes are the same."""

    def __init__(self, log_dir: str | None, process_rank: int = 0, resume: bool = False, native: bool = True):
        self.active = log_dir is not None and process_rank == 0
        self.path = None
        self._lib = self._h = None
        if self.active:
            os.makedirs(log_dir, exist_ok=True)
            self.path = os.path.join(log_dir, "main.log")
            if native:
                try:
                    from . import hostlib

                    self._lib = hostlib.lib()
                    self._h = self._lib.llmk_logger_create(log_dir.encode(), 0, int(resume))
                except Exception:
                    self._lib = self._h = None
            if self._h is None and not resume:
                open(self.path, "w").close()

    def _append(self, line: str) -> None:
        if self.active:
            with open(self.path, "a") as f:
                f.write(line)

    def log_eval(self, step: int, val: float) -> None:
        if self._h is not None:
            self._lib.llmk_logger_eval(self._h, step, val)
        else:
            self._append("s:%d eval:%.4f\n" % (step, _f32(val)))

    def log_val(self, step: int, val_loss: float) -> None:
        if self._h is not None:
            self._lib.llmk_logger_val(self._h, step, val_loss)
        else:
            self._append("s:%d tel:%.4f\n" % (step, _f32(val_loss)))

    def log_train(self, step: int, train_loss: float, learning_rate: float, grad_norm: float) -> None:
        if self._h is not None:
            self._lib.llmk_logger_train(self._h, step, train_loss, learning_rate, grad_norm)
        else:
            self._append("s:%d trl:%.4f lr:%.6f norm:%.2f\n" % (step, _f32(train_loss), _f32(learning_rate), _f32(grad_norm)))

    def __del__(self):
        try:
            if self._h is not None:
                self._lib.llmk_logger_destroy(self._h)
        except Exception:
            pass


_LINE = re.compile(r"^s:(\d+) (.*)$")


def parse_log(path: str) -> dict:
    """Return ``{"train": {step: (loss, lr, norm)}, "val": {step: loss}, "eval": {step: acc}}``."""
    out = {"train": {}, "val": {}, "eval": {}}
    with open(path) as f:
        for line in f:
            m = _LINE.match(line.strip())
            if not m:
                continue
            step = int(m.group(1))
            fields = dict(kv.split(":", 1) for kv in m.group(2).split())
            if "trl" in fields:
                out["train"][step] = (float(fields["trl"]), float(fields.get("lr", "nan")), float(fields.get("norm", "nan")))
            if "tel" in fields:
                out["val"][step] = float(fields["tel"])
            if "eval" in fields:
                out["eval"][step] = float(fields["eval"])
    return out


def validate_log(path: str, final_step: int | None = None, max_final_train_loss: float | None = None,
                 max_final_val_loss: float | None = None, require_decrease: bool = True) -> list[str]:
    """Checks in the spirit of the reference's dev/validate_training_log.py; returns a list of problems."""
    import math

    log = parse_log(path)
    problems = []
    tr = log["train"]
    if not tr:
        return ["no training lines"]
    steps = sorted(tr)
    if final_step is not None and steps[-1] != final_step:
        problems.append(f"final step is {steps[-1]}, expected {final_step}")
    if any(not math.isfinite(v[0]) for v in tr.values()):
        problems.append("non-finite training loss")
    if require_decrease and len(steps) > 1 and not tr[steps[-1]][0] < tr[steps[0]][0]:
        problems.append("training loss did not decrease")
    if max_final_train_loss is not None and tr[steps[-1]][0] > max_final_train_loss:
        problems.append("final training loss above threshold")
    if max_final_val_loss is not None and log["val"]:
        if log["val"][max(log["val"])] > max_final_val_loss:
            problems.append("final validation loss above threshold")
    return problems


def compare_logs(path_a: str, path_b: str, rel_tol: float = 0.02, abs_tol: float = 0.02) -> list[str]:
    """Curve comparison of two runs (how 'N GPUs == 1 GPU' style checks are expressed)."""
    a, b = parse_log(path_a)["train"], parse_log(path_b)["train"]
    problems = []
    common = sorted(set(a) & set(b))
    if not common:
        return ["no common steps"]
    for s in common:
        la, lb = a[s][0], b[s][0]
        if abs(la - lb) > abs_tol + rel_tol * max(abs(la), abs(lb)):
            problems.append(f"step {s}: {la} vs {lb}")
    return problems
