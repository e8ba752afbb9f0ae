"""ZeRO sharding arithmetic (host only, no GPU).

Sharding rule (kept from the reference so optimizer-state files stay interchangeable,
llmc/zero.cuh:580-614 and train_gpt2.cu:1292-1308): every tensor is split PER LAYER SLICE into
``P`` equal contiguous parts; rank ``r`` owns elements ``[r*S/P, (r+1)*S/P)`` of every layer slice of
size ``S``. Its optimizer state (m, v, master) is the concatenation over tensors of ``L`` blocks of
``S/P`` elements, located at ``tensor.offset / P + l * S/P``. Expert-parallel tensors of a MoE model
are different: the expert dimension is split across ranks (rank ``r`` owns experts
``[r*E/P, (r+1)*E/P)`` completely) and they are neither reduced nor gathered.

The functions here produce *segment tables*: lists of ``(param_off, grad_off, state_off, length,
decay)`` that the optimizer kernels walk (``ops/optim.py``), plus the per-layer bucket description
used by the gradient reduce-scatter and the parameter all-gather.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..models.config import ModelConfig, ParamLayout, TensorSlot


class ZeroError(ValueError):
    pass


def validate_zero_stage(stage: int) -> None:
    if stage < 0 or stage > 3:
        raise ZeroError(f"Invalid ZeRO stage {stage}: supported stages are 0, 1, 2 and 3")


def validate_sharding(config: ModelConfig, num_processes: int, stage: int) -> list[str]:
    """Messages describing every tensor that cannot be split; empty when the model shards cleanly."""
    validate_zero_stage(stage)
    problems = []
    if stage == 0 or num_processes == 1:
        return problems
    for slot in config.layout().slots:
        if slot.spec.expert:
            E = slot.spec.shape[0]
            if E % num_processes != 0 and num_processes % E != 0:
                problems.append(f"{slot.spec.name}: {E} experts cannot be spread over {num_processes} processes")
            continue
        if slot.size % num_processes != 0:
            problems.append(f"{slot.spec.name}: per-layer size {slot.size} is not divisible by {num_processes} processes")
        elif (slot.size // num_processes) % 8 != 0:
            problems.append(f"{slot.spec.name}: shard of {slot.size // num_processes} elements is not a multiple of 8 (16 bytes)")
    return problems


@dataclass(frozen=True)
class Segment:
    tensor: str
    layer: int
    param_off: int   # element offset in the flat parameter buffer
    state_off: int   # element offset in this rank's m / v / master buffers
    length: int
    decay: bool


class ZeroPlan:
    """Which elements rank ``rank`` of ``num_processes`` updates, and where their state lives."""

    def __init__(self, config: ModelConfig, num_processes: int = 1, rank: int = 0, stage: int = 0):
        validate_zero_stage(stage)
        self.config, self.P, self.rank, self.stage = config, num_processes, rank, stage
        self.layout: ParamLayout = config.layout()
        self.sharded = stage >= 1 and num_processes > 1
        if self.sharded:
            problems = validate_sharding(config, num_processes, stage)
            if problems:
                raise ZeroError("model cannot be sharded: " + "; ".join(problems))
        self.segments: list[Segment] = []
        state_off = 0
        for slot in self.layout.slots:
            if slot.spec.expert and num_processes > 1:
                # expert parallel: whole experts, complete gradients, no reduction
                E = slot.spec.shape[0]
                per_expert = slot.size // E
                owned = [e for e in range(E) if self._expert_owner(e, E) == rank]
                for l in range(slot.layers):
                    for e in owned:
                        self.segments.append(Segment(slot.spec.name, l, slot.offset + l * slot.size + e * per_expert, state_off,
                                                     per_expert, slot.spec.decay))
                        state_off += per_expert
                continue
            if self.sharded:
                shard = slot.size // num_processes
                base = slot.offset // num_processes
                for l in range(slot.layers):
                    self.segments.append(Segment(slot.spec.name, l, slot.offset + l * slot.size + rank * shard,
                                                 base + l * shard, shard, slot.spec.decay))
                state_off = max(state_off, base + slot.layers * shard)
            else:
                for l in range(slot.layers):
                    self.segments.append(Segment(slot.spec.name, l, slot.offset + l * slot.size, slot.offset + l * slot.size,
                                                 slot.size, slot.spec.decay))
                state_off = max(state_off, slot.offset + slot.total)
        self.state_elements = state_off if not self._has_experts() or num_processes == 1 else self._state_total()

    def _has_experts(self) -> bool:
        return any(s.spec.expert for s in self.layout.slots)

    def _state_total(self) -> int:
        # with expert-parallel tensors the state buffer is simply packed in segment order
        total = 0
        segs = []
        for s in self.segments:
            segs.append(Segment(s.tensor, s.layer, s.param_off, total, s.length, s.decay))
            total += s.length
        self.segments = segs
        return total

    def _expert_owner(self, e: int, E: int) -> int:
        if E >= self.P:
            return e // (E // self.P)
        return e * (self.P // E)  # fewer experts than ranks: expert e lives on the first rank of its group

    # ------------------------------------------------------------------ tables
    def segment_rows(self, merge: bool = True):
        """Rows ``(param_off, grad_off, state_off, length, decay)`` for ``ops.optim.make_segments``.
        Adjacent segments that are contiguous in both buffers are merged when ``merge``."""
        rows = []
        for s in self.segments:
            if merge and rows:
                p, g, st, n, d = rows[-1]
                if p + n == s.param_off and st + n == s.state_off and d == s.decay:
                    rows[-1] = (p, g, st, n + s.length, d)
                    continue
            rows.append((s.param_off, s.param_off, s.state_off, s.length, s.decay))
        return rows

    def shard_interval(self, tensor: str, layer: int) -> tuple[int, int]:
        """Element interval (start, end) inside the layer slice of ``tensor`` that this rank owns."""
        slot: TensorSlot = self.layout[tensor]
        if not self.sharded or slot.spec.expert:
            return 0, slot.size
        shard = slot.size // self.P
        return self.rank * shard, (self.rank + 1) * shard

    def layer_bucket(self, layer: int | None) -> list[tuple[str, int, int]]:
        """Dense tensors reduced together: ``layer`` = block index, or ``None`` for the non-block tensors.
        Returns ``(name, element offset of the slice in the flat buffer, slice size)``."""
        out = []
        for slot in self.layout.slots:
            if slot.spec.expert and self.P > 1:
                continue
            if layer is None and not slot.spec.layered:
                out.append((slot.spec.name, slot.offset, slot.size))
            elif layer is not None and slot.spec.layered:
                out.append((slot.spec.name, slot.offset + layer * slot.size, slot.size))
        return out


def shard_intervals_table(config: ModelConfig, num_processes: int) -> dict:
    """For tests and the dry run: {tensor: [(layer, rank, start, end) ...]} in flat-buffer coordinates."""
    table = {}
    layout = config.layout()
    for slot in layout.slots:
        rows = []
        if slot.spec.expert:
            continue
        shard = slot.size // num_processes
        for l in range(slot.layers):
            for r in range(num_processes):
                start = slot.offset + l * slot.size + r * shard
                rows.append((l, r, start, start + shard))
        table[slot.spec.name] = rows
    return table
