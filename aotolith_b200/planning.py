"""Storage planning: value lifetimes, reusable slots, arena size.

Derived from shapes only, so a host can budget before loading a model. Same
record shapes as ``src/aotolith/planning.py`` of the reference
(``ValueLifetime``, ``BufferSlot``, ``StoragePlan``, ``plan_storage``,
``tensor_nbytes``). Slots are 256-byte aligned here: that is the alignment the
device allocator gives and what vectorised kernel accesses assume.
"""

from __future__ import annotations

from dataclasses import dataclass

from .ir import Graph, TensorType

BUFFER_ALIGNMENT = 256


def tensor_nbytes(tensor_type: TensorType) -> int:
    return tensor_type.nbytes


@dataclass(frozen=True, slots=True)
class ValueLifetime:
    value_id: str
    tensor_type: TensorType
    start: int  # index of the producing op, -1 for inputs
    end: int    # one past the last op that reads it (len(ops)+1 for outputs)
    size_bytes: int
    is_input: bool
    is_output: bool

    @property
    def overlaps(self) -> bool:
        return self.end > self.start


@dataclass(frozen=True, slots=True)
class BufferSlot:
    slot_id: int
    offset_bytes: int
    size_bytes: int
    alignment_bytes: int
    value_ids: tuple[str, ...]


@dataclass(frozen=True, slots=True)
class StoragePlan:
    lifetimes: tuple[ValueLifetime, ...]
    slots: tuple[BufferSlot, ...]
    release_after_op: tuple[tuple[str, ...], ...]
    peak_live_bytes: int
    arena_size_bytes: int


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


def plan_storage(graph: Graph) -> StoragePlan:
    """Lifetimes of every value, first-fit slot reuse for intermediates."""

    graph.validate()
    ops = graph.ops
    born = {out: index for index, op in enumerate(ops) for out in op.outputs}
    last = {value: -1 for value in list(graph.inputs) + list(born)}
    for index, op in enumerate(ops):
        for value in op.inputs:
            last[value] = index
    for value in graph.outputs:
        last[value] = len(ops)
    inputs, outputs = set(graph.inputs), set(graph.outputs)
    lifetimes = []
    for value in sorted(last):
        start = born.get(value, -1)
        lifetimes.append(
            ValueLifetime(
                value_id=value,
                tensor_type=graph.value(value).type,
                start=start,
                end=max(last[value], start) + 1,
                size_bytes=tensor_nbytes(graph.value(value).type),
                is_input=value in inputs,
                is_output=value in outputs,
            )
        )
    release: list[list[str]] = [[] for _ in ops]
    for value, index in last.items():
        index = max(index, born.get(value, -1))
        if value not in outputs and 0 <= index < len(ops):
            release[index].append(value)

    # first-fit over intermediates, in order of birth
    slots: list[tuple[int, list[ValueLifetime]]] = []
    for life in sorted(
        (l for l in lifetimes if not l.is_input and not l.is_output), key=lambda l: (l.start, l.value_id)
    ):
        for index, (size, tenants) in enumerate(slots):
            if size >= life.size_bytes and all(
                life.start >= other.end or other.start >= life.end for other in tenants
            ):
                tenants.append(life)
                break
        else:
            slots.append((life.size_bytes, [life]))
    placed: list[BufferSlot] = []
    offset = 0
    for slot_id, (size, tenants) in enumerate(slots):
        offset = _round_up(offset, BUFFER_ALIGNMENT)
        placed.append(
            BufferSlot(slot_id, offset, size, BUFFER_ALIGNMENT, tuple(t.value_id for t in tenants))
        )
        offset += size

    events: dict[int, int] = {}
    for life in lifetimes:
        events[life.start] = events.get(life.start, 0) + life.size_bytes
        events[life.end] = events.get(life.end, 0) - life.size_bytes
    live = peak = 0
    for index in sorted(events):
        live += events[index]
        peak = max(peak, live)
    return StoragePlan(
        lifetimes=tuple(lifetimes),
        slots=tuple(placed),
        release_after_op=tuple(tuple(sorted(values)) for values in release),
        peak_live_bytes=peak,
        arena_size_bytes=_round_up(offset, BUFFER_ALIGNMENT),
    )
