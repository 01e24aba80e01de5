"""A small mutable view of a graph for pattern rewrites.

A pass opens a ``Rewriter`` on a graph, asks who produces and who consumes a
value, replaces operations, and closes it: ``finish()`` drops dead operations,
restores a valid execution order and validates. Matches are "narrow" in the
sense the reference's passes are (``src/aotolith/passes/graph.py:16-51``): a
value may be absorbed into a fused operation only if that operation is its
single consumer and it is not a graph output.
"""

from __future__ import annotations

from collections import defaultdict

from ..ir import Graph, Operation, TensorType, Value

LAYOUT_OPS = frozenset({"reshape", "transpose", "unsqueeze", "squeeze", "expand", "slice", "permute"})


class Rewriter:
    def __init__(self, graph: Graph) -> None:
        self.inputs = graph.inputs
        self.outputs = list(graph.outputs)
        self.values: dict[str, Value] = dict(graph.values)
        self.ops: list[Operation] = list(graph.ops)
        self._index_dirty = True
        self._producer: dict[str, Operation] = {}
        self._users: dict[str, list[Operation]] = {}
        self._fresh = 0

    # -- indexes -------------------------------------------------------------
    def _reindex(self) -> None:
        if not self._index_dirty:
            return
        self._producer = {}
        users: dict[str, list[Operation]] = defaultdict(list)
        for op in self.ops:
            for out in op.outputs:
                self._producer[out] = op
            for value in dict.fromkeys(op.inputs):
                users[value].append(op)
        self._users = users
        self._index_dirty = False

    def producer(self, value_id: str) -> Operation | None:
        self._reindex()
        return self._producer.get(value_id)

    def users(self, value_id: str) -> list[Operation]:
        self._reindex()
        return list(self._users.get(value_id, ()))

    def is_output(self, value_id: str) -> bool:
        return value_id in self.outputs

    def single_use(self, value_id: str) -> bool:
        """Exactly one consuming operation and not a graph output."""

        return not self.is_output(value_id) and len(self.users(value_id)) == 1

    def type(self, value_id: str) -> TensorType:
        return self.values[value_id].type

    def shape(self, value_id: str) -> tuple[int, ...]:
        return self.values[value_id].type.shape

    # -- edits ---------------------------------------------------------------
    def new_value(self, ttype: TensorType, hint: str = "r") -> str:
        while True:
            value_id = f"{hint}{self._fresh}"
            self._fresh += 1
            if value_id not in self.values:
                break
        self.values[value_id] = Value(value_id, ttype)
        return value_id

    def named_value(self, value_id: str, ttype: TensorType) -> str:
        """Register ``value_id`` (uniquified if taken) with ``ttype``."""

        candidate, suffix = value_id, 0
        while candidate in self.values:
            suffix += 1
            candidate = f"{value_id}_{suffix}"
        self.values[candidate] = Value(candidate, ttype)
        return candidate

    def replace(self, old: Operation, *new: Operation) -> None:
        """Put ``new`` where ``old`` was."""

        position = next(i for i, op in enumerate(self.ops) if op is old)
        self.ops[position : position + 1] = list(new)
        self._index_dirty = True

    def insert_before(self, anchor: Operation, *new: Operation) -> None:
        position = next(i for i, op in enumerate(self.ops) if op is anchor)
        self.ops[position:position] = list(new)
        self._index_dirty = True

    def erase(self, *ops: Operation) -> None:
        doomed = {id(op) for op in ops}
        self.ops = [op for op in self.ops if id(op) not in doomed]
        self._index_dirty = True

    def replace_uses(self, old: str, new: str) -> None:
        """Every consumer (and graph output) of ``old`` reads ``new`` instead."""

        if old == new:
            return
        for index, op in enumerate(self.ops):
            if old in op.inputs:
                self.ops[index] = Operation(
                    op.op, tuple(new if v == old else v for v in op.inputs), op.outputs, op.attrs
                )
        self.outputs = [new if v == old else v for v in self.outputs]
        self._index_dirty = True

    # -- closing -------------------------------------------------------------
    def dce(self) -> None:
        live = set(self.outputs)
        kept: list[Operation] = []
        for op in reversed(self.ops):
            if any(out in live for out in op.outputs):
                kept.append(op)
                live.update(op.inputs)
        kept.reverse()
        self.ops = kept
        self._index_dirty = True

    def _sorted(self) -> list[Operation]:
        defined = set(self.inputs)
        pending = list(self.ops)
        ordered: list[Operation] = []
        while pending:
            progressed = False
            rest: list[Operation] = []
            for op in pending:
                if all(value in defined for value in op.inputs):
                    ordered.append(op)
                    defined.update(op.outputs)
                    progressed = True
                else:
                    rest.append(op)
            if not progressed:
                # leave the cycle / undefined value for validate() to report
                ordered.extend(rest)
                break
            pending = rest
        return ordered

    def finish(self) -> Graph:
        self.dce()
        ops = self._sorted()
        used = set(self.inputs) | set(self.outputs)
        for op in ops:
            used.update(op.inputs)
            used.update(op.outputs)
            for inner in op.attrs.get("body", ()):  # values internal to a fused region keep their types
                used.update(inner.inputs)
                used.update(inner.outputs)
        values = {key: value for key, value in self.values.items() if key in used}
        graph = Graph(tuple(self.inputs), values, tuple(ops), tuple(self.outputs))
        graph.validate()
        return graph


def see_through_reshapes(rw: Rewriter, value_id: str) -> str:
    """Follow single-input ``reshape`` producers back to their source."""

    while True:
        op = rw.producer(value_id)
        if op is None or op.op != "reshape":
            return value_id
        value_id = op.inputs[0]
