"""Common-subexpression elimination by value numbering.

Two operations with the same name, the same (already merged) inputs, the same
output types and the same attributes compute the same values; the later one is
dropped. This is what collapses the per-layer rotary-table gathers and mask
conversions of a decoder graph into one
(reference: ``src/aotolith/passes/cse.py:13-55``).
"""

from __future__ import annotations

from ..ir import Graph, Operation
from .rewriter import Rewriter


def _freeze(value, rename):
    if isinstance(value, Operation):
        local = dict(rename)
        inputs = tuple(local.get(v, v) for v in value.inputs)
        return ("op", value.op, inputs, len(value.outputs), _freeze(value.attrs, rename))
    if isinstance(value, dict):
        return tuple(sorted((key, _freeze(item, rename)) for key, item in value.items()))
    if isinstance(value, (list, tuple)):
        if value and all(isinstance(item, Operation) for item in value):
            # a fused body: number its internal values by position
            local = dict(rename)
            frozen = []
            for position, item in enumerate(value):
                frozen.append(_freeze(item, local))
                for slot, out in enumerate(item.outputs):
                    local[out] = f"%{position}.{slot}"
            return tuple(frozen)
        return tuple(_freeze(item, rename) for item in value)
    if isinstance(value, float) and value != value:
        return "nan"
    return value


def eliminate_common_subexpressions(graph: Graph) -> Graph:
    rw = Rewriter(graph)
    seen: dict[object, Operation] = {}
    for op in list(rw.ops):
        current = next(candidate for candidate in rw.ops if candidate.outputs == op.outputs)
        key = (
            current.op,
            current.inputs,
            tuple(rw.type(out) for out in current.outputs),
            _freeze(current.attrs, {}),
        )
        first = seen.get(key)
        if first is None:
            seen[key] = current
            continue
        for mine, theirs in zip(current.outputs, first.outputs):
            rw.replace_uses(mine, theirs)
        rw.erase(current)
    return rw.finish()
