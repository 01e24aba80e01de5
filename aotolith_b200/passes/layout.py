"""Layout clean-up passes: dead views, unit-axis transposes, matmul operand layouts.

Behavioural counterparts of ``src/aotolith/passes/layout.py`` and
``passes/canonicalize.py`` in the reference. IR values are logical (row-major)
tensors, so a ``transpose`` that only moves unit axes is a ``reshape``.
"""

from __future__ import annotations

from ..ir import Graph, Operation
from .rewriter import Rewriter

_RESHAPE_LIKE = ("reshape", "unsqueeze", "squeeze")


def _moves_only_unit_axes(shape: tuple[int, ...], dim0: int, dim1: int) -> bool:
    rank = len(shape)
    dim0, dim1 = dim0 % rank, dim1 % rank
    order = list(range(rank))
    order[dim0], order[dim1] = order[dim1], order[dim0]
    before = [axis for axis in range(rank) if shape[axis] != 1]
    after = [axis for axis in order if shape[axis] != 1]
    return before == after


def _full_slice(op: Operation, shape: tuple[int, ...]) -> bool:
    dim = int(op.attrs["dim"]) % len(shape)
    extent = shape[dim]
    start, end, step = int(op.attrs["start"]), int(op.attrs["end"]), int(op.attrs.get("step", 1))
    if start < 0:
        start += extent
    if end < 0:
        end += extent
    return step == 1 and start <= 0 and end >= extent


def _simplify_once(rw: Rewriter) -> bool:
    changed = False
    for op in list(rw.ops):
        if op not in rw.ops:
            continue
        kind = op.op
        if kind not in ("reshape", "expand", "slice", "transpose", "squeeze", "unsqueeze", "cast"):
            continue
        source = op.inputs[0]
        in_type, out_type = rw.type(source), rw.type(op.outputs[0])
        # identity views
        identity = False
        if kind in ("reshape", "expand", "cast"):
            identity = in_type == out_type
        elif kind == "slice":
            identity = _full_slice(op, in_type.shape)
        elif kind == "transpose":
            rank = len(in_type.shape)
            identity = int(op.attrs["dim0"]) % rank == int(op.attrs["dim1"]) % rank
        if identity:
            rw.replace_uses(op.outputs[0], source)
            rw.erase(op)
            changed = True
            continue
        if kind == "transpose" and _moves_only_unit_axes(
            in_type.shape, int(op.attrs["dim0"]), int(op.attrs["dim1"])
        ):
            rw.replace(op, Operation("reshape", op.inputs, op.outputs, {"shape": out_type.shape}))
            changed = True
            continue
        producer = rw.producer(source)
        if producer is None:
            continue
        if kind == "reshape" and producer.op in _RESHAPE_LIKE:
            rw.replace(op, Operation("reshape", producer.inputs, op.outputs, dict(op.attrs)))
            changed = True
            continue
        if kind in ("squeeze", "unsqueeze") and producer.op == "reshape":
            rw.replace(op, Operation("reshape", producer.inputs, op.outputs, {"shape": out_type.shape}))
            changed = True
            continue
        if kind == "squeeze" and producer.op == "unsqueeze" and rw.type(producer.inputs[0]) == out_type:
            rw.replace_uses(op.outputs[0], producer.inputs[0])
            rw.erase(op)
            changed = True
            continue
        if kind == "transpose" and producer.op == "transpose":
            rank = len(in_type.shape)
            mine = {int(op.attrs["dim0"]) % rank, int(op.attrs["dim1"]) % rank}
            theirs = {int(producer.attrs["dim0"]) % rank, int(producer.attrs["dim1"]) % rank}
            if mine == theirs:
                rw.replace_uses(op.outputs[0], producer.inputs[0])
                rw.erase(op)
                changed = True
                continue
    return changed


def simplify_layouts(graph: Graph) -> Graph:
    """Drop identity views, turn unit-axis transposes into reshapes, fold view chains."""

    rw = Rewriter(graph)
    while _simplify_once(rw):
        rw.dce()
    return rw.finish()


def collapse_trailing_layouts(graph: Graph) -> Graph:
    """The same sweep, run on the final graph: every fusion leaves views of its own."""

    return simplify_layouts(graph)


def canonicalize_batched_matmul(graph: Graph) -> Graph:
    """Undo PyTorch's expand-and-bmm spelling of a rank-N ``F.linear``.

    ``matmul(x[..., M, K], expand(w[K, N]) -> [1.., K, N])`` reads ``w``
    directly; the product broadcasts to the same shape.
    """

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "matmul" or len(op.inputs) != 2:
            continue
        right = rw.producer(op.inputs[1])
        if right is None or right.op != "expand" or not rw.single_use(op.inputs[1]):
            continue
        inner = rw.shape(right.inputs[0])
        outer = rw.shape(op.inputs[1])
        if len(inner) != 2 or outer[-2:] != inner or any(dim != 1 for dim in outer[:-2]):
            continue
        rw.replace(op, Operation("matmul", (op.inputs[0], right.inputs[0]), op.outputs, dict(op.attrs)))
    graph = rw.finish()
    return simplify_layouts(graph)


def fold_matmul_input_layouts(graph: Graph) -> Graph:
    """A single-use transpose of the last two axes of a matmul operand becomes a flag."""

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op not in ("matmul", "addmm"):
            continue
        base = 1 if op.op == "addmm" else 0
        if len(op.inputs) != base + 2:
            continue
        inputs = list(op.inputs)
        attrs = dict(op.attrs)
        touched = False
        for offset, flag in ((0, "transpose_a"), (1, "transpose_b")):
            value = inputs[base + offset]
            producer = rw.producer(value)
            if producer is None or producer.op != "transpose" or not rw.single_use(value):
                continue
            rank = len(rw.shape(value))
            if rank < 2:
                continue
            dims = {int(producer.attrs["dim0"]) % rank, int(producer.attrs["dim1"]) % rank}
            if dims != {rank - 1, rank - 2}:
                continue
            inputs[base + offset] = producer.inputs[0]
            if attrs.get(flag, False):
                attrs.pop(flag)
            else:
                attrs[flag] = True
            touched = True
        if touched:
            rw.replace(op, Operation(op.op, tuple(inputs), op.outputs, attrs))
    return rw.finish()
