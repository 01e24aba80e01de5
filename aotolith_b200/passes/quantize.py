"""Fold a ``dequantize_i4`` / ``dequantize_i8`` into the matmul that consumes it (decode rows only).

``matmul(x, dequantize_i4(Wp, S)){transpose_b}`` becomes
``matmul(x, Wp, S){weight_group_size, weight_bits}`` when the activation is a
single row, the unpacked weight has no other consumer and is not a graph
output. With more rows the pair is kept apart: the reference semantics there is
"materialise the bf16 weight, then a dense product"
(``src/aotolith/passes/quantize.py:43-112``).
"""

from __future__ import annotations

from ..ir import Graph, Operation
from .rewriter import Rewriter

#: unpack operation -> bits a code (``src/aotolith/passes/quantize.py:31`` of the reference)
_UNPACK_OPS = {"dequantize_i4": 4, "dequantize_i8": 8}


def fold_quantized_weights(graph: Graph) -> Graph:
    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op not in ("matmul", "addmm"):
            continue
        base = 1 if op.op == "addmm" else 0
        if len(op.inputs) != base + 2 or not op.attrs.get("transpose_b", False):
            continue
        if op.attrs.get("transpose_a", False) or "weight_group_size" in op.attrs:
            continue
        weight = op.inputs[base + 1]
        unpack = rw.producer(weight)
        if unpack is None or unpack.op not in _UNPACK_OPS or not rw.single_use(weight):
            continue
        left_shape = rw.shape(op.inputs[base])
        if len(left_shape) < 2 or left_shape[-2] != 1:
            continue
        attrs = {key: value for key, value in op.attrs.items() if key != "transpose_b"}
        attrs["weight_group_size"] = int(unpack.attrs["group_size"])
        attrs["weight_bits"] = _UNPACK_OPS[unpack.op]
        inputs = op.inputs[: base + 1] + tuple(unpack.inputs)
        rw.replace(op, Operation(op.op, inputs, op.outputs, attrs))
    return rw.finish()
