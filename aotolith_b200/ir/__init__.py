"""Typed SSA IR: dtypes, tensor types, values, operations, graphs.

The vocabulary and field names are those of the reference compiler
(``src/aotolith/ir/types.py``, ``ir/op.py``, ``ir/graph.py``) because they are
the contract between the rewrite pipeline and a backend: a backend receives a
``Graph`` and binds kernels to ``Operation``s by ``op`` name, operand order and
``attrs``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..errors import IRValidationError


class DType(str, Enum):
    F16 = "float16"
    BF16 = "bfloat16"
    F32 = "float32"
    BOOL = "bool"
    I32 = "int32"
    I64 = "int64"


#: bytes per element
DTYPE_ITEMSIZE: dict[DType, int] = {
    DType.F16: 2,
    DType.BF16: 2,
    DType.F32: 4,
    DType.BOOL: 1,
    DType.I32: 4,
    DType.I64: 8,
}


@dataclass(frozen=True, slots=True)
class TensorType:
    shape: tuple[int, ...]
    dtype: DType

    def __post_init__(self) -> None:
        if any((not isinstance(dim, int)) or dim <= 0 for dim in self.shape):
            raise ValueError(f"tensor dimensions must be static and positive: {self.shape}")

    @property
    def numel(self) -> int:
        count = 1
        for dim in self.shape:
            count *= dim
        return count

    @property
    def nbytes(self) -> int:
        return self.numel * DTYPE_ITEMSIZE[self.dtype]


@dataclass(frozen=True, slots=True)
class Value:
    id: str
    type: TensorType


@dataclass(frozen=True, slots=True)
class Operation:
    """One operation: ``outputs = op(inputs) {attrs}``; at least one output."""

    op: str
    inputs: tuple[str, ...]
    outputs: tuple[str, ...]
    attrs: dict[str, object] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.outputs:
            raise ValueError(f"{self.op} must produce at least one value")
        if len(set(self.outputs)) != len(self.outputs):
            raise ValueError(f"{self.op} must produce distinct values: {self.outputs}")

    @property
    def output(self) -> str:
        if len(self.outputs) != 1:
            raise ValueError(
                f"{self.op} produces {len(self.outputs)} values; select one instead of "
                "asking for a single output"
            )
        return self.outputs[0]


@dataclass(frozen=True, slots=True)
class Graph:
    """Inputs, typed values, operations in execution order, outputs."""

    inputs: tuple[str, ...]
    values: dict[str, Value]
    ops: tuple[Operation, ...]
    outputs: tuple[str, ...]

    def validate(self) -> None:
        """Every value is typed and defined exactly once before use."""

        if len(set(self.inputs)) != len(self.inputs):
            raise IRValidationError("graph inputs must be unique")
        if not set(self.inputs) <= set(self.values):
            raise IRValidationError("every graph input must have a value type")
        if not set(self.outputs) <= set(self.values):
            raise IRValidationError("every graph output must have a value type")
        defined = set(self.inputs)
        for op in self.ops:
            missing = [value for value in op.inputs if value not in defined]
            if missing:
                raise IRValidationError(f"{op.op} uses undefined values: {sorted(missing)}")
            untyped = [value for value in op.outputs if value not in self.values]
            if untyped:
                raise IRValidationError(f"{op.op} produces values without types: {sorted(untyped)}")
            again = [value for value in op.outputs if value in defined]
            if again:
                raise IRValidationError(f"values defined more than once: {sorted(again)}")
            defined.update(op.outputs)
        undefined = [value for value in self.outputs if value not in defined]
        if undefined:
            raise IRValidationError(f"undefined graph outputs: {sorted(undefined)}")

    def value(self, value_id: str) -> Value:
        return self.values[value_id]

    def replace_ops(self, ops: tuple[Operation, ...]) -> "Graph":
        graph = Graph(self.inputs, self.values, tuple(ops), self.outputs)
        graph.validate()
        return graph


__all__ = ["DTYPE_ITEMSIZE", "DType", "Graph", "Operation", "TensorType", "Value"]
