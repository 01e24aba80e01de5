"""ATen (FX) graph -> typed IR, for the operator set the decoder graphs use.

The handlers cover what tracing the static-cache adapters produces: embedding,
the decomposed ``F.rms_norm``, ``F.linear`` in its 2-D (``t`` + ``mm`` /
``addmm``) and 3-D (``expand`` + ``bmm``) spellings, views, ``split`` /
``slice`` / ``select``, ``cat`` / ``stack``, the rotary arithmetic, the boolean
mask conversion, SDPA and the ``dequantize_i4`` / ``dequantize_i8`` operators. The emitted spelling
(op names, attribute names, operand orders) is the one the reference's
legaliser produces (``src/aotolith/legalize/``): ``aten.t`` becomes
``transpose{dim0:1, dim1:0}``, ``torch.stack`` becomes ``unsqueeze`` x n +
``cat``, ``aten.select`` becomes ``slice`` + ``squeeze``, ``aten._to_copy``
becomes ``cast``, open-ended slices keep ``end = 2**63 - 1``. Anything else is
refused with ``UnsupportedOperationError`` naming the target.
"""

from __future__ import annotations

from typing import Any

import torch

from ..errors import CompilationError, UnsupportedDTypeError, UnsupportedOperationError
from ..ir import DType, Graph, Operation, TensorType, Value

INT64_MAX = 9223372036854775807

_DTYPES = {
    torch.float16: DType.F16,
    torch.bfloat16: DType.BF16,
    torch.float32: DType.F32,
    torch.bool: DType.BOOL,
    torch.int32: DType.I32,
    torch.int64: DType.I64,
}


def tensor_type_of(tensor: Any, what: str = "value") -> TensorType:
    dtype = _DTYPES.get(tensor.dtype)
    if dtype is None:
        raise UnsupportedDTypeError(f"{what} has dtype {tensor.dtype}, which the IR does not cover")
    shape = tuple(int(dim) for dim in tensor.shape)
    return TensorType(shape, dtype)


class _Lowering:
    def __init__(self, traced, promoted_constants):
        self.traced = traced
        self.promoted = promoted_constants
        self.values: dict[str, Value] = {}
        self.ops: list[Operation] = []
        self.inputs: list[str] = []
        self.ids: dict[Any, Any] = {}  # fx node -> value id (or tuple of ids / None)
        self.skip: set[Any] = set()
        self._counter = 0

    # -- helpers -----------------------------------------------------------
    def fresh(self, ttype: TensorType) -> str:
        value_id = f"v{self._counter}"
        self._counter += 1
        self.values[value_id] = Value(value_id, ttype)
        return value_id

    def emit(self, op: str, inputs, out_type: TensorType, attrs=None) -> str:
        out = self.fresh(out_type)
        self.ops.append(Operation(op, tuple(inputs), (out,), dict(attrs or {})))
        return out

    def node_type(self, node) -> TensorType:
        return tensor_type_of(node.meta["val"], f"node {node.name}")

    def arg(self, node) -> str:
        if not isinstance(node, torch.fx.Node):
            raise UnsupportedOperationError(
                f"a non-tensor operand ({node!r}) reached an operator that needs a tensor"
            )
        value = self.ids.get(node)
        if not isinstance(value, str):
            raise CompilationError(f"FX node {node.name} has no single IR value")
        return value

    def type_of(self, value_id: str) -> TensorType:
        return self.values[value_id].type


def _norm_dim(dim: int, rank: int) -> int:
    return dim % rank if rank else 0


# ---------------------------------------------------------------------------
# handlers: (lowering, node) -> None; they record self.ids[node]
# ---------------------------------------------------------------------------

def _embedding(lw, node):
    weight, indices = node.args[:2]
    padding_idx = node.args[2] if len(node.args) > 2 else -1
    lw.ids[node] = lw.emit(
        "embedding", (lw.arg(weight), lw.arg(indices)), lw.node_type(node),
        {"padding_idx": int(padding_idx), "scale_grad_by_freq": False, "sparse": False},
    )


def _to_copy(lw, node):
    source = lw.arg(node.args[0])
    out_type = lw.node_type(node)
    if out_type == lw.type_of(source):
        lw.ids[node] = source
        return
    lw.ids[node] = lw.emit("cast", (source,), out_type)


def _rms_norm_chain(lw, node) -> bool:
    """``x * rsqrt(mean(x**2, -1, keepdim) + eps)`` rooted at ``pow`` -> ``rms_norm``."""

    source, exponent = node.args
    if exponent != 2 or len(node.users) != 1:
        return False
    mean = next(iter(node.users))
    if str(mean.target) != "aten.mean.dim":
        return False
    rank = len(node.meta["val"].shape)
    dims = mean.args[1]
    keepdim = mean.args[2] if len(mean.args) > 2 else False
    if [_norm_dim(d, rank) for d in dims] != [rank - 1] or not keepdim or len(mean.users) != 1:
        return False
    add = next(iter(mean.users))
    if str(add.target) not in ("aten.add_.Scalar", "aten.add.Scalar", "aten.add.Tensor"):
        return False
    eps = add.args[1]
    if not isinstance(eps, (int, float)) or len(add.users) != 1:
        return False
    rsqrt = next(iter(add.users))
    if str(rsqrt.target) != "aten.rsqrt.default" or len(rsqrt.users) != 1:
        return False
    mul = next(iter(rsqrt.users))
    if str(mul.target) != "aten.mul.Tensor" or set(mul.args) != {source, rsqrt}:
        return False
    width = int(node.meta["val"].shape[-1])
    lw.ids[mul] = lw.emit(
        "rms_norm", (lw.arg(source),), lw.node_type(mul),
        {"normalized_shape": (width,), "eps": float(eps), "has_weight": False},
    )
    lw.skip.update((mean, add, rsqrt))
    return True


def _pow(lw, node):
    if not _rms_norm_chain(lw, node):
        raise UnsupportedOperationError(
            "unsupported FX target: aten.pow.Tensor_Scalar outside the RMS-norm pattern"
        )


def _binary(name):
    def handler(lw, node):
        left, right = node.args[:2]
        attrs = {}
        if name == "add":
            attrs["alpha"] = float(node.kwargs.get("alpha", 1.0))
        numbers = [isinstance(v, (int, float)) and not isinstance(v, bool) for v in (left, right)]
        if numbers[0] != numbers[1]:
            # one tensor and one Python number: the number travels as an attribute, as in the
            # reference's lowering (``legalize/elementwise.py:693-719``)
            attrs["scalar"] = left if numbers[0] else right
            attrs["scalar_position"] = "lhs" if numbers[0] else "rhs"
            tensor = right if numbers[0] else left
            lw.ids[node] = lw.emit(name, (lw.arg(tensor),), lw.node_type(node), attrs)
            return
        lw.ids[node] = lw.emit(name, (lw.arg(left), lw.arg(right)), lw.node_type(node), attrs)
    return handler


def _unary(name):
    def handler(lw, node):
        lw.ids[node] = lw.emit(name, (lw.arg(node.args[0]),), lw.node_type(node))
    return handler


def _reshape(lw, node):
    out_type = lw.node_type(node)
    # the attribute keeps the shape as the program asked for it (a -1 stays a -1, as in the
    # reference's graphs); the value's type carries the resolved one
    asked = node.args[1] if len(node.args) > 1 else out_type.shape
    if not all(isinstance(d, int) and not isinstance(d, bool) for d in asked):
        asked = out_type.shape
    lw.ids[node] = lw.emit("reshape", (lw.arg(node.args[0]),), out_type, {"shape": tuple(int(d) for d in asked)})


def _t(lw, node):
    lw.ids[node] = lw.emit("transpose", (lw.arg(node.args[0]),), lw.node_type(node), {"dim0": 1, "dim1": 0})


def _transpose(lw, node):
    source, dim0, dim1 = node.args
    lw.ids[node] = lw.emit(
        "transpose", (lw.arg(source),), lw.node_type(node), {"dim0": int(dim0), "dim1": int(dim1)}
    )


def _expand(lw, node):
    out_type = lw.node_type(node)
    lw.ids[node] = lw.emit("expand", (lw.arg(node.args[0]),), out_type, {"shape": out_type.shape})


def _unsqueeze(lw, node):
    lw.ids[node] = lw.emit("unsqueeze", (lw.arg(node.args[0]),), lw.node_type(node), {"dim": int(node.args[1])})


def _squeeze_dim(lw, node):
    lw.ids[node] = lw.emit("squeeze", (lw.arg(node.args[0]),), lw.node_type(node), {"dim": int(node.args[1])})


def _slice(lw, node):
    source = node.args[0]
    dim = int(node.args[1]) if len(node.args) > 1 else 0
    start = node.args[2] if len(node.args) > 2 and node.args[2] is not None else 0
    end = node.args[3] if len(node.args) > 3 and node.args[3] is not None else INT64_MAX
    step = int(node.args[4]) if len(node.args) > 4 else 1
    lw.ids[node] = lw.emit(
        "slice", (lw.arg(source),), lw.node_type(node),
        {"dim": dim, "start": int(start), "end": int(end), "step": step},
    )


def _select(lw, node):
    source, dim, index = node.args
    source_id = lw.arg(source)
    source_type = lw.type_of(source_id)
    rank = len(source_type.shape)
    axis = _norm_dim(int(dim), rank)
    index = int(index) % source_type.shape[axis]
    kept = list(source_type.shape)
    kept[axis] = 1
    sliced = lw.emit(
        "slice", (source_id,), TensorType(tuple(kept), source_type.dtype),
        {"dim": axis, "start": index, "end": index + 1, "step": 1},
    )
    lw.ids[node] = lw.emit("squeeze", (sliced,), lw.node_type(node), {"dim": axis})


def _split_with_sizes(lw, node):
    source, sizes = node.args[:2]
    dim = int(node.args[2]) if len(node.args) > 2 else 0
    source_id = lw.arg(source)
    source_type = lw.type_of(source_id)
    axis = _norm_dim(dim, len(source_type.shape))
    pieces = []
    start = 0
    for size in sizes:
        shape = list(source_type.shape)
        shape[axis] = int(size)
        pieces.append((start, start + int(size), TensorType(tuple(shape), source_type.dtype)))
        start += int(size)
    lw.ids[node] = ("split", source_id, axis, pieces)


def _getitem(lw, node):
    parent, index = node.args
    record = lw.ids.get(parent)
    if isinstance(record, tuple) and record and record[0] == "split":
        _, source_id, axis, pieces = record
        start, end, out_type = pieces[index]
        lw.ids[node] = lw.emit(
            "slice", (source_id,), out_type, {"dim": axis, "start": start, "end": end, "step": 1}
        )
        return
    if isinstance(record, tuple) and record and record[0] == "tuple":
        value = record[1][index]
        if value is None:
            if node.users:
                raise UnsupportedOperationError(
                    f"output {index} of {parent.target} is not produced by the lowered operator"
                )
            return
        lw.ids[node] = value
        return
    raise UnsupportedOperationError(f"getitem on {parent.target} is not supported")


def _is_empty(node) -> bool:
    value = getattr(node, "meta", {}).get("val") if isinstance(node, torch.fx.Node) else None
    return isinstance(value, torch.Tensor) and value.numel() == 0


def _cat(lw, node):
    # an operand without elements contributes nothing (an empty cache that a model concatenates
    # its first keys to): it is dropped, and a concatenation of one tensor is that tensor
    tensors = [t for t in node.args[0] if not _is_empty(t)]
    dim = int(node.args[1]) if len(node.args) > 1 else 0
    if len(tensors) == 1:
        lw.ids[node] = lw.arg(tensors[0])
        return
    lw.ids[node] = lw.emit("cat", tuple(lw.arg(t) for t in tensors), lw.node_type(node), {"dim": dim})


def _stack(lw, node):
    tensors = node.args[0]
    dim = int(node.args[1]) if len(node.args) > 1 else 0
    lifted = []
    for tensor in tensors:
        source = lw.arg(tensor)
        source_type = lw.type_of(source)
        axis = dim % (len(source_type.shape) + 1)
        shape = source_type.shape[:axis] + (1,) + source_type.shape[axis:]
        lifted.append(lw.emit("unsqueeze", (source,), TensorType(shape, source_type.dtype), {"dim": axis}))
    out_type = lw.node_type(node)
    axis = dim % len(out_type.shape)
    lw.ids[node] = lw.emit("cat", tuple(lifted), out_type, {"dim": axis})


def _mm(lw, node):
    lw.ids[node] = lw.emit("matmul", (lw.arg(node.args[0]), lw.arg(node.args[1])), lw.node_type(node))


def _addmm(lw, node):
    bias, left, right = node.args[:3]
    lw.ids[node] = lw.emit(
        "addmm", (lw.arg(bias), lw.arg(left), lw.arg(right)), lw.node_type(node),
        {"alpha": float(node.kwargs.get("alpha", 1.0)), "beta": float(node.kwargs.get("beta", 1.0))},
    )


def _scalar_tensor(lw, node):
    lw.ids[node] = lw.emit("scalar_tensor", (), lw.node_type(node), {"value": float(node.args[0])})


def _where(lw, node):
    lw.ids[node] = lw.emit("where", tuple(lw.arg(a) for a in node.args[:3]), lw.node_type(node))


def _sdpa(lw, node):
    """Any ATen SDPA variant -> ``attention(q, k, v[, mask])``; only output 0 is produced."""

    query, key, value = node.args[:3]
    kwargs = dict(node.kwargs)
    target = str(node.target)
    positional = list(node.args[3:])
    mask = kwargs.get("attn_mask")
    dropout = kwargs.get("dropout_p", 0.0)
    causal = kwargs.get("is_causal", False)
    scale = kwargs.get("scale")
    if "flash_attention_for_cpu" in target or "flash_attention" in target:
        if positional:
            dropout = positional[0]
        if len(positional) > 1:
            causal = positional[1]
    else:  # aten.scaled_dot_product_attention / _efficient: (q,k,v,attn_mask,dropout,is_causal)
        if positional:
            mask = positional[0]
        if len(positional) > 1:
            dropout = positional[1]
        if len(positional) > 2:
            causal = positional[2]
    if dropout:
        raise UnsupportedOperationError("attention dropout is not supported in a compiled plan")
    head_dim = int(query.meta["val"].shape[-1])
    inputs = [lw.arg(query), lw.arg(key), lw.arg(value)]
    if mask is not None:
        inputs.append(lw.arg(mask))
    value_meta = node.meta["val"]
    out_meta = value_meta[0] if isinstance(value_meta, (tuple, list)) else value_meta
    out = lw.emit(
        "attention", tuple(inputs), tensor_type_of(out_meta),
        {
            "scale": float(scale) if scale is not None else float(head_dim) ** -0.5,
            "has_mask": mask is not None,
            "causal": bool(causal),
            "safe_softmax": True,
        },
    )
    if isinstance(value_meta, (tuple, list)):
        lw.ids[node] = ("tuple", [out] + [None] * (len(value_meta) - 1))
    else:
        lw.ids[node] = out


def _dequantize_i4(lw, node):
    packed, scales, group_size = node.args
    lw.ids[node] = lw.emit(
        "dequantize_i4", (lw.arg(packed), lw.arg(scales)), lw.node_type(node),
        {"group_size": int(group_size)},
    )


def _dequantize_i8(lw, node):
    packed, scales, group_size = node.args
    lw.ids[node] = lw.emit(
        "dequantize_i8", (lw.arg(packed), lw.arg(scales)), lw.node_type(node),
        {"group_size": int(group_size)},
    )


def _alias(lw, node):
    if _is_empty(node):
        return
    lw.ids[node] = lw.arg(node.args[0])


def _arange(lw, node):
    """``arange(end)`` / ``arange(start, end[, step])`` with Python numbers: an op without inputs."""

    numbers = list(node.args)
    if not 1 <= len(numbers) <= 3 or not all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in numbers):
        raise UnsupportedOperationError("arange takes one to three Python numbers on this frontend")
    start, end, step = (0, numbers[0], 1) if len(numbers) == 1 else (numbers + [1])[:3]
    if step == 0:
        raise UnsupportedOperationError("arange.step must be nonzero")
    lw.ids[node] = lw.emit("arange", (), lw.node_type(node), {"start": start, "end": end, "step": step})


HANDLERS = {
    "aten.embedding.default": _embedding,
    "aten._to_copy.default": _to_copy,
    "aten.pow.Tensor_Scalar": _pow,
    "aten.mul.Tensor": _binary("mul"),
    "aten.add.Tensor": _binary("add"),
    "aten.neg.default": _unary("neg"),
    "aten.cos.default": _unary("cos"),
    "aten.sin.default": _unary("sin"),
    "aten.arange.default": _arange,
    "aten.arange.start": _arange,
    "aten.arange.start_step": _arange,
    "aten.lift_fresh_copy.default": _alias,
    "aten.lift_fresh.default": _alias,
    "aten.silu.default": _unary("silu"),
    "aten.view.default": _reshape,
    "aten._unsafe_view.default": _reshape,
    "aten.reshape.default": _reshape,
    "aten.t.default": _t,
    "aten.transpose.int": _transpose,
    "aten.expand.default": _expand,
    "aten.unsqueeze.default": _unsqueeze,
    "aten.squeeze.dim": _squeeze_dim,
    "aten.slice.Tensor": _slice,
    "aten.select.int": _select,
    "aten.split_with_sizes.default": _split_with_sizes,
    "<built-in function getitem>": _getitem,
    "aten.cat.default": _cat,
    "aten.stack.default": _stack,
    "aten.mm.default": _mm,
    "aten.bmm.default": _mm,
    "aten.addmm.default": _addmm,
    "aten.scalar_tensor.default": _scalar_tensor,
    "aten.where.self": _where,
    "aten._scaled_dot_product_flash_attention_for_cpu.default": _sdpa,
    "aten.scaled_dot_product_attention.default": _sdpa,
    "aten.clone.default": _alias,
    "aten.detach.default": _alias,
    "aten.alias.default": _alias,
    "aten.contiguous.default": _alias,
}

#: custom operators are matched by suffix so the namespace can change
_SUFFIX_HANDLERS = {".dequantize_i4.default": _dequantize_i4, ".dequantize_i8.default": _dequantize_i8}


def _constant(traced, node):
    target = traced
    for part in str(node.target).split("."):
        target = getattr(target, part)
    return target


def legalize(traced, promoted_constants: list[Any] | None = None) -> Graph:
    """Build the IR graph of one traced ``fx.GraphModule``."""

    lw = _Lowering(traced, promoted_constants)
    outputs: tuple[str, ...] = ()
    for node in traced.graph.nodes:
        if node in lw.skip:
            continue
        if node.op == "placeholder":
            value_id = f"arg{len(lw.inputs)}"
            lw.values[value_id] = Value(value_id, lw.node_type(node))
            lw.inputs.append(value_id)
            lw.ids[node] = value_id
        elif node.op == "get_attr":
            if getattr(_constant(traced, node), "numel", lambda: 1)() == 0:
                continue  # an empty constant: whatever uses it drops it
            if promoted_constants is None:
                raise UnsupportedOperationError(
                    f"the trace captured tensor {node.target!r} as a constant; pass it as an "
                    "input or register it as a buffer"
                )
            constant = _constant(traced, node)
            value_id = f"arg{len(lw.inputs)}"
            lw.values[value_id] = Value(value_id, tensor_type_of(constant, f"constant {node.target!r}"))
            lw.inputs.append(value_id)
            lw.ids[node] = value_id
            promoted_constants.append(constant)
        elif node.op == "call_function":
            if node in lw.ids:
                continue
            if not node.users:
                continue
            target = str(node.target)
            handler = HANDLERS.get(target)
            if handler is None:
                for suffix, candidate in _SUFFIX_HANDLERS.items():
                    if target.endswith(suffix):
                        handler = candidate
            if handler is None:
                raise UnsupportedOperationError(
                    f"unsupported FX target: {target}",
                    hint="the cuda-sm100 frontend lowers the operator set of the static-cache "
                    "decoder graphs; run other operators outside the compiled region",
                )
            handler(lw, node)
        elif node.op == "output":
            flat = []

            def collect(item):
                if isinstance(item, (tuple, list)):
                    for sub in item:
                        collect(sub)
                elif isinstance(item, torch.fx.Node):
                    flat.append(lw.arg(item))
                elif item is not None:
                    raise CompilationError(f"unsupported graph output {item!r}")

            collect(node.args[0])
            outputs = tuple(flat)
        else:
            raise CompilationError(f"unsupported FX node kind: {node.op}")
    return Graph(tuple(lw.inputs), lw.values, tuple(lw.ops), outputs)
