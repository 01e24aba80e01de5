"""Fusion passes of the rewrite pipeline.

Each pass is ``Graph -> Graph`` and matches narrowly (absorbed values have one
consumer and are not graph outputs). Operand-order conventions of the fused
operations, which the backend binds kernels by:

* packed ``matmul``: ``(x, Wp, S[, Wp2, S2][, gate][, w_norm])``
* packed ``addmm``:  ``(bias_or_residual, x, Wp, S[, w_norm])``
* dense forms carry the weight in place of ``Wp, S``.

Behavioural counterparts of ``src/aotolith/passes/fusion.py``,
``passes/norm.py`` and ``passes/matchers/*`` in the reference.
"""

from __future__ import annotations

from ..ir import Graph, Operation, TensorType
from .rewriter import Rewriter, see_through_reshapes

#: operations a pointwise region may contain
POINTWISE_OPS = frozenset(
    {"add", "sub", "mul", "div", "neg", "silu", "sigmoid", "exp", "tanh", "relu", "gelu",
     "where", "scalar_tensor", "cast", "cos", "sin"}
)


def fuse_attention(graph: Graph) -> Graph:
    """Decomposed QK^T/softmax/PV -> ``attention``.

    SDPA reaches the IR as one ``attention`` node already (the legaliser maps
    every ATen SDPA variant onto it), so there is nothing to match in the
    graphs this frontend captures; the pass keeps its slot in the pipeline.
    """

    return graph


# ---------------------------------------------------------------------------
# norm scale
# ---------------------------------------------------------------------------

def fuse_norm_scale(graph: Graph) -> Graph:
    """``cast(mul(rms_norm(cast(x)), w))`` -> ``rms_norm(x, w){has_weight}``.

    The norm already computes in fp32 and rounds once, so the fold is
    bit-identical.
    """

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "rms_norm" or op.attrs.get("has_weight", False) or len(op.inputs) != 1:
            continue
        normed = op.outputs[0]
        if not rw.single_use(normed):
            continue
        scale = rw.users(normed)[0]
        if scale.op != "mul" or normed not in scale.inputs:
            continue
        weight = scale.inputs[1] if scale.inputs[0] == normed else scale.inputs[0]
        weight_producer = rw.producer(weight)
        if weight_producer is not None and weight_producer.op == "cast":
            weight = weight_producer.inputs[0]
        width = int(op.attrs["normalized_shape"][-1])
        if rw.shape(weight) != (width,):
            continue
        result = scale.outputs[0]
        tail = None
        if rw.single_use(result):
            candidate = rw.users(result)[0]
            if candidate.op == "cast":
                tail = candidate
        source = op.inputs[0]
        head = rw.producer(source)
        if head is not None and head.op == "cast":
            source = head.inputs[0]
        final = tail.outputs[0] if tail is not None else result
        if tail is not None and rw.type(final).dtype != rw.type(source).dtype:
            continue
        attrs = dict(op.attrs)
        attrs["has_weight"] = True
        fused = Operation("rms_norm", (source, weight), (final,), attrs)
        if tail is not None:
            rw.erase(op, scale)
            rw.replace(tail, fused)
        else:
            rw.erase(op)
            rw.replace(scale, fused)
    return rw.finish()


# ---------------------------------------------------------------------------
# rope
# ---------------------------------------------------------------------------

def _match_rotate_half(rw: Rewriter, value_id: str):
    """``cat(neg(x[..., D/2:]), x[..., :D/2])`` -> ``x`` or None."""

    cat = rw.producer(value_id)
    if cat is None or cat.op != "cat" or len(cat.inputs) != 2 or not rw.single_use(value_id):
        return None
    rank = len(rw.shape(value_id))
    if int(cat.attrs["dim"]) % rank != rank - 1:
        return None
    neg = rw.producer(cat.inputs[0])
    low = rw.producer(cat.inputs[1])
    if neg is None or low is None or neg.op != "neg" or low.op != "slice":
        return None
    high = rw.producer(neg.inputs[0])
    if high is None or high.op != "slice" or high.inputs[0] != low.inputs[0]:
        return None
    source = low.inputs[0]
    width = rw.shape(source)[-1]
    half = width // 2
    if width % 2:
        return None
    for piece, (start, end) in ((high, (half, width)), (low, (0, half))):
        if int(piece.attrs["dim"]) % rank != rank - 1 or int(piece.attrs.get("step", 1)) != 1:
            return None
        if int(piece.attrs["start"]) != start or min(int(piece.attrs["end"]), width) != end:
            return None
    if not (rw.single_use(cat.inputs[0]) and rw.single_use(cat.inputs[1]) and rw.single_use(neg.inputs[0])):
        return None
    return source


def fuse_rope(graph: Graph) -> Graph:
    """``x*cos + rotate_half(x)*sin`` -> ``rope(x, cos, sin)``."""

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "add" or float(op.attrs.get("alpha", 1.0)) != 1.0 or len(op.inputs) != 2:
            continue
        terms = [rw.producer(v) for v in op.inputs]
        if any(t is None or t.op != "mul" for t in terms):
            continue
        if not all(rw.single_use(v) for v in op.inputs):
            continue
        match = None
        for straight, turned in ((terms[0], terms[1]), (terms[1], terms[0])):
            for rotated_id, sine in (turned.inputs, turned.inputs[::-1]):
                source = _match_rotate_half(rw, rotated_id)
                if source is None:
                    continue
                if source not in straight.inputs:
                    continue
                cosine = straight.inputs[1] if straight.inputs[0] == source else straight.inputs[0]
                match = (source, cosine, sine)
                break
            if match:
                break
        if match is None:
            continue
        source, cosine, sine = match
        width = rw.shape(source)[-1]
        if rw.type(cosine).dtype != rw.type(sine).dtype:
            continue
        if rw.shape(cosine)[-1] not in (1, width) or rw.shape(sine)[-1] not in (1, width):
            continue
        rw.replace(op, Operation("rope", (source, cosine, sine), op.outputs, {}))
    return rw.finish()


# ---------------------------------------------------------------------------
# residual epilogue
# ---------------------------------------------------------------------------

def _matmul_behind(rw: Rewriter, value_id: str, limit: int = 2):
    """``value_id`` as at most ``limit`` single-use reshapes of a single-use matmul."""

    hops = 0
    while True:
        op = rw.producer(value_id)
        if op is None or not rw.single_use(value_id):
            return None
        if op.op == "matmul":
            return op
        if op.op != "reshape" or hops == limit:
            return None
        value_id = op.inputs[0]
        hops += 1


def fuse_residual_epilogue(graph: Graph) -> Graph:
    """``residual + matmul(...)`` -> ``addmm(residual, x, W...){alpha=beta=1}``."""

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "add" or float(op.attrs.get("alpha", 1.0)) != 1.0 or len(op.inputs) != 2:
            continue
        chosen = None
        for product_id, residual_id in (op.inputs[::-1], op.inputs):
            product = _matmul_behind(rw, product_id)
            if product is None or "epilogue" in product.attrs:
                continue
            if rw.type(residual_id).numel != rw.type(product.outputs[0]).numel:
                continue
            if rw.type(residual_id).dtype != rw.type(product.outputs[0]).dtype:
                continue
            chosen = (product, residual_id)
            break
        if chosen is None:
            continue
        product, residual_id = chosen
        product_type = rw.type(product.outputs[0])
        new_ops = []
        if rw.shape(residual_id) != product_type.shape:
            reshaped = rw.named_value(f"{residual_id}_epilogue", TensorType(product_type.shape, product_type.dtype))
            new_ops.append(Operation("reshape", (residual_id,), (reshaped,), {"shape": product_type.shape}))
            residual_id = reshaped
        attrs = dict(product.attrs)
        attrs["alpha"] = 1.0
        attrs["beta"] = 1.0
        out_type = rw.type(op.outputs[0])
        if out_type.shape == product_type.shape:
            new_ops.append(Operation("addmm", (residual_id,) + product.inputs, op.outputs, attrs))
        else:
            total = rw.new_value(product_type, "v")
            new_ops.append(Operation("addmm", (residual_id,) + product.inputs, (total,), attrs))
            new_ops.append(Operation("reshape", (total,), op.outputs, {"shape": out_type.shape}))
        rw.replace(op, *new_ops)
    return rw.finish()


# ---------------------------------------------------------------------------
# pointwise regions
# ---------------------------------------------------------------------------

def fuse_pointwise(graph: Graph) -> Graph:
    """Maximal single-use pointwise regions (two or more operations) -> ``fused_elementwise``."""

    rw = Rewriter(graph)
    region_of: dict[str, int] = {}   # value id -> region
    members: dict[int, list[Operation]] = {}
    next_region = 0
    for op in rw.ops:
        if op.op not in POINTWISE_OPS or len(op.outputs) != 1:
            continue
        region = next_region
        next_region += 1
        members[region] = []
        for value in op.inputs:
            inner = region_of.get(value)
            if inner is None or inner == region or not rw.single_use(value):
                continue
            members[region] = members.pop(inner) + members[region]
            for key, owner in list(region_of.items()):
                if owner == inner:
                    region_of[key] = region
        members[region].append(op)
        region_of[op.outputs[0]] = region
    for ops in members.values():
        if len(ops) < 2:
            continue
        order = {id(op): index for index, op in enumerate(rw.ops)}
        ops = sorted(ops, key=lambda item: order[id(item)])
        produced = {out for item in ops for out in item.outputs}
        external: list[str] = []
        for item in ops:
            for value in item.inputs:
                if value not in produced and value not in external:
                    external.append(value)
        root = ops[-1]
        fused = Operation("fused_elementwise", tuple(external), root.outputs, {"body": tuple(ops)})
        rw.erase(*ops[:-1])
        rw.replace(root, fused)
    return rw.finish()


def _silu_mul_body(op: Operation):
    """``(gate, up)`` if ``op`` is ``fused_elementwise[silu(gate) -> s, mul(s, up)]``."""

    if op.op != "fused_elementwise":
        return None
    body = op.attrs.get("body", ())
    if len(body) != 2 or body[0].op != "silu" or body[1].op != "mul":
        return None
    activated = body[0].outputs[0]
    if activated not in body[1].inputs or body[1].outputs != op.outputs:
        return None
    gate = body[0].inputs[0]
    up = body[1].inputs[1] if body[1].inputs[0] == activated else body[1].inputs[0]
    if up == activated:
        return None
    return gate, up


def _is_packed(op: Operation) -> bool:
    return "weight_group_size" in op.attrs


def fuse_gate_up_projection(graph: Graph) -> Graph:
    """Two projections of one activation row joined by ``silu(a)*b`` -> one paired matmul."""

    rw = Rewriter(graph)
    for op in list(rw.ops):
        pair = _silu_mul_body(op)
        if pair is None:
            continue
        gate_mm = _matmul_behind(rw, pair[0])
        up_mm = _matmul_behind(rw, pair[1])
        if gate_mm is None or up_mm is None or gate_mm is up_mm:
            continue
        if gate_mm.attrs != up_mm.attrs or "epilogue" in gate_mm.attrs:
            continue
        if len(gate_mm.inputs) != len(up_mm.inputs):
            continue
        if rw.shape(gate_mm.inputs[0]) != rw.shape(up_mm.inputs[0]) or see_through_reshapes(
            rw, gate_mm.inputs[0]
        ) != see_through_reshapes(rw, up_mm.inputs[0]):
            continue
        if rw.type(gate_mm.outputs[0]) != rw.type(up_mm.outputs[0]):
            continue
        left_shape = rw.shape(gate_mm.inputs[0])
        rows = 1
        for dim in left_shape[:-1]:
            rows *= dim
        inner = left_shape[-1]
        if rows != 1:
            continue
        if _is_packed(gate_mm):
            if inner % 8 or gate_mm.attrs.get("transpose_b", False) or len(gate_mm.inputs) != 3:
                continue
        elif inner % 4 or len(gate_mm.inputs) != 2:
            continue
        attrs = dict(gate_mm.attrs)
        attrs["epilogue"] = "silu_mul_paired"
        inputs = gate_mm.inputs + up_mm.inputs[1:]
        product_type = rw.type(gate_mm.outputs[0])
        out_type = rw.type(op.outputs[0])
        if out_type.shape == product_type.shape:
            rw.replace(op, Operation("matmul", inputs, op.outputs, attrs))
        else:
            joined = rw.new_value(product_type, "v")
            rw.replace(
                op,
                Operation("matmul", inputs, (joined,), attrs),
                Operation("reshape", (joined,), op.outputs, {"shape": out_type.shape}),
            )
    return rw.finish()


def fuse_activation_epilogue(graph: Graph) -> Graph:
    """``silu(gate) * up`` folded into the up projection: ``matmul(x, Wu, gate){epilogue="silu_mul"}``."""

    rw = Rewriter(graph)
    for op in list(rw.ops):
        pair = _silu_mul_body(op)
        if pair is None:
            continue
        gate_id, up_id = pair
        up_mm = _matmul_behind(rw, up_id)
        if up_mm is None or "epilogue" in up_mm.attrs:
            continue
        product_type = rw.type(up_mm.outputs[0])
        if rw.type(gate_id).numel != product_type.numel:
            continue
        # read the gate in the projection's own shape, reusing an existing value when one has it
        source = gate_id
        while rw.shape(source) != product_type.shape:
            producer = rw.producer(source)
            if producer is None or producer.op != "reshape":
                break
            source = producer.inputs[0]
        new_ops = []
        if rw.shape(source) != product_type.shape:
            source = rw.named_value(f"{gate_id}_epilogue", product_type)
            new_ops.append(Operation("reshape", (gate_id,), (source,), {"shape": product_type.shape}))
        # the gate must already exist where the up projection runs
        order = {id(item): index for index, item in enumerate(rw.ops)}
        gate_producer = rw.producer(source)
        if gate_producer is not None and order[id(gate_producer)] > order[id(op)]:
            continue
        attrs = dict(up_mm.attrs)
        attrs["epilogue"] = "silu_mul"
        inputs = up_mm.inputs + (source,)
        out_type = rw.type(op.outputs[0])
        if out_type.shape == product_type.shape:
            new_ops.append(Operation("matmul", inputs, op.outputs, attrs))
        else:
            joined = rw.new_value(product_type, "v")
            new_ops.append(Operation("matmul", inputs, (joined,), attrs))
            new_ops.append(Operation("reshape", (joined,), op.outputs, {"shape": out_type.shape}))
        rw.replace(op, *new_ops)
    return rw.finish()


# ---------------------------------------------------------------------------
# rms norm into the projection that consumes it
# ---------------------------------------------------------------------------

def _activation_slot(op: Operation) -> int:
    return 1 if op.op == "addmm" else 0


def fuse_rms_norm_epilogue(graph: Graph, *, native_matmul: bool = False) -> Graph:
    """Fold ``rms_norm(x, w)`` into the single-row projections that consume it.

    Applies when every consumer (through reshapes) is a ``matmul``/``addmm``
    reading it as the activation, the whole tensor is one row whose width is a
    multiple of eight, and the projection is packed (always) or dense with
    ``native_matmul``. The norm weight is appended as the projection's last
    operand and ``rms_norm_eps`` recorded.
    """

    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "rms_norm" or not op.attrs.get("has_weight", False) or len(op.inputs) != 2:
            continue
        normed = op.outputs[0]
        if rw.is_output(normed):
            continue
        norm_type = rw.type(normed)
        width = norm_type.shape[-1]
        if norm_type.numel != width or width % 8:
            continue
        if tuple(op.attrs.get("normalized_shape", ())) != (width,):
            continue
        # collect (projection, value it reads) through reshape chains
        frontier = [normed]
        readers: list[tuple[Operation, str]] = []
        views: list[Operation] = []
        ok = True
        while frontier and ok:
            value = frontier.pop()
            if value != normed and rw.is_output(value):
                ok = False
                break
            for user in rw.users(value):
                if user.op == "reshape":
                    views.append(user)
                    frontier.append(user.outputs[0])
                elif user.op in ("matmul", "addmm") and user.inputs[_activation_slot(user)] == value:
                    if user.inputs.count(value) != 1 or "rms_norm_eps" in user.attrs:
                        ok = False
                    elif not (_is_packed(user) or native_matmul):
                        ok = False
                    else:
                        readers.append((user, value))
                else:
                    ok = False
        if not ok or not readers:
            continue
        source, weight = op.inputs
        for reader, value in readers:
            current = next(item for item in rw.ops if item.outputs == reader.outputs)
            wanted = rw.type(value)
            if rw.shape(source) == wanted.shape:
                feed = source
            else:
                feed = rw.new_value(TensorType(wanted.shape, rw.type(source).dtype), "v")
                rw.insert_before(current, Operation("reshape", (source,), (feed,), {"shape": wanted.shape}))
            slot = _activation_slot(current)
            inputs = list(current.inputs)
            inputs[slot] = feed
            inputs.append(weight)
            attrs = dict(current.attrs)
            attrs["rms_norm_eps"] = float(op.attrs["eps"])
            rw.replace(current, Operation(current.op, tuple(inputs), current.outputs, attrs))
    return rw.finish()
