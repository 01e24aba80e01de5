"""Lowered decode graph -> stage program of the persistent decode-step kernel.

``build_step_program(graph)`` walks the lowered decode graph in order and
recognises it as a chain of three stage kinds (``include/aoto_sm100.h``):

* ``GEMV``      a packed ``matmul`` / ``addmm`` over one activation row, with its
                norm, bias/residual and paired-SiLU epilogue; when the activation
                is an ``embedding`` of the step's token the gather is folded in;
* ``ATTENTION`` ``rope_kv_cache_append`` + the boolean-mask conversion + the
                ``attention`` that reads the appended window;
* ``PICK``      (added by the greedy stepper, not part of the graph) the greedy
                token from the LM-head stage's per-CTA maxima.

Everything else in the graph must be a view (``reshape`` / ``unsqueeze``), a
table gather the attention stage performs itself (rotary rows by position) or
the closing ``cat`` that assembles the next cache from the per-layer pairs. A
graph with any other operation has no program (``None``) and runs operation by
operation instead.

The program is symbolic: operands are references to graph inputs, to
intermediates (placed in one arena at the offsets the storage plan assigned)
or to the two outputs. ``bind`` turns it into the device array the kernel reads.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from .. import _native as N
from ..ir import DType, Graph


@dataclass(frozen=True, slots=True)
class Ref:
    """Where a stage operand lives: ``("input", id)``, ``("arena", id)`` or ``("output", index)``."""

    space: str
    key: object
    offset: int = 0  # bytes from the start of that buffer


@dataclass(slots=True)
class StageSpec:
    kind: int
    op_indices: tuple[int, ...]
    refs: dict[str, Ref] = field(default_factory=dict)
    ints: dict[str, int] = field(default_factory=dict)
    floats: dict[str, float] = field(default_factory=dict)
    flags: int = 0


@dataclass(slots=True)
class StepProgram:
    stages: list[StageSpec]
    token_input: str
    position_input: str
    mask_input: str
    cache_input: str
    logits_output: str
    cache_output: str
    arena_bytes: int
    arena_offsets: dict[str, int]
    vocab: int
    capacity: int


def _numel(shape) -> int:
    count = 1
    for dim in shape:
        count *= dim
    return count


class _Unsupported(Exception):
    pass


def build_step_program(graph: Graph) -> StepProgram | None:
    try:
        return _build(graph)
    except _Unsupported:
        return None


def _build(graph: Graph) -> StepProgram:
    if len(graph.outputs) != 2:
        raise _Unsupported
    value = graph.value
    inputs = set(graph.inputs)
    # Every stage result gets its own region of the arena (a few KB each): a step's
    # intermediates are tiny next to its weights, and a region that is written once per
    # launch needs no reasoning about reuse between stages that run on different SMs.
    offsets: dict[str, int] = {}
    arena_top = 0

    # symbolic environment: what each value IS for the kernel
    env: dict[str, tuple] = {}
    for value_id in graph.inputs:
        env[value_id] = ("tensor", Ref("input", value_id))

    def tensor_ref(value_id: str) -> Ref:
        kind = env.get(value_id)
        if kind is None or kind[0] != "tensor":
            raise _Unsupported
        return kind[1]

    # a value whose view (reshape chain) is a graph output lives in that output buffer
    lands_in: dict[str, int] = {out: i for i, out in enumerate(graph.outputs)}
    for op in reversed(graph.ops):
        if op.op in ("reshape", "unsqueeze", "squeeze") and op.outputs[0] in lands_in:
            lands_in.setdefault(op.inputs[0], lands_in[op.outputs[0]])

    def place(value_id: str) -> Ref:
        if value_id in lands_in:
            return Ref("output", lands_in[value_id])
        nonlocal arena_top
        if value_id not in offsets:
            offsets[value_id] = arena_top
            # a stamped vector: 8 bytes per two bf16 values
            arena_top += (value(value_id).type.numel * 4 + 255) // 256 * 256
        return Ref("arena", value_id, 0)

    stages: list[StageSpec] = []
    token_input = position_input = mask_input = cache_input = None
    appended: dict[str, dict] = {}   # keys value id -> pending attention description
    pairs: dict[str, int] = {}       # new_pair value id -> layer
    cache_output = None

    for index, op in enumerate(graph.ops):
        kind = op.op
        out = op.outputs[0]
        if kind == "embedding":
            table, ids = op.inputs
            if table not in inputs or ids not in inputs:
                raise _Unsupported
            if value(ids).type.shape != (1, 1) or value(table).type.dtype != DType.BF16:
                raise _Unsupported
            env[out] = ("gather", table, ids, index)
        elif kind in ("reshape", "unsqueeze", "squeeze"):
            source = env.get(op.inputs[0])
            if source is None:
                raise _Unsupported
            if source[0] in ("tensor", "gather", "mask", "pair"):
                env[out] = source  # contiguous data, same bytes
            else:
                raise _Unsupported
        elif kind == "fused_elementwise":
            body = op.attrs.get("body", ())
            constants = {b.outputs[0]: float(b.attrs["value"]) for b in body if b.op == "scalar_tensor"}
            where = body[-1] if body else None
            if (where is None or where.op != "where" or len(op.inputs) != 1 or op.inputs[0] not in inputs
                    or constants.get(where.inputs[1]) != 0.0
                    or constants.get(where.inputs[2]) != float("-inf")
                    or value(op.inputs[0]).type.dtype != DType.BOOL):
                raise _Unsupported
            env[out] = ("mask", op.inputs[0])
            mask_input = op.inputs[0]
        elif kind in ("matmul", "addmm"):
            if "weight_group_size" not in op.attrs or int(op.attrs.get("weight_bits", 4)) != 4:
                raise _Unsupported
            if int(op.attrs["weight_group_size"]) != 64 or op.attrs.get("epilogue") == "silu_mul":
                raise _Unsupported
            is_addmm = kind == "addmm"
            base = 1 if is_addmm else 0
            x_id = op.inputs[base]
            x_shape = value(x_id).type.shape
            if _numel(x_shape) != x_shape[-1] or value(x_id).type.dtype != DType.BF16:
                raise _Unsupported
            spec = StageSpec(N.STAGE_GEMV, (index,))
            source = env.get(x_id)
            if source is None:
                raise _Unsupported
            if source[0] == "gather":
                _, table, ids, _ = source
                spec.refs["x"] = Ref("input", table)
                spec.refs["x_index"] = Ref("input", ids)
                spec.ints["x_rows"] = value(table).type.shape[0]
                spec.flags |= N.STAGE_FLAG_X_GATHER
                token_input = ids
            else:
                spec.refs["x"] = tensor_ref(x_id)
            spec.refs["packed"] = tensor_ref(op.inputs[base + 1])
            spec.refs["scales"] = tensor_ref(op.inputs[base + 2])
            position = base + 3
            epilogue = N.EPILOGUE_NONE
            if op.attrs.get("epilogue") == "silu_mul_paired":
                spec.refs["packed2"] = tensor_ref(op.inputs[position])
                spec.refs["scales2"] = tensor_ref(op.inputs[position + 1])
                position += 2
                epilogue = N.EPILOGUE_SILU_MUL_PAIRED
            if "rms_norm_eps" in op.attrs:
                spec.refs["norm_weight"] = tensor_ref(op.inputs[position])
                spec.floats["rms_norm_eps"] = float(op.attrs["rms_norm_eps"])
                position += 1
            if position != len(op.inputs):
                raise _Unsupported
            n_rows, words = value(op.inputs[base + 1]).type.shape
            if words * 8 != x_shape[-1]:
                raise _Unsupported
            addend_mode = N.STAGE_ADDEND_NONE
            if is_addmm:
                addend_id = op.inputs[0]
                if _numel(value(addend_id).type.shape) != n_rows:
                    raise _Unsupported
                source = env.get(addend_id)
                if source is None:
                    raise _Unsupported
                if source[0] == "gather":
                    # the residual of the first layer is the embedding row itself
                    _, table, ids, _ = source
                    if value(table).type.shape[1] != n_rows:
                        raise _Unsupported
                    spec.refs["addend"] = Ref("input", table)
                    spec.refs.setdefault("x_index", Ref("input", ids))
                    spec.ints.setdefault("x_rows", value(table).type.shape[0])
                    if spec.refs["x_index"] != Ref("input", ids):
                        raise _Unsupported
                    addend_mode = N.STAGE_ADDEND_GATHER
                else:
                    spec.refs["addend"] = tensor_ref(addend_id)
                    addend_mode = (
                        N.STAGE_ADDEND_PLAIN if spec.refs["addend"].space == "input" else N.STAGE_ADDEND_STAMPED
                    )
            spec.ints.update(N=n_rows, K=words * 8, group_size=64, addend_mode=addend_mode, epilogue=epilogue)
            spec.floats.update(alpha=float(op.attrs.get("alpha", 1.0)), beta=float(op.attrs.get("beta", 1.0)))
            spec.refs["out"] = place(out)
            if spec.refs["out"].space == "output":
                spec.flags |= N.STAGE_FLAG_OUT_PLAIN
            env[out] = ("tensor", spec.refs["out"])
            stages.append(spec)
        elif kind == "rope_kv_cache_append":
            cache, row, cosine, sine = op.inputs
            if cache not in inputs:
                raise _Unsupported
            cos_src, sin_src = env.get(cosine), env.get(sine)
            if not cos_src or not sin_src or cos_src[0] != "gather" or sin_src[0] != "gather":
                raise _Unsupported
            if cos_src[2] != sin_src[2]:
                raise _Unsupported
            cache_input, position_input = cache, cos_src[2]
            query, pair, keys, values = op.outputs
            description = dict(
                index=index, cache=cache, row=tensor_ref(row), cos=cos_src[1], sin=sin_src[1],
                position=cos_src[2], pair=pair, query=query, values=values, attrs=dict(op.attrs),
            )
            appended[keys] = description
            env[pair] = ("pair", int(op.attrs["layer"]))
            pairs[pair] = int(op.attrs["layer"])
            env[query] = ("query", keys)
            env[keys] = ("keys", keys)
            env[values] = ("values", keys)
        elif kind == "attention":
            if len(op.inputs) != 4 or op.attrs.get("causal", False):
                raise _Unsupported
            query, keys, values, mask = op.inputs
            description = appended.get(keys)
            mask_src = env.get(mask)
            if (description is None or env.get(query) != ("query", keys) or env.get(values) != ("values", keys)
                    or not mask_src or mask_src[0] != "mask"):
                raise _Unsupported
            cache_shape = value(description["cache"]).type.shape
            layers, _, batch, kv_heads, capacity, head_dim = cache_shape
            query_heads = int(description["attrs"]["query_heads"])
            if batch != 1 or value(mask_src[1]).type.shape != (1, 1, 1, capacity):
                raise _Unsupported
            layer = int(description["attrs"]["layer"])
            pair_bytes = 2 * kv_heads * capacity * head_dim * 2
            spec = StageSpec(N.STAGE_ATTENTION, (description["index"], index))
            spec.refs.update(
                row=description["row"],
                cos_table=Ref("input", description["cos"]),
                sin_table=Ref("input", description["sin"]),
                position=Ref("input", description["position"]),
                cache_in=Ref("input", description["cache"], layer * pair_bytes),
                cache_out=Ref("output", 1, layer * pair_bytes),
                mask=Ref("input", mask_src[1]),
                attn_out=place(out),
            )
            spec.ints.update(
                query_heads=query_heads, kv_heads=kv_heads, capacity=capacity, head_dim=head_dim,
                query_start=int(description["attrs"]["query_start"]),
                key_start=int(description["attrs"]["key_start"]),
                value_start=int(description["attrs"]["value_start"]),
                table_rows=value(description["cos"]).type.shape[0],
            )
            spec.floats["scale"] = float(op.attrs["scale"])
            env[out] = ("tensor", spec.refs["attn_out"])
            stages.append(spec)
        elif kind == "cat":
            layers_seen = []
            for part in op.inputs:
                source = env.get(part)
                if not source or source[0] != "pair":
                    raise _Unsupported
                layers_seen.append(source[1])
            if layers_seen != list(range(len(layers_seen))) or out != graph.outputs[1]:
                raise _Unsupported
            cache_output = out
            env[out] = ("tensor", Ref("output", 1))
        else:
            raise _Unsupported

    logits_output = graph.outputs[0]
    final = env.get(logits_output)
    if (final is None or final[0] != "tensor" or final[1].space != "output" or cache_output is None
            or token_input is None or position_input is None or mask_input is None or cache_input is None):
        raise _Unsupported
    if not stages or stages[-1].kind != N.STAGE_GEMV or stages[-1].refs["out"].space != "output":
        raise _Unsupported
    if len(pairs) != value(cache_input).type.shape[0]:
        raise _Unsupported
    capacity = value(cache_input).type.shape[4]
    return StepProgram(
        stages=stages, token_input=token_input, position_input=position_input, mask_input=mask_input,
        cache_input=cache_input, logits_output=logits_output, cache_output=cache_output,
        arena_bytes=max(arena_top, 256), arena_offsets=offsets,
        vocab=_numel(value(logits_output).type.shape), capacity=capacity,
    )


def stage_array(program: StepProgram, resolve, *, greedy: dict | None = None):
    """ctypes array of ``aoto_step_stage`` for ``program``.

    ``resolve(ref) -> int`` maps a reference to a device address. ``greedy``
    (``token``, ``generated``, ``counters`` device addresses and
    ``generated_capacity``) appends the pick stage and makes every attention
    stage derive the step's position and window from the counters.
    """

    count = len(program.stages) + (1 if greedy else 0)
    array = (N.StepStage * count)()
    for slot, spec in enumerate(program.stages):
        stage = array[slot]
        stage.kind = spec.kind
        stage.flags = spec.flags
        for name, ref in spec.refs.items():
            setattr(stage, name, resolve(ref))
        for name, number in spec.ints.items():
            setattr(stage, name, number)
        for name, number in spec.floats.items():
            setattr(stage, name, number)
    if greedy:
        last = array[len(program.stages) - 1]
        last.flags |= N.STAGE_FLAG_ARGMAX
        for slot, spec in enumerate(program.stages):
            if spec.kind == N.STAGE_ATTENTION:
                array[slot].flags |= N.STAGE_FLAG_WINDOW
                array[slot].counters = greedy["counters"]
        pick = array[count - 1]
        pick.kind = N.STAGE_PICK
        pick.token = greedy["token"]
        pick.generated = greedy["generated"]
        pick.counters = greedy["counters"]
        pick.generated_capacity = greedy["generated_capacity"]
    return array


def to_device(array, device: torch.device) -> torch.Tensor:
    raw = bytes(array)
    host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    return host.to(device)


def supported(array) -> bool:
    return bool(N.load().aoto_sm100_decode_step_supported(array, len(array)))


def scratch_bytes(array) -> int:
    return int(N.load().aoto_sm100_decode_step_scratch_bytes(array, len(array)))


def launch(stages_dev: torch.Tensor, count: int, epoch: int, status: torch.Tensor,
           scratch: torch.Tensor, ctas: int = 0, trace: torch.Tensor | None = None) -> None:
    """One decode step. ``epoch`` must be non-zero and new for the arena; ``trace``
    (int64 ``[count * 4]``) collects CTA 0's per-stage timestamps."""

    args = N.DecodeStepArgs(stages_dev.data_ptr(), count, ctas, epoch & 0xFFFFFFFF or 1, 0, status.data_ptr(),
                            scratch.data_ptr(), scratch.numel(),
                            trace.data_ptr() if trace is not None else None)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    N.check(N.load().aoto_sm100_decode_step(ctypes.byref(args), stream), "aoto_sm100_decode_step")
