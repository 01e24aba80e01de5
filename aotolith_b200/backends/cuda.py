"""The ``cuda-sm100`` backend: lowered graph -> plan of sm_100a kernel launches.

``CudaBackend.compile(graph, *, tune_inputs=None) -> CompiledPlan`` is the whole
interface (the reference's ``Backend`` protocol,
``src/aotolith/backends/__init__.py:41-55``). For every operation it records
one ``KernelSelection`` (implementation ``"cuda_kernel"``, ``"view"`` or
``"copy"``, with the reason) and one callable keyed by the operation's first
output id, as ``src/aotolith/backends/reference.py:59-96`` and the Apple
backend do for their targets.

Selection is per operation plus two whole-graph decisions the kernels make
possible:

* a ``dequantize_i4`` whose only readers are ``matmul``/``addmm{transpose_b}``
  is not materialised: the reader launches the packed GEMM, which unpacks the
  weight on the fly with the same rounding (``bf16(code) * bf16(scale)``);
* the per-layer cache pairs a decode step produces are written directly into
  the tensor the closing ``cat`` returns, so the step copies each window once.

There is no interpreter behind this backend: an operation without a kernel (or
a dtype the kernels do not cover) fails compilation with the operation named.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from .. import ops
from .._log import logger
from ..errors import CompilationError, UnsupportedDTypeError, UnsupportedOperationError
from ..ir import DType, Graph, Operation
from ..planning import plan_storage
from ..runtime.plan import CompiledPlan, KernelArtifact, current_context
from ..runtime.step_program import build_step_program
from ..selection import COPY, CUDA_KERNEL, VIEW, KernelSelection

TARGET = "cuda-sm100"
ARCHITECTURE = "sm_100a"


@dataclass(frozen=True, slots=True)
class PackedWeight:
    """A ``dequantize_i4`` / ``dequantize_i8`` result that was never materialised."""

    packed: torch.Tensor
    scales: torch.Tensor
    group_size: int
    bits: int = 4


_UNPACK_BITS = {"dequantize_i4": 4, "dequantize_i8": 8}


def _device_name() -> str:
    if torch.cuda.is_available():
        return torch.cuda.get_device_name(torch.cuda.current_device())
    return "no CUDA device visible at compile time"


class _Builder:
    def __init__(self, graph: Graph) -> None:
        self.graph = graph
        self.callables: dict[str, Callable[..., Any]] = {}
        self.selections: list[KernelSelection] = []
        self.kernels: list[KernelArtifact] = []
        self.device_name = _device_name()
        self.producer = {out: op for op in graph.ops for out in op.outputs}
        self.users: dict[str, list[Operation]] = {}
        for op in graph.ops:
            for value in dict.fromkeys(op.inputs):
                self.users.setdefault(value, []).append(op)
        self.folded_weights = self._find_folded_weights()
        self.cache_destinations, self.elided_cats = self._find_cache_assembly()

    # -- whole-graph decisions -------------------------------------------------
    def _find_folded_weights(self) -> set[str]:
        folded: set[str] = set()
        for op in self.graph.ops:
            if op.op not in _UNPACK_BITS:
                continue
            out = op.outputs[0]
            readers = self.users.get(out, [])
            if not readers or out in self.graph.outputs:
                continue
            ok = True
            for reader in readers:
                if reader.op not in ("matmul", "addmm") or not reader.attrs.get("transpose_b", False):
                    ok = False
                    break
                slot = 2 if reader.op == "addmm" else 1
                if reader.inputs[slot] != out or reader.inputs.count(out) != 1:
                    ok = False
                    break
                if reader.attrs.get("transpose_a", False) or "weight_group_size" in reader.attrs:
                    ok = False
                    break
            if ok and self.graph.value(out).type.dtype == DType.BF16:
                folded.add(out)
        return folded

    def _find_cache_assembly(self):
        """``cat(unsqueeze(pair_0), ..., unsqueeze(pair_{L-1}), dim 0)`` of appended pairs."""

        destinations: dict[str, tuple[str, int]] = {}  # pair value -> (cat output, index)
        elided: set[str] = set()
        for op in self.graph.ops:
            if op.op != "cat" or int(op.attrs.get("dim", 0)) != 0:
                continue
            found = []
            for index, value in enumerate(op.inputs):
                lift = self.producer.get(value)
                if lift is None or lift.op != "unsqueeze" or int(lift.attrs["dim"]) != 0:
                    break
                if len(self.users.get(value, [])) != 1 or value in self.graph.outputs:
                    break
                pair = lift.inputs[0]
                maker = self.producer.get(pair)
                if maker is None or maker.op not in ("rope_kv_cache_append", "kv_cache_append"):
                    break
                slot = 1 if maker.op == "rope_kv_cache_append" else 0
                if maker.outputs[slot] != pair or pair in self.graph.outputs:
                    break
                if len(self.users.get(pair, [])) != 1:
                    break
                found.append((pair, index))
            else:
                if found and self.graph.value(op.outputs[0]).type.shape[0] == len(found):
                    for pair, index in found:
                        destinations[pair] = (op.outputs[0], index)
                    elided.add(op.outputs[0])
        return destinations, elided

    # -- recording -------------------------------------------------------------
    def record(self, index: int, op: Operation, implementation: str, reason: str,
               fn: Callable[..., Any], artifact: str | None = None, params=()) -> None:
        self.callables[op.outputs[0]] = fn
        self.selections.append(
            KernelSelection(
                op_index=index, op=op.op, output_id=op.outputs[0], implementation=implementation,
                kind=op.op, reason=reason, artifact_name=artifact,
                device_name=self.device_name, device_architecture=ARCHITECTURE,
            )
        )
        if implementation == CUDA_KERNEL and artifact is not None:
            self.kernels.append(
                KernelArtifact(name=artifact, kind=op.op, input_ids=op.inputs, output_ids=op.outputs,
                               params=tuple(params))
            )

    def dtype_of(self, value_id: str) -> DType:
        return self.graph.value(value_id).type.dtype

    def shape_of(self, value_id: str) -> tuple[int, ...]:
        return self.graph.value(value_id).type.shape

    def need_bf16(self, op: Operation, *value_ids: str) -> None:
        for value_id in value_ids:
            if self.dtype_of(value_id) != DType.BF16:
                raise UnsupportedDTypeError(
                    f"{op.op}: the cuda-sm100 kernels compute in bfloat16, but {value_id} is "
                    f"{self.dtype_of(value_id).value}",
                    hint="convert the model with .bfloat16() before compiling for this target",
                )


# ---------------------------------------------------------------------------
# per-operation lowering
# ---------------------------------------------------------------------------

def _lower_layout(b: _Builder, index: int, op: Operation) -> bool:
    kind = op.op
    out_shape = b.shape_of(op.outputs[0])
    if kind == "reshape":
        fn = lambda x, _s=out_shape: x.reshape(_s)
    elif kind == "unsqueeze":
        fn = lambda x, _d=int(op.attrs["dim"]): x.unsqueeze(_d)
    elif kind == "squeeze":
        fn = lambda x, _d=int(op.attrs["dim"]): x.squeeze(_d)
    elif kind == "transpose":
        fn = lambda x, _a=int(op.attrs["dim0"]), _b=int(op.attrs["dim1"]): x.transpose(_a, _b)
    elif kind == "expand":
        fn = lambda x, _s=out_shape: x.expand(_s)
    elif kind == "slice":
        dim = int(op.attrs["dim"])
        start, end, step = int(op.attrs["start"]), int(op.attrs["end"]), int(op.attrs.get("step", 1))
        extent = b.shape_of(op.inputs[0])[dim % len(b.shape_of(op.inputs[0]))]
        if start < 0:
            start += extent
        if end < 0:
            end += extent
        end = min(end, extent)
        fn = lambda x, _d=dim, _s=start, _e=end, _st=step: x[(slice(None),) * (_d % x.dim()) + (slice(_s, _e, _st),)]
    elif kind == "cat":
        out = op.outputs[0]
        if out in b.elided_cats:
            def fn(*parts, _out=out):
                context = current_context()
                buffer = context.buffers.pop(_out, None) if context is not None else None
                if buffer is None:
                    return torch.cat(parts, dim=0)
                return buffer
            b.record(index, op, VIEW, "every part was written in place by the operation that made it", fn)
            return True
        dim = int(op.attrs["dim"])
        fn = lambda *parts, _d=dim: torch.cat(parts, dim=_d)
        b.record(index, op, COPY, "concatenation of separately produced parts: one device copy", fn)
        return True
    else:
        return False
    reason = "layout operation: a view of its operand, no data moves"
    if kind == "reshape":
        reason = "layout operation: a view (or one copy when the operand is a strided view)"
    b.record(index, op, VIEW, reason, fn)
    return True


def _lower_embedding(b: _Builder, index: int, op: Operation) -> None:
    b.need_bf16(op, op.inputs[0])
    if b.dtype_of(op.inputs[1]) != DType.I64:
        raise UnsupportedDTypeError(f"embedding indices must be int64, got {b.dtype_of(op.inputs[1]).value}")

    def fn(table, ids):
        context = current_context()
        return ops.embedding(table, ids, bad_index=context.bad_index if context is not None else None)

    b.record(index, op, CUDA_KERNEL, "row gather with the bounds flag of the plan call", fn,
             "aoto_sm100_embedding")


def _lower_mask_region(b: _Builder, index: int, op: Operation) -> None:
    body = op.attrs.get("body", ())
    constants = {item.outputs[0]: float(item.attrs["value"]) for item in body if item.op == "scalar_tensor"}
    where = body[-1] if body else None
    if (
        where is None or where.op != "where" or len(body) != len(constants) + 1
        or len(op.inputs) != 1 or where.inputs[0] != op.inputs[0]
        or where.inputs[1] not in constants or where.inputs[2] not in constants
        or b.dtype_of(op.inputs[0]) != DType.BOOL or b.dtype_of(op.outputs[0]) != DType.BF16
    ):
        kinds = [item.op for item in body]
        raise UnsupportedOperationError(
            f"fused_elementwise region {kinds} has no cuda-sm100 kernel",
            hint="the target lowers the boolean-mask conversion where(mask, a, b); other pointwise "
            "regions of the decoder graphs are folded into matmul epilogues",
        )
    on_true, on_false = constants[where.inputs[1]], constants[where.inputs[2]]
    fn = lambda mask, _t=on_true, _f=on_false: ops.mask_select(mask, _t, _f)
    b.record(index, op, CUDA_KERNEL, "boolean mask to additive mask in one pass", fn,
             "aoto_sm100_mask_select", (("on_true", on_true), ("on_false", on_false)))


def _lower_attention(b: _Builder, index: int, op: Operation) -> None:
    b.need_bf16(op, *op.inputs)
    query_shape = b.shape_of(op.inputs[0])
    if len(query_shape) != 4 or query_shape[0] != 1:
        raise UnsupportedOperationError(
            f"attention over {query_shape}: the cuda-sm100 kernels take [1, heads, length, dim] operands"
        )
    scale, causal = float(op.attrs["scale"]), bool(op.attrs.get("causal", False))
    has_mask = bool(op.attrs.get("has_mask", False))
    decode = query_shape[2] == 1

    def fn(query, key, value, mask=None, _s=scale, _c=causal):
        return ops.attention(query, key, value, mask, scale=_s, causal=_c)

    variant = "decode_split_kv" if decode else "prefill_tiled"
    reason = (
        "single-query attention over the cache: split-KV kernel, fp32 softmax statistics"
        if decode else "multi-query attention: tiled kernel with an online softmax"
    )
    b.record(index, op, CUDA_KERNEL, reason, fn, f"aoto_sm100_attention[{variant}]",
             (("scale", scale), ("causal", causal), ("has_mask", has_mask)))


def _lower_cache_append(b: _Builder, index: int, op: Operation) -> None:
    rotate = op.op == "rope_kv_cache_append"
    b.need_bf16(op, *op.inputs)
    pair_id = op.outputs[1] if rotate else op.outputs[0]
    destination = b.cache_destinations.get(pair_id)
    cat_shape = b.shape_of(destination[0]) if destination else None
    attrs = {key: int(value) for key, value in op.attrs.items()}

    def place(device):
        if destination is None:
            return None
        context = current_context()
        if context is None:
            return None
        buffer = context.buffers.get(destination[0])
        if buffer is None:
            buffer = torch.empty(cat_shape, dtype=torch.bfloat16, device=device)
            context.buffers[destination[0]] = buffer
        return buffer[destination[1]]

    if rotate:
        def fn(cache, row, cosine, sine):
            return ops.rope_kv_cache_append(cache, row, cosine, sine, new_pair=place(cache.device), **attrs)
    else:
        def fn(cache, key, row):
            return ops.kv_cache_append(cache, key, row, new_pair=place(cache.device), **attrs)

    reason = "window shift, rotation and slot write in one kernel"
    if destination is not None:
        reason += "; the pair is written inside the next cache tensor"
    b.record(index, op, CUDA_KERNEL, reason, fn, f"aoto_sm100_kv_cache_append[rotate={int(rotate)}]",
             tuple(attrs.items()))


def _lower_rope(b: _Builder, index: int, op: Operation) -> None:
    b.need_bf16(op, *op.inputs)
    if len(b.shape_of(op.inputs[0])) != 4:
        raise UnsupportedOperationError(f"rope over {b.shape_of(op.inputs[0])}: rank-4 values only")
    b.record(index, op, CUDA_KERNEL, "rotation with the bf16 rounding points of the unfused form",
             lambda x, c, s: ops.rope(x, c, s), "aoto_sm100_rope")


def _lower_rms_norm(b: _Builder, index: int, op: Operation) -> None:
    b.need_bf16(op, *op.inputs)
    width = b.shape_of(op.inputs[0])[-1]
    if tuple(op.attrs.get("normalized_shape", (width,))) != (width,):
        raise UnsupportedOperationError("rms_norm over more than the last axis has no cuda-sm100 kernel")
    eps = float(op.attrs.get("eps", 1e-5))
    if op.attrs.get("has_weight", False):
        fn = lambda x, w, _e=eps: ops.rms_norm(x, w, _e)
    else:
        fn = lambda x, _e=eps: ops.rms_norm(x, None, _e)
    b.record(index, op, CUDA_KERNEL, "one CTA per row, fp32 statistics, one rounding", fn,
             "aoto_sm100_rms_norm", (("eps", eps),))


def _lower_dequantize(b: _Builder, index: int, op: Operation) -> None:
    group = int(op.attrs["group_size"])
    bits = _UNPACK_BITS[op.op]
    if b.dtype_of(op.inputs[1]) != DType.BF16:
        raise UnsupportedDTypeError(f"{op.op}: scales must be bfloat16 on this target")
    if op.outputs[0] in b.folded_weights:
        fn = lambda packed, scales, _g=group, _b=bits: PackedWeight(packed, scales, _g, _b)
        readers = [str(b.graph.ops.index(r)) for r in b.users[op.outputs[0]]]
        b.record(index, op, CUDA_KERNEL,
                 "not materialised: unpacked inside the GEMM of operation " + ", ".join(readers), fn,
                 "aoto_sm100_qmatmul[weight operand]", (("group_size", group), ("weight_bits", bits)))
        return
    if bits == 8:
        fn = lambda packed, scales, _g=group: ops.dequantize_i8(packed, scales, _g)
    else:
        fn = lambda packed, scales, _g=group: ops.dequantize_i4(packed, scales, _g)
    b.record(index, op, CUDA_KERNEL, "streaming unpack, one rounding per element", fn,
             f"aoto_sm100_{op.op}", (("group_size", group),))


def _lower_projection(b: _Builder, index: int, op: Operation) -> None:
    """``matmul`` / ``addmm`` in their packed and dequantised-weight forms."""

    is_addmm = op.op == "addmm"
    attrs = op.attrs
    inputs = list(op.inputs)
    epilogue = attrs.get("epilogue")
    has_norm = "rms_norm_eps" in attrs
    eps = float(attrs.get("rms_norm_eps", 0.0))
    alpha = float(attrs.get("alpha", 1.0))
    beta = float(attrs.get("beta", 1.0))
    base = 1 if is_addmm else 0
    x_id = inputs[base]
    b.need_bf16(op, x_id, op.outputs[0])
    out_shape = b.shape_of(op.outputs[0])
    rows = 1
    for dim in b.shape_of(x_id)[:-1]:
        rows *= dim

    if "weight_group_size" in attrs:
        bits = int(attrs.get("weight_bits", 4))
        if bits not in (4, 8):
            raise UnsupportedOperationError(f"packed projections with {bits}-bit weights have no cuda-sm100 kernel")
        group = int(attrs["weight_group_size"])
        position = base + 3
        paired = epilogue == "silu_mul_paired"
        second = (position, position + 1) if paired else None
        if paired:
            position += 2
        gate_at = None
        if epilogue == "silu_mul":
            gate_at = position
            position += 1
        norm_at = position if has_norm else None
        expected = position + (1 if has_norm else 0)
        if len(inputs) != expected:
            raise CompilationError(f"packed {op.op} has {len(inputs)} operands, expected {expected}")

        def fn(*args, _g=group, _s=out_shape):
            x = args[base]
            out = ops.qmatmul(
                x, args[base + 1], args[base + 2], group_size=_g,
                addend=args[0] if is_addmm else None,
                norm_weight=args[norm_at] if norm_at is not None else None, rms_norm_eps=eps,
                packed2=args[second[0]] if second else None, scales2=args[second[1]] if second else None,
                gate=args[gate_at] if gate_at is not None else None, alpha=alpha, beta=beta,
                weight_bits=bits,
            )
            return out.reshape(_s)

        n_rows, words = b.shape_of(inputs[base + 1])
        per_word = 32 // bits
        variant = ops.qmatmul_variant(rows, n_rows, words * per_word, group, paired, weight_bits=bits)
        reason = "streamed packed words, in-register decode, tensor-pipe accumulate"
        if variant == "qgemv_generic":
            reason = "shape outside the fast variant (group 64, K % 128 == 0): one warp per row"
        if bits == 8:
            reason = "eight-bit words: one warp per weight row, weights rounded to bf16 as code*scale"
        if has_norm:
            reason += "; RMS norm applied while staging the activation"
        if paired:
            reason += "; gate/up pair with the SiLU-mul epilogue"
        b.record(index, op, CUDA_KERNEL, reason, fn, f"aoto_sm100_qmatmul[{variant}]",
                 (("M", rows), ("N", n_rows), ("K", words * per_word), ("group_size", group), ("weight_bits", bits)))
        return

    weight_id = inputs[base + 1]
    if weight_id not in b.folded_weights and _is_dense_projection(b, op, weight_id, has_norm, epilogue):
        _lower_dense_projection(b, index, op, base, rows, out_shape, alpha, beta, epilogue)
        return
    if weight_id not in b.folded_weights or has_norm or epilogue not in (None, "silu_mul"):
        raise UnsupportedOperationError(
            f"dense {op.op} (operand {weight_id}) has no cuda-sm100 kernel: this target covers "
            "4-bit packed projections",
            hint="compile with quantize=<group size>",
        )
    gate_at = base + 2 if epilogue == "silu_mul" else None

    unpack = b.producer[weight_id]
    n_rows, words = b.shape_of(unpack.inputs[0])
    unpack_bits = _UNPACK_BITS[unpack.op]
    variant = ops.qmatmul_variant(rows, n_rows, words * (32 // unpack_bits), int(unpack.attrs["group_size"]),
                                  weight_bits=unpack_bits)
    # The tcgen05 kernel converts its constant weights before it waits for the producer of its
    # activations, so it is launched as a programmatic dependent: in a recorded plan its start and
    # the first weight tiles overlap the tail of the kernel before it.
    dependent = variant == "gemm_tcgen05"

    def fn(*args, _s=out_shape):
        weight = args[base + 1]
        out = ops.qmatmul(
            args[base], weight.packed, weight.scales, group_size=weight.group_size,
            addend=args[0] if is_addmm else None,
            gate=args[gate_at] if gate_at is not None else None, alpha=alpha, beta=beta,
            weight_bits=weight.bits, pdl=dependent,
        )
        return out.reshape(_s)

    b.record(index, op, CUDA_KERNEL,
             "multi-row projection over a packed weight: unpacked to bf16 on the fly, never stored",
             fn, f"aoto_sm100_qmatmul[{variant}]",
             (("M", rows), ("N", n_rows), ("K", words * (32 // unpack_bits)), ("weight_bits", unpack_bits)))


def _is_dense_projection(b: _Builder, op: Operation, weight_id: str, has_norm: bool, epilogue) -> bool:
    """A dense decoder's projection: ``x @ W^T`` with ``W [N, K]`` a bf16 tensor bound to the plan."""

    if has_norm or epilogue not in (None, "silu_mul", "silu_mul_paired") or not op.attrs.get("transpose_b", False):
        return False
    if op.attrs.get("transpose_a", False) or weight_id not in b.graph.inputs:
        return False
    shape = b.shape_of(weight_id)
    return len(shape) == 2 and b.dtype_of(weight_id) == DType.BF16 and shape[1] % 8 == 0


def _lower_dense_projection(b: _Builder, index: int, op: Operation, base: int, rows: int, out_shape, alpha: float,
                            beta: float, epilogue) -> None:
    """``matmul`` / ``addmm`` over a dense bf16 weight (``quantize=None`` decoders)."""

    is_addmm = op.op == "addmm"
    inputs = list(op.inputs)
    paired = epilogue == "silu_mul_paired"
    second_at = base + 2 if paired else None
    gate_at = base + 2 if epilogue == "silu_mul" else None
    expected = base + 2 + (1 if paired or gate_at is not None else 0)
    if len(inputs) != expected:
        raise CompilationError(f"dense {op.op} has {len(inputs)} operands, expected {expected}")
    if paired and rows != 1:
        raise UnsupportedOperationError("the paired gate/up form of a dense projection takes one activation row")
    n_rows, inner = b.shape_of(inputs[base + 1])

    def fn(*args, _s=out_shape):
        out = ops.dmatmul(
            args[base], args[base + 1], addend=args[0] if is_addmm else None,
            weight2=args[second_at] if second_at is not None else None,
            gate=args[gate_at] if gate_at is not None else None, alpha=alpha, beta=beta,
        )
        return out.reshape(_s)

    variant = ops.dmatmul_variant(rows, n_rows, inner, paired)
    if variant == "none":
        raise UnsupportedOperationError(f"no dense kernel for a projection of {rows} x {inner} onto {n_rows} rows")
    reason = "dense bf16 weight: a warp per weight row, fp32 accumulate, rounded once"
    if paired:
        reason += "; gate/up pair with the SiLU-mul epilogue"
    b.record(index, op, CUDA_KERNEL, reason, fn, f"aoto_sm100_qmatmul[{variant}]",
             (("M", rows), ("N", n_rows), ("K", inner), ("weight_bits", 16)))


class CudaBackend:
    """Backend for ``target="cuda-sm100"``."""

    target = TARGET

    def __init__(self, *, codegen_matmul: bool = True, codegen_attention: bool = True) -> None:
        # Both are always on for the operations this target covers; the flags
        # exist so callers written against the reference's options keep working.
        self.codegen_matmul = True
        self.codegen_attention = True

    def compile(self, graph: Graph, *, tune_inputs: Any = None) -> CompiledPlan:
        graph.validate()
        builder = _Builder(graph)
        for index, op in enumerate(graph.ops):
            kind = op.op
            if _lower_layout(builder, index, op):
                continue
            if kind == "embedding":
                _lower_embedding(builder, index, op)
            elif kind == "fused_elementwise":
                _lower_mask_region(builder, index, op)
            elif kind == "attention":
                _lower_attention(builder, index, op)
            elif kind in ("rope_kv_cache_append", "kv_cache_append"):
                _lower_cache_append(builder, index, op)
            elif kind == "rope":
                _lower_rope(builder, index, op)
            elif kind == "rms_norm":
                _lower_rms_norm(builder, index, op)
            elif kind in _UNPACK_BITS:
                _lower_dequantize(builder, index, op)
            elif kind in ("matmul", "addmm"):
                _lower_projection(builder, index, op)
            else:
                raise UnsupportedOperationError(
                    f"operation {kind} has no cuda-sm100 kernel",
                    hint="this target covers the static-cache decoder path; there is no "
                    "interpreter to fall back to",
                )
        native = sum(1 for s in builder.selections if s.implementation == CUDA_KERNEL)
        logger.info(
            "cuda-sm100: %d operations, %d kernels, %d views, %d copies",
            len(graph.ops), native,
            sum(1 for s in builder.selections if s.implementation == VIEW),
            sum(1 for s in builder.selections if s.implementation == COPY),
        )
        device = f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cuda:0"
        return CompiledPlan(
            graph=graph,
            kernels=tuple(builder.kernels),
            selections=tuple(builder.selections),
            _callables=builder.callables,
            storage_plan=plan_storage(graph),
            device=device,
            step_program=build_step_program(graph),
        )
