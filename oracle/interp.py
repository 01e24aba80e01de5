"""CPU interpreter of a lowered graph with the reference's fallback semantics.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Restates the dispatch of ``src/aotolith/runtime/mlx_ops/__init__.py::
_evaluate_mlx_op`` (``:239-620``) and the run loop of
``src/aotolith/runtime/plan.py:379-491`` for the operations the static-cache
decoder graphs contain, on PyTorch CPU tensors; arithmetic is in
``oracle/ops_ref.py``. Layout operations follow
``src/aotolith/runtime/mlx_ops/layout.py:19-142``.
"""

from __future__ import annotations

import torch

from . import ops_ref as ref

INT64_MAX = 9223372036854775807

_TORCH = {
    "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
    "bool": torch.bool, "int32": torch.int32, "int64": torch.int64,
}


def _projection(op, args):
    attrs = op.attrs
    is_addmm = op.op == "addmm"
    base = 1 if is_addmm else 0
    x = args[base]
    eps = float(attrs.get("rms_norm_eps", 0.0))
    has_norm = "rms_norm_eps" in attrs
    alpha, beta = float(attrs.get("alpha", 1.0)), float(attrs.get("beta", 1.0))
    epilogue = attrs.get("epilogue")
    if "weight_group_size" in attrs:
        group = int(attrs["weight_group_size"])
        position = base + 3
        packed2 = scales2 = gate = None
        if epilogue == "silu_mul_paired":
            packed2, scales2 = args[position], args[position + 1]
            position += 2
        elif epilogue == "silu_mul":
            gate = args[position]
            position += 1
        norm_weight = args[position] if has_norm else None
        flat = x.reshape(-1, x.shape[-1])
        addend = args[0] if is_addmm else None
        if addend is not None and addend.dim() > 1:
            addend = addend.reshape(flat.shape[0], -1)
        out = ref.packed_matmul(
            flat, args[base + 1], args[base + 2], group, addend=addend, alpha=alpha, beta=beta,
            norm_weight=norm_weight, rms_norm_eps=eps, packed2=packed2, scales2=scales2,
            gate=None if gate is None else gate.reshape(flat.shape[0], -1),
            weight_bits=int(attrs.get("weight_bits", 4)),
        )
        return out
    # dense form (the weight is a materialised tensor)
    left = x if not has_norm else ref.matmul_norm_prologue(x, args[-1], eps)
    right = args[base + 1]
    if attrs.get("transpose_a", False):
        left = left.transpose(-1, -2)
    if attrs.get("transpose_b", False):
        right = right.transpose(-1, -2)
    product = (left.float() @ right.float()).to(left.dtype)
    if epilogue == "silu_mul_paired":
        # runtime/mlx_ops/__init__.py:589-596: the gate projection first, ``product * (left @ paired /
        # (1 + exp(-product)))`` in the operands' dtype
        paired = args[base + 2]
        if attrs.get("transpose_b", False):
            paired = paired.transpose(-1, -2)
        other = (left.float() @ paired.float()).to(left.dtype)
        return product * (other / (1.0 + torch.exp(-product)))
    if is_addmm:
        product = beta * args[0] + alpha * product
    if epilogue == "silu_mul":
        gate = args[base + 2]
        product = product * (gate / (1.0 + torch.exp(-gate)))
    elif epilogue is not None:
        raise ValueError(f"unsupported matmul epilogue {epilogue!r}")
    return product


def _pointwise(op, args, out_dtype):
    kind = op.op
    if "scalar" in op.attrs and kind in ("mul", "add"):
        # one operand is a Python number (``scalar_position`` says which side)
        number = op.attrs["scalar"]
        args = [number, args[0]] if op.attrs.get("scalar_position") == "lhs" else [args[0], number]
    if kind == "scalar_tensor":
        return torch.tensor(float(op.attrs["value"]), dtype=out_dtype)
    if kind == "where":
        return torch.where(args[0], args[1], args[2])
    if kind == "mul":
        return args[0] * args[1]
    if kind == "add":
        return args[0] + float(op.attrs.get("alpha", 1.0)) * args[1] if float(op.attrs.get("alpha", 1.0)) != 1.0 else args[0] + args[1]
    if kind == "neg":
        return -args[0]
    if kind == "cos":
        return torch.cos(args[0])
    if kind == "sin":
        return torch.sin(args[0])
    if kind == "silu":
        return args[0] / (1.0 + torch.exp(-args[0]))
    if kind == "cast":
        return args[0].to(out_dtype)
    raise NotImplementedError(f"oracle has no pointwise rule for {kind}")


def _dtype_of(name: str, unrounded: bool):
    dtype = _TORCH[name]
    return torch.float64 if unrounded and dtype.is_floating_point else dtype


def evaluate(graph, op, env, unrounded: bool = False):
    args = [env[v] for v in op.inputs]
    kind = op.op
    out_type = graph.value(op.outputs[0]).type
    out_dtype = _dtype_of(out_type.dtype.value, unrounded)
    if kind == "fused_elementwise":
        local = dict(env)
        for item in op.attrs["body"]:
            item_dtype = _dtype_of(graph.value(item.outputs[0]).type.dtype.value, unrounded)
            local[item.outputs[0]] = _pointwise(item, [local[v] for v in item.inputs], item_dtype)
        return local[op.outputs[0]]
    if kind == "embedding":
        return ref.embedding(args[0], args[1])
    if kind == "arange":
        return torch.arange(op.attrs["start"], op.attrs["end"], op.attrs["step"], dtype=out_dtype)
    if kind == "reshape":
        return args[0].reshape(out_type.shape)
    if kind == "unsqueeze":
        return args[0].unsqueeze(int(op.attrs["dim"]))
    if kind == "squeeze":
        return args[0].squeeze(int(op.attrs["dim"]))
    if kind == "transpose":
        return args[0].transpose(int(op.attrs["dim0"]), int(op.attrs["dim1"]))
    if kind == "expand":
        return args[0].expand(out_type.shape)
    if kind == "slice":
        dim = int(op.attrs["dim"]) % args[0].dim()
        end = int(op.attrs["end"])
        index = [slice(None)] * args[0].dim()
        index[dim] = slice(int(op.attrs["start"]), None if end == INT64_MAX else end, int(op.attrs.get("step", 1)))
        return args[0][tuple(index)]
    if kind == "cat":
        return torch.cat(args, dim=int(op.attrs["dim"]))
    if kind == "rms_norm":
        weight = args[1] if op.attrs.get("has_weight", False) else None
        return ref.rms_norm(args[0], weight, float(op.attrs.get("eps", 1e-5))).to(out_dtype)
    if kind == "dequantize_i4":
        return ref.dequantize_i4(args[0], args[1], int(op.attrs["group_size"]))
    if kind == "dequantize_i8":
        return ref.dequantize_i8(args[0], args[1], int(op.attrs["group_size"]))
    if kind in ("matmul", "addmm"):
        return _projection(op, args).reshape(out_type.shape)
    if kind == "rope":
        return ref.rope(*args)
    if kind == "rope_kv_cache_append":
        return ref.rope_kv_cache_append(*args, **{k: int(v) for k, v in op.attrs.items()})
    if kind == "kv_cache_append":
        return ref.kv_cache_append(*args, **{k: int(v) for k, v in op.attrs.items()})
    if kind == "attention":
        mask = args[3] if len(args) == 4 else None
        return ref.attention(args[0], args[1], args[2], mask, scale=float(op.attrs["scale"]),
                             causal=bool(op.attrs.get("causal", False)))
    return _pointwise(op, args, out_dtype)


def run_graph(graph, inputs, unrounded: bool = False):
    """Execute ``graph`` on CPU tensors in operation order; returns the outputs as a tuple.

    ``unrounded`` evaluates the same operations on the same stored values (bf16 weights, scales
    and tables widened exactly) in float64 with no intermediate rounding to the graph's dtypes.
    It is not the reference's arithmetic: it is the yardstick that says how far a bf16 pipeline -
    the oracle's or the GPU's - sits from the value both approximate.
    """

    if len(inputs) != len(graph.inputs):
        raise ValueError(f"expected {len(graph.inputs)} inputs, received {len(inputs)}")
    env = {value: tensor.detach().cpu() for value, tensor in zip(graph.inputs, inputs)}
    if unrounded:
        env = {k: (t.double() if t.dtype.is_floating_point else t) for k, t in env.items()}
    for op in graph.ops:
        result = evaluate(graph, op, env, unrounded)
        if len(op.outputs) == 1:
            env[op.outputs[0]] = result
        else:
            for out, value in zip(op.outputs, result):
                env[out] = value
    return tuple(env[v] for v in graph.outputs)


def run_module_plan(module_plan, *inputs, unrounded: bool = False):
    """Run a ``CompiledModulePlan``'s lowered graph on the CPU with its bound state."""

    state = [t.detach().cpu() for t in module_plan._state_values]
    return run_graph(module_plan.plan.graph, [*(torch.as_tensor(i) for i in inputs), *state], unrounded)


class OracleRuntime:
    """The greedy loop of ``models/decoder.py:811-1087`` over the oracle interpreter."""

    def __init__(self, runtime, unrounded: bool = False) -> None:
        self.rt = runtime
        self.unrounded = unrounded

    def prefill(self, ids, length=None):
        from aotolith_b200.models.decoder import prefill_mask

        rt = self.rt
        ids = torch.as_tensor(ids, dtype=torch.int64).reshape(1, -1)
        length = ids.shape[1]
        pad = rt.prompt_length - length
        padded = torch.cat((torch.zeros((1, pad), dtype=torch.int64), ids), dim=1)
        positions = torch.cat((torch.zeros((1, pad), dtype=torch.int64), torch.arange(length)[None, :]), dim=1)
        mask = torch.from_numpy(prefill_mask(length, rt.prompt_length))
        logits, compact = run_module_plan(rt.prefill, padded, positions, mask, unrounded=self.unrounded)
        zeros = torch.zeros(compact.shape[:4] + (rt.cache_capacity - rt.prompt_length,) + compact.shape[5:], dtype=compact.dtype)
        return logits, torch.cat((zeros, compact), dim=4)

    def decode(self, token, cache, valid_length):
        rt = self.rt
        mask = (torch.arange(rt.cache_capacity) >= rt.cache_capacity - valid_length).reshape(1, 1, 1, -1)
        return run_module_plan(
            rt.decode, torch.as_tensor(token, dtype=torch.int64).reshape(1, 1),
            torch.tensor([[valid_length - 1]], dtype=torch.int64), mask, cache, unrounded=self.unrounded,
        )

    def decode_rows(self, tokens, cache, valid_length):
        """The step over ``decode_rows`` tokens: positions and mask as the runtime builds them."""

        from aotolith_b200.models.decoder import decode_rows_mask

        rt = self.rt
        rows = rt.decode_rows
        mask = torch.from_numpy(decode_rows_mask(valid_length, rt.cache_capacity, rows))
        return run_module_plan(
            rt.rows, torch.as_tensor(tokens, dtype=torch.int64).reshape(1, rows),
            torch.arange(valid_length - rows, valid_length, dtype=torch.int64)[None, :], mask, cache,
            unrounded=self.unrounded,
        )

    def greedy(self, ids, steps):
        ids = torch.as_tensor(ids, dtype=torch.int64).reshape(1, -1)
        valid = ids.shape[1]
        logits, cache = self.prefill(ids)
        trace = [logits]
        token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        tokens = [int(token)]
        for _ in range(steps - 1):
            valid += 1
            logits, cache = self.decode(token, cache, valid)
            trace.append(logits)
            token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
            tokens.append(int(token))
        return tokens, trace, cache
