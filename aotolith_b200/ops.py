"""Tensor-level entry to the sm_100a kernels.

Each function takes CUDA ``torch.Tensor`` operands, allocates the output with
torch (the library itself never allocates) and launches through the C ABI on
torch's current stream. There is no other implementation behind these names: a
CPU tensor, a missing library or an unsupported variant raises.

Operand orders follow the lowered IR of the reference compiler so the backend
can bind an operation's inputs positionally.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _native as N
from .errors import DeviceError, PlanInputError


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def check_operand_devices(devices, current_index: int) -> None:
    """Refuse operands that are not all on the current CUDA device.

    The kernels are launched on the current device's current stream and never
    look at which device a pointer belongs to: an operand of another GPU would be
    dereferenced on the wrong one. ``devices`` are the operands' ``torch.device``s.
    """

    seen = []
    for device in devices:
        if device.type != "cuda":
            raise DeviceError(
                f"the cuda-sm100 kernels take CUDA tensors; got a tensor on {device}",
                hint="there is no CPU path on this target; move the operands to the GPU",
            )
        index = current_index if device.index is None else device.index
        if index not in seen:
            seen.append(index)
    if len(seen) > 1:
        raise DeviceError(
            f"the operands of one kernel sit on different GPUs: cuda:{seen[0]} and cuda:{seen[1]}",
            hint="move every operand to the device the plan was compiled for",
        )
    if seen and seen[0] != current_index:
        raise DeviceError(
            f"the operands are on cuda:{seen[0]} but the current CUDA device is cuda:{current_index}",
            hint="run the call under `with torch.cuda.device(tensor.device):`",
        )


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    devices = [tensor.device for tensor in tensors if tensor is not None]
    on_gpu = bool(devices) and all(device.type == "cuda" for device in devices)
    check_operand_devices(devices, torch.cuda.current_device() if on_gpu else -1)


def _bf16(tensor: torch.Tensor | None, name: str) -> None:
    if tensor is not None and tensor.dtype != torch.bfloat16:
        raise PlanInputError(f"{name} must be bfloat16 on this target, got {tensor.dtype}")


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_RETIRED_WORKSPACES: list[torch.Tensor] = []


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A zero-initialised scratch buffer for the current stream of ``device``.

    Kernels that use it restore the parts that must start at zero (arrival
    counters), so it is cleared only when it is created or has to grow. One
    buffer per (device, stream): launches on one stream are ordered, launches
    on different streams never share scratch.

    While a CUDA graph is being recorded the key is the recording stream, so
    recorded launches get a buffer of their own: its zero fill becomes a node of
    the graph that first needed it (and runs again with every replay, which is
    harmless), and the registry keeps the buffer alive after that graph is gone,
    so later recordings on the same stream can go on using it. A buffer that has to
    grow is replaced, never freed: graphs recorded earlier still hold its address
    (sizes grow geometrically with the largest request, so what is kept stays small).
    """

    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buffer = _WORKSPACES.get(key)
    if buffer is None or buffer.numel() < nbytes:
        if buffer is not None:
            _RETIRED_WORKSPACES.append(buffer)
            nbytes = max(nbytes, 2 * buffer.numel())
        buffer = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buffer
    return buffer


def _dense(tensor: torch.Tensor | None) -> torch.Tensor | None:
    if tensor is None or tensor.is_contiguous():
        return tensor
    return tensor.contiguous()


def qmatmul(
    x: torch.Tensor,
    packed: torch.Tensor,
    scales: torch.Tensor,
    *,
    group_size: int,
    addend: torch.Tensor | None = None,
    norm_weight: torch.Tensor | None = None,
    rms_norm_eps: float = 0.0,
    packed2: torch.Tensor | None = None,
    scales2: torch.Tensor | None = None,
    gate: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 1.0,
    out: torch.Tensor | None = None,
    pdl: bool = False,
    weight_bits: int = 4,
) -> torch.Tensor:
    """``beta*addend + alpha*(x_hat @ W^T)`` with a packed 4- or 8-bit ``W`` (+ epilogue).

    ``x`` is ``[..., K]``; the result is ``[..., N]``. ``addend`` is a bias ``[N]``
    or a residual shaped like the output. ``packed2/scales2`` select the paired
    ``silu(y)*y2`` form, ``gate`` the ``y*silu(gate)`` form. ``weight_bits`` says how
    the words are packed: eight codes a word (4) or four (8).
    """

    if weight_bits not in (4, 8):
        raise PlanInputError(f"weight_bits must be 4 or 8, got {weight_bits!r}")
    per_word = 32 // weight_bits

    _need_cuda(x, packed, scales, addend, norm_weight, packed2, scales2, gate)
    _bf16(x, "x"); _bf16(scales, "scales"); _bf16(addend, "addend")
    _bf16(norm_weight, "norm_weight"); _bf16(gate, "gate")
    if packed.dtype != torch.int32 or packed.dim() != 2:
        raise PlanInputError(f"packed weight must be int32 [N, K/{per_word}], got {packed.dtype} {tuple(packed.shape)}")
    K = x.shape[-1]
    n_rows, words = packed.shape
    if words * per_word != K:
        raise PlanInputError(f"x has K={K} but the packed weight holds {words * per_word} codes per row")
    M = x.numel() // K
    x2 = _dense(x).reshape(M, K)
    packed, scales = _dense(packed), _dense(scales)
    out_shape = tuple(x.shape[:-1]) + (n_rows,)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=x.device)
    args = N.QMatmulArgs()
    args.x, args.packed, args.scales = _ptr(x2), _ptr(packed), _ptr(scales)
    args.out = _ptr(out)
    args.M, args.N, args.K, args.group_size = M, n_rows, K, group_size
    args.alpha, args.beta, args.rms_norm_eps = alpha, beta, rms_norm_eps
    args.flags = (N.FLAG_PDL if pdl else 0) | (N.FLAG_WEIGHT_BITS_8 if weight_bits == 8 else 0)
    keep = [x2, packed, scales]
    if addend is not None:
        addend = _dense(addend)
        if addend.numel() == n_rows and (M == 1 or addend.dim() == 1):
            args.addend_kind = N.ADDEND_VECTOR
        elif addend.numel() == M * n_rows:
            args.addend_kind = N.ADDEND_FULL
        else:
            raise PlanInputError(
                f"addend of shape {tuple(addend.shape)} is neither a bias [N] nor shaped like the output"
            )
        args.addend = _ptr(addend)
        keep.append(addend)
    if norm_weight is not None:
        norm_weight = _dense(norm_weight)
        args.norm_weight = _ptr(norm_weight)
        keep.append(norm_weight)
    if packed2 is not None:
        packed2, scales2 = _dense(packed2), _dense(scales2)
        args.packed2, args.scales2 = _ptr(packed2), _ptr(scales2)
        args.epilogue = N.EPILOGUE_SILU_MUL_PAIRED
        keep += [packed2, scales2]
    elif gate is not None:
        gate = _dense(gate)
        if gate.numel() != M * n_rows:
            raise PlanInputError("gate must be shaped like the output")
        args.gate = _ptr(gate)
        args.epilogue = N.EPILOGUE_SILU_MUL
        keep.append(gate)
    lib = N.load()
    need = lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(args)) if M > 1 else 0
    if need:
        scratch = workspace(x.device, need)
        args.scratch, args.scratch_bytes = _ptr(scratch), scratch.numel()
        keep.append(scratch)
    N.check(lib.aoto_sm100_qmatmul(ctypes.byref(args), _stream()), "aoto_sm100_qmatmul")
    return out


def dmatmul(
    x: torch.Tensor,
    weight: torch.Tensor,
    *,
    addend: torch.Tensor | None = None,
    weight2: torch.Tensor | None = None,
    gate: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 1.0,
    out: torch.Tensor | None = None,
    pdl: bool = False,
) -> torch.Tensor:
    """``beta*addend + alpha*(x @ W^T)`` with a dense bf16 ``W [N, K]`` (+ epilogue).

    The unquantised counterpart of :func:`qmatmul`: ``addend`` is a bias ``[N]`` or a residual
    shaped like the output, ``weight2`` selects the paired ``silu(y)*y2`` form (one row of ``x``),
    ``gate`` the ``y*silu(gate)`` form. Same entry point, ``AOTO_FLAG_WEIGHT_DENSE``.
    """

    _need_cuda(x, weight, addend, weight2, gate)
    _bf16(x, "x"); _bf16(weight, "weight"); _bf16(addend, "addend"); _bf16(weight2, "weight2"); _bf16(gate, "gate")
    K = x.shape[-1]
    if weight.dim() != 2 or weight.shape[1] != K:
        raise PlanInputError(f"x has K={K} but the weight is {tuple(weight.shape)}")
    if weight2 is not None and tuple(weight2.shape) != tuple(weight.shape):
        raise PlanInputError("the two weights of the paired form must have one shape")
    n_rows = weight.shape[0]
    M = x.numel() // K
    x2, weight = _dense(x).reshape(M, K), _dense(weight)
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (n_rows,), dtype=torch.bfloat16, device=x.device)
    args = N.QMatmulArgs()
    args.x, args.packed, args.out = _ptr(x2), _ptr(weight), _ptr(out)
    args.M, args.N, args.K, args.group_size = M, n_rows, K, K
    args.alpha, args.beta = alpha, beta
    args.flags = (N.FLAG_PDL if pdl else 0) | N.FLAG_WEIGHT_DENSE
    keep = [x2, weight]
    if addend is not None:
        addend = _dense(addend)
        if addend.numel() == n_rows and (M == 1 or addend.dim() == 1):
            args.addend_kind = N.ADDEND_VECTOR
        elif addend.numel() == M * n_rows:
            args.addend_kind = N.ADDEND_FULL
        else:
            raise PlanInputError(
                f"addend of shape {tuple(addend.shape)} is neither a bias [N] nor shaped like the output"
            )
        args.addend = _ptr(addend)
        keep.append(addend)
    if weight2 is not None:
        weight2 = _dense(weight2)
        args.packed2 = _ptr(weight2)
        args.epilogue = N.EPILOGUE_SILU_MUL_PAIRED
        keep.append(weight2)
    elif gate is not None:
        gate = _dense(gate)
        if gate.numel() != M * n_rows:
            raise PlanInputError("gate must be shaped like the output")
        args.gate = _ptr(gate)
        args.epilogue = N.EPILOGUE_SILU_MUL
        keep.append(gate)
    N.check(N.load().aoto_sm100_qmatmul(ctypes.byref(args), _stream()), "aoto_sm100_qmatmul")
    return out


def dmatmul_variant(M: int, n_rows: int, K: int, paired: bool = False) -> str:
    """Name of the kernel variant the library would launch for a dense projection of this shape."""

    args = N.QMatmulArgs()
    args.M, args.N, args.K, args.group_size = M, n_rows, K, K
    args.flags = N.FLAG_WEIGHT_DENSE
    args.epilogue = N.EPILOGUE_SILU_MUL_PAIRED if paired else N.EPILOGUE_NONE
    return N.load().aoto_sm100_qmatmul_variant(ctypes.byref(args)).decode()


def qmatmul_variant(M: int, n_rows: int, K: int, group_size: int, paired: bool = False, weight_bits: int = 4) -> str:
    """Name of the kernel variant the library would launch for this shape."""

    args = N.QMatmulArgs()
    args.M, args.N, args.K, args.group_size = M, n_rows, K, group_size
    args.flags = N.FLAG_WEIGHT_BITS_8 if weight_bits == 8 else 0
    args.epilogue = N.EPILOGUE_SILU_MUL_PAIRED if paired else N.EPILOGUE_NONE
    return N.load().aoto_sm100_qmatmul_variant(ctypes.byref(args)).decode()


def dequantize_i4(packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    """``[N, K]`` bf16 weight: ``bf16(code) * scale`` rounded once."""

    _need_cuda(packed, scales)
    _bf16(scales, "scales")
    packed, scales = _dense(packed), _dense(scales)
    n_rows, words = packed.shape
    out = torch.empty((n_rows, words * 8), dtype=torch.bfloat16, device=packed.device)
    args = N.DequantizeArgs(_ptr(packed), _ptr(scales), _ptr(out), n_rows, words * 8, group_size)
    N.check(N.load().aoto_sm100_dequantize_i4(ctypes.byref(args), _stream()), "aoto_sm100_dequantize_i4")
    return out


def dequantize_i8(packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    """``[N, K]`` bf16 weight of eight-bit codes (four a word): ``bf16(code) * scale`` rounded once."""

    _need_cuda(packed, scales)
    _bf16(scales, "scales")
    packed, scales = _dense(packed), _dense(scales)
    n_rows, words = packed.shape
    out = torch.empty((n_rows, words * 4), dtype=torch.bfloat16, device=packed.device)
    args = N.DequantizeArgs(_ptr(packed), _ptr(scales), _ptr(out), n_rows, words * 4, group_size)
    N.check(N.load().aoto_sm100_dequantize_i8(ctypes.byref(args), _stream()), "aoto_sm100_dequantize_i8")
    return out


def rms_norm(
    x: torch.Tensor,
    weight: torch.Tensor | None,
    eps: float,
    residual: torch.Tensor | None = None,
    return_sum: bool = False,
):
    """RMS norm over the last axis, optionally of ``x + residual``."""

    _need_cuda(x, weight, residual)
    _bf16(x, "x"); _bf16(weight, "weight"); _bf16(residual, "residual")
    H = x.shape[-1]
    x2, residual, weight = _dense(x), _dense(residual), _dense(weight)
    out = torch.empty_like(x2)
    total = torch.empty_like(x2) if (return_sum and residual is not None) else None
    args = N.RmsNormArgs(_ptr(x2), _ptr(residual), _ptr(weight), _ptr(out), _ptr(total),
                         x2.numel() // H, H, eps)
    N.check(N.load().aoto_sm100_rms_norm(ctypes.byref(args), _stream()), "aoto_sm100_rms_norm")
    return (out, total) if return_sum else out


def rope(x: torch.Tensor, cosine: torch.Tensor, sine: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x [B,heads,T,D]`` with tables broadcastable to ``[1,1,T,D]``.

    ``x`` may be a strided view with a unit last stride (a transposed slice of a
    projection row is read in place).
    """

    _need_cuda(x, cosine, sine)
    _bf16(x, "x"); _bf16(cosine, "cos"); _bf16(sine, "sin")
    if x.dim() != 4:
        raise PlanInputError(f"rope expects a rank-4 value, got {tuple(x.shape)}")
    B, heads, T, D = x.shape
    if x.stride(3) != 1:
        x = x.contiguous()
    cos2 = _dense(cosine.expand(1, 1, T, D)).reshape(T, D)
    sin2 = _dense(sine.expand(1, 1, T, D)).reshape(T, D)
    out = torch.empty((B, heads, T, D), dtype=torch.bfloat16, device=x.device)
    args = N.RopeArgs(_ptr(x), _ptr(cos2), _ptr(sin2), _ptr(out), B, heads, T, D,
                      x.stride(0), x.stride(1), x.stride(2))
    N.check(N.load().aoto_sm100_rope(ctypes.byref(args), _stream()), "aoto_sm100_rope")
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor, bad_index: torch.Tensor | None = None) -> torch.Tensor:
    """Row gather ``table[ids]`` for int64 ids; ``bad_index`` collects a bounds violation."""

    _need_cuda(table, ids, bad_index)
    _bf16(table, "table")
    if ids.dtype != torch.int64:
        raise PlanInputError(f"embedding indices must be int64, got {ids.dtype}")
    table, ids_c = _dense(table), _dense(ids)
    rows, width = table.shape
    out = torch.empty(tuple(ids.shape) + (width,), dtype=torch.bfloat16, device=table.device)
    args = N.EmbeddingArgs(_ptr(table), _ptr(ids_c), _ptr(out), _ptr(bad_index), rows, width, ids_c.numel())
    N.check(N.load().aoto_sm100_embedding(ctypes.byref(args), _stream()), "aoto_sm100_embedding")
    return out


def mask_select(mask: torch.Tensor, on_true: float, on_false: float) -> torch.Tensor:
    """``where(mask, on_true, on_false)`` as bf16 (boolean mask -> additive mask)."""

    _need_cuda(mask)
    if mask.dtype != torch.bool:
        raise PlanInputError(f"mask must be bool, got {mask.dtype}")
    mask_c = _dense(mask)
    out = torch.empty(mask.shape, dtype=torch.bfloat16, device=mask.device)
    args = N.MaskSelectArgs(_ptr(mask_c), _ptr(out), mask_c.numel(), on_true, on_false)
    N.check(N.load().aoto_sm100_mask_select(ctypes.byref(args), _stream()), "aoto_sm100_mask_select")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the first maximum along the last axis (int64)."""

    _need_cuda(logits)
    _bf16(logits, "logits")
    logits = _dense(logits)
    width = logits.shape[-1]
    rows = logits.numel() // width
    if out is None:
        out = torch.empty(logits.shape[:-1], dtype=torch.int64, device=logits.device)
    lib = N.load()
    need = lib.aoto_sm100_argmax_scratch_bytes(rows, width)
    scratch = workspace(logits.device, need) if need else None
    args = N.ArgmaxArgs(_ptr(logits), _ptr(out), _ptr(scratch), scratch.numel() if need else 0, rows, width)
    N.check(lib.aoto_sm100_argmax(ctypes.byref(args), _stream()), "aoto_sm100_argmax")
    return out


def rope_kv_cache_append(
    cache: torch.Tensor,
    row: torch.Tensor,
    cosine: torch.Tensor,
    sine: torch.Tensor,
    *,
    layer: int,
    query_start: int,
    key_start: int,
    value_start: int,
    query_heads: int,
    new_pair: torch.Tensor | None = None,
):
    """One layer's decode-step update: ``(query, new_pair, keys, values)``.

    ``cache`` is ``[L,2,1,KVH,C,D]`` and is not modified. ``new_pair`` may be a
    preallocated ``[2,1,KVH,C,D]`` slice of the next cache.
    """

    _need_cuda(cache, row, cosine, sine)
    _bf16(cache, "cache"); _bf16(row, "row")
    cache, row = _dense(cache), _dense(row)
    L, two, batch, kvh, C, D = cache.shape
    if two != 2 or batch != 1:
        raise PlanInputError(f"cache must be [L,2,1,KVH,C,D], got {tuple(cache.shape)}")
    cos_row, sin_row = _dense(cosine).reshape(-1), _dense(sine).reshape(-1)
    if new_pair is None:
        new_pair = torch.empty((2, 1, kvh, C, D), dtype=torch.bfloat16, device=cache.device)
    query = torch.empty((1, query_heads, 1, D), dtype=torch.bfloat16, device=cache.device)
    args = N.KvAppendArgs(_ptr(cache), _ptr(row), None, _ptr(cos_row), _ptr(sin_row), _ptr(query),
                          _ptr(new_pair), layer, L, kvh, C, D, query_heads, query_start, key_start,
                          value_start, 1)
    N.check(N.load().aoto_sm100_kv_cache_append(ctypes.byref(args), _stream()), "aoto_sm100_kv_cache_append")
    return query, new_pair, new_pair[0], new_pair[1]


def kv_cache_append(
    cache: torch.Tensor,
    key: torch.Tensor,
    row: torch.Tensor,
    *,
    layer: int,
    value_start: int,
    new_pair: torch.Tensor | None = None,
):
    """The un-rotated form: ``(new_pair, keys, values)`` from an already rotated key."""

    _need_cuda(cache, key, row)
    cache, row, key = _dense(cache), _dense(row), _dense(key)
    L, _, _, kvh, C, D = cache.shape
    if new_pair is None:
        new_pair = torch.empty((2, 1, kvh, C, D), dtype=torch.bfloat16, device=cache.device)
    args = N.KvAppendArgs(_ptr(cache), _ptr(row), _ptr(key), None, None, None, _ptr(new_pair),
                          layer, L, kvh, C, D, 0, 0, 0, value_start, 0)
    N.check(N.load().aoto_sm100_kv_cache_append(ctypes.byref(args), _stream()), "aoto_sm100_kv_cache_append")
    return new_pair, new_pair[0], new_pair[1]


def attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    mask: torch.Tensor | None = None,
    *,
    scale: float | None = None,
    causal: bool = False,
    optional_workspace: bool = True,
) -> torch.Tensor:
    """GQA scaled-dot-product attention, batch 1. ``mask`` is additive bf16 ``[1,1,Lq,Lk]``.

    A split decode window needs a workspace; a long masked prefill only runs faster with one (the
    mask tiles are classified first). ``optional_workspace=False`` withholds it in the second case.
    """

    _need_cuda(query, key, value, mask)
    _bf16(query, "query"); _bf16(key, "key"); _bf16(value, "value"); _bf16(mask, "mask")
    if query.dim() != 4 or query.shape[0] != 1:
        raise PlanInputError(f"attention expects [1,heads,L,D] operands, got {tuple(query.shape)}")
    query, key, value, mask = _dense(query), _dense(key), _dense(value), _dense(mask)
    _, qh, lq, D = query.shape
    _, kvh, lk, _ = key.shape
    if mask is not None and mask.numel() != lq * lk:
        raise PlanInputError(f"mask must broadcast as [1,1,{lq},{lk}], got {tuple(mask.shape)}")
    out = torch.empty_like(query)
    args = N.AttentionArgs()
    args.q, args.k, args.v, args.mask, args.out = _ptr(query), _ptr(key), _ptr(value), _ptr(mask), _ptr(out)
    args.query_heads, args.kv_heads, args.q_len, args.kv_len, args.head_dim = qh, kvh, lq, lk, D
    args.causal = int(causal)
    args.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    lib = N.load()
    need = lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args))
    if need and (lq == 1 or optional_workspace):
        scratch = workspace(query.device, need)
        args.scratch, args.scratch_bytes = _ptr(scratch), scratch.numel()
    N.check(lib.aoto_sm100_attention(ctypes.byref(args), _stream()), "aoto_sm100_attention")
    return out


def step_inputs(counters: torch.Tensor, position: torch.Tensor, mask: torch.Tensor) -> None:
    """Write the coming step's rotary position and boolean window mask from the device counters."""

    _need_cuda(counters, position, mask)
    if counters.dtype != torch.int32 or position.dtype != torch.int64 or mask.dtype != torch.bool:
        raise PlanInputError("step_inputs expects int32 counters, an int64 position and a bool mask")
    args = N.StepInputsArgs(_ptr(counters), _ptr(position), _ptr(mask), mask.numel())
    N.check(N.load().aoto_sm100_step_inputs(ctypes.byref(args), _stream()), "aoto_sm100_step_inputs")


def greedy_pick(logits: torch.Tensor, token: torch.Tensor, generated: torch.Tensor, counters: torch.Tensor) -> None:
    """Greedy token of one logits row into ``token`` and ``generated[counters[1]]``; advance the counters."""

    _need_cuda(logits, token, generated, counters)
    _bf16(logits, "logits")
    if token.dtype != torch.int64 or generated.dtype != torch.int64 or counters.dtype != torch.int32:
        raise PlanInputError("greedy_pick expects int64 token/generated buffers and int32 counters")
    logits = _dense(logits)
    lib = N.load()
    need = lib.aoto_sm100_argmax_scratch_bytes(1, logits.numel())
    scratch = workspace(logits.device, need) if need else None
    args = N.GreedyPickArgs(_ptr(logits), _ptr(token), _ptr(generated), _ptr(counters),
                            _ptr(scratch), scratch.numel() if need else 0,
                            logits.numel(), generated.numel())
    N.check(lib.aoto_sm100_greedy_pick(ctypes.byref(args), _stream()), "aoto_sm100_greedy_pick")
