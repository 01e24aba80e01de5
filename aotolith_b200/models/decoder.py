"""Static KV-cache compilation and the greedy-decoding runtime for decoder families.

Mirrors the public surface of ``src/aotolith/models/decoder.py`` in the
reference: ``compile_decoder_static_cache`` / ``compile_decoder_bucketed``
build ``DecoderStaticCacheRuntime`` / ``DecoderBucketedRuntime`` objects with
``prefill_ids``, ``prefill_padded``, ``pad_cache``, ``decode_token``,
``decode_mask``, ``greedy_generate``, ``save``, ``memory_footprint`` and
``check_memory_budget``. Arrays are CUDA ``torch.Tensor``s.

Cache contract (reference ``decoder.py:565-615, 870-979``): the cache is
``[layers, 2, 1, kv_heads, capacity, head_dim]`` with ``capacity =
prompt_length + max_new_tokens``; prefill returns a compact cache of the prompt
width that the host left-pads with zeros; each decode step drops slot 0 and
appends the new pair at the last slot, so real tokens always occupy the last
``valid_length`` slots, the decode mask is ``arange(capacity) >= capacity -
valid_length`` and the rotary position of the decoded token is
``valid_length - 1``.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ..buckets import share_plan_state
from ..compiler import DEFAULT_TARGET, CompiledModulePlan, compile_module
from ..errors import (
    BucketRangeError,
    CompilationError,
    DynamicShapeError,
    IRValidationError,
    MemoryBudgetError,
    PlanInputError,
    UnsupportedModelError,
)
from ..ir import TensorType
from ..planning import tensor_nbytes
from ..runtime.plan import MEMORY_POLICIES
from .adapters import (  # noqa: F401 - re-exported
    FAMILIES,
    DecoderDecodeModule,
    DecoderRowsModule,
    DecoderFamily,
    DecoderPrefillModule,
    QuantizedDecoderDecodeModule,
    QuantizedDecoderRowsModule,
    QuantizedDecoderPrefillModule,
    family_for,
)


def prefill_mask(length: int, bucket: int) -> np.ndarray:
    """Rank-4 boolean mask ``[1,1,bucket,bucket]`` for a prompt left-padded into ``bucket``.

    ``[query, key]`` is True when the key is a real token at or before the
    query: ``(key <= query) & (key >= bucket - length)``. At ``length == bucket``
    this is the plain causal mask.
    """

    if bucket <= 0 or length <= 0:
        raise PlanInputError(f"need 0 < length <= bucket, got length={length}, bucket={bucket}")
    if length > bucket:
        raise BucketRangeError(f"a {length}-token prompt does not fit a {bucket}-token bucket")
    query = np.arange(bucket)[:, None]
    key = np.arange(bucket)[None, :]
    return ((key <= query) & (key >= bucket - length))[None, None]


def decode_rows_mask(valid_length: int, capacity: int, rows: int) -> np.ndarray:
    """Boolean ``[1,1,rows,capacity]`` mask of a step over ``rows`` new tokens.

    After the step the cache holds ``valid_length`` tokens in its last ``valid_length`` slots and
    the new tokens sit in the last ``rows`` of them: row ``j`` admits every slot that holds a token
    up to its own. With one row this is the reference's ``decode_mask``
    (``models/decoder.py:960-979``).
    """

    if rows < 1 or capacity < rows:
        raise PlanInputError(f"need 1 <= rows <= capacity, got rows={rows}, capacity={capacity}")
    if not rows <= valid_length <= capacity:
        raise PlanInputError(f"valid_length must be in [{rows}, {capacity}], got {valid_length}")
    slot = np.arange(capacity)[None, :]
    row = np.arange(rows)[:, None]
    return ((slot >= capacity - valid_length) & (slot <= capacity - rows + row))[None, None]


def _mb(value: int) -> str:
    for limit, unit in ((1 << 30, "GiB"), (1 << 20, "MiB"), (1 << 10, "KiB")):
        if value >= limit:
            return f"{value / limit:.2f} {unit}"
    return f"{value} B"


@dataclass(frozen=True, slots=True)
class DecoderMemoryFootprint:
    """Resident bytes of one bucket and what one step needs on top.

    ``step_peak_bytes`` counts a second cache: a decode step creates the cache it
    returns before the one it was given can be dropped.
    """

    weights_bytes: int
    cache_bytes: int
    scratch_bytes: int
    masks_bytes: int
    step_peak_bytes: int

    def describe(self) -> str:
        return (
            f"weights {_mb(self.weights_bytes)}, cache {_mb(self.cache_bytes)}, "
            f"masks {_mb(self.masks_bytes)}, scratch {_mb(self.scratch_bytes)}, "
            f"step peak {_mb(self.step_peak_bytes)}"
        )


def _as_input_ids(input_ids: Any, device: torch.device) -> torch.Tensor:
    if isinstance(input_ids, torch.Tensor):
        ids = input_ids.to(dtype=torch.int64)
    else:
        ids = torch.from_numpy(np.asarray(input_ids, dtype=np.int64))
    if ids.dim() == 1:
        ids = ids[None, :]
    if ids.device != device:
        if ids.device.type == "cpu" and device.type == "cuda":
            ids = ids.pin_memory()
        ids = ids.to(device, non_blocking=True)
    return ids


@dataclass(frozen=True, slots=True)
class DecoderStaticCacheRuntime:
    """Prefill and decode plans of one prompt length plus the host-side cache helpers."""

    prefill: CompiledModulePlan
    decode: CompiledModulePlan
    prompt_length: int
    max_new_tokens: int
    cache_capacity: int
    num_layers: int
    num_key_value_heads: int
    head_dim: int
    family: str
    memory: str
    _prefill_mask: torch.Tensor
    _sessions: dict
    rows: CompiledModulePlan | None = None      # the step over ``decode_rows`` tokens, when one was compiled
    decode_rows: int = 0

    @property
    def device(self) -> torch.device:
        return torch.device(self.decode.plan.device)

    # -- prefill -------------------------------------------------------------
    def prefill_ids(self, input_ids: Any) -> tuple[torch.Tensor, torch.Tensor]:
        ids = _as_input_ids(input_ids, self.device)
        if tuple(ids.shape) != (1, self.prompt_length):
            raise PlanInputError(f"expected prompt shape (1, {self.prompt_length}), got {tuple(ids.shape)}")
        positions = torch.arange(self.prompt_length, dtype=torch.int64, device=self.device)[None, :]
        logits, cache = self.prefill(ids, positions, self._prefill_mask, memory=self.memory)
        return logits, cache

    def prefill_padded(self, input_ids: Any) -> tuple[torch.Tensor, torch.Tensor]:
        """Prefill a prompt no longer than the plan, left-padding the rest.

        Pads only ever occupy cache slots the decode masks exclude, so logits and
        the real part of the compact cache match an exact-length plan.
        """

        ids = _as_input_ids(input_ids, self.device)
        if ids.shape[0] != 1:
            raise PlanInputError(f"expected batch size 1, got {ids.shape[0]}")
        length = int(ids.shape[1])
        if length < 1:
            raise PlanInputError(f"prompt length must be positive, got {length}")
        if length > self.prompt_length:
            raise BucketRangeError(
                f"a {length}-token prompt does not fit the {self.prompt_length}-token plan"
            )
        if length == self.prompt_length:
            return self.prefill_ids(ids)
        padding = self.prompt_length - length
        zeros = torch.zeros((1, padding), dtype=torch.int64, device=self.device)
        padded_ids = torch.cat((zeros, ids), dim=1)
        padded_positions = torch.cat(
            (zeros, torch.arange(length, dtype=torch.int64, device=self.device)[None, :]), dim=1
        )
        mask = torch.from_numpy(prefill_mask(length, self.prompt_length)).to(self.device)
        return self.prefill(padded_ids, padded_positions, mask, memory=self.memory)

    def pad_cache(self, compact_cache: torch.Tensor) -> torch.Tensor:
        expected = (self.num_layers, 2, 1, self.num_key_value_heads, self.prompt_length, self.head_dim)
        if tuple(compact_cache.shape) != expected:
            raise PlanInputError(
                f"expected compact cache shape {expected}, got {tuple(compact_cache.shape)}"
            )
        padding = torch.zeros(
            expected[:4] + (self.cache_capacity - self.prompt_length,) + expected[5:],
            dtype=compact_cache.dtype, device=compact_cache.device,
        )
        return torch.cat((padding, compact_cache), dim=4)

    # -- decode --------------------------------------------------------------
    def decode_mask(self, valid_length: int) -> torch.Tensor:
        """Boolean ``[1,1,1,capacity]`` mask selecting the last ``valid_length`` slots."""

        if not 1 <= valid_length <= self.cache_capacity:
            raise PlanInputError(f"valid_length must be in [1, {self.cache_capacity}], got {valid_length}")
        window = torch.arange(self.cache_capacity, device=self.device) >= self.cache_capacity - valid_length
        return window.reshape(1, 1, 1, self.cache_capacity)

    def decode_token(
        self, token: Any, cache: torch.Tensor, valid_length: int, *, verify_token: bool = True
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """One decode step: ``(logits, next_cache)``.

        ``valid_length`` counts the tokens the cache holds after this step; the
        token being embedded sits at rotary position ``valid_length - 1``.
        ``verify_token`` checks the token against the vocabulary, which costs
        one device synchronisation per step.
        """

        if valid_length < 1 or valid_length >= self.cache_capacity:
            raise PlanInputError(f"valid_length must be in [1, {self.cache_capacity}), got {valid_length}")
        token = _as_input_ids(token, self.device).reshape(1, 1)
        position = torch.full((1, 1), valid_length - 1, dtype=torch.int64, device=self.device)
        return self.decode(
            token, position, self.decode_mask(valid_length), cache,
            verify_index_bounds=verify_token, memory=self.memory,
        )

    def decode_tokens(
        self, tokens: Any, cache: torch.Tensor, valid_length: int, *, verify_tokens: bool = True
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """One step over ``decode_rows`` tokens: ``(logits [1, rows, vocab], next_cache)``.

        The plan a host that verifies proposed tokens needs (the reference's stated next step,
        ``docs/host-runtime.md:186-208``): the tokens sit at rotary positions ``valid_length - rows
        .. valid_length - 1``, row ``j`` attends to everything up to its own token, the window moves
        by ``rows`` slots and row ``j`` of the logits predicts the token after token ``j``. The
        weights are streamed once for all rows. A host that accepts fewer than ``rows`` tokens keeps
        the cache it passed in and replays the accepted ones.
        """

        if self.rows is None:
            raise PlanInputError("this runtime has no multi-row step", hint="compile with decode_rows=<m>")
        count = self.decode_rows
        if valid_length < count or valid_length > self.cache_capacity:
            raise PlanInputError(f"valid_length must be in [{count}, {self.cache_capacity}], got {valid_length}")
        ids = _as_input_ids(tokens, self.device)
        if tuple(ids.shape) != (1, count):
            raise PlanInputError(f"expected tokens of shape (1, {count}), got {tuple(ids.shape)}")
        positions = torch.arange(valid_length - count, valid_length, dtype=torch.int64, device=self.device)[None, :]
        mask = torch.from_numpy(decode_rows_mask(valid_length, self.cache_capacity, count)).to(self.device)
        return self.rows(ids, positions, mask, cache, verify_index_bounds=verify_tokens, memory=self.memory)

    def greedy_generate(
        self, input_ids: Any, *, max_new_tokens: int | None = None, sync_each_step: bool = False
    ) -> torch.Tensor:
        """Greedy tokens ``[1, steps]`` (int64, on the plan's device)."""

        steps = self.max_new_tokens if max_new_tokens is None else max_new_tokens
        if steps < 0 or steps > self.max_new_tokens:
            raise PlanInputError(f"max_new_tokens must be in [0, {self.max_new_tokens}], got {steps}")
        if steps == 0:
            return torch.zeros((1, 0), dtype=torch.int64, device=self.device)
        logits, compact = self.prefill_ids(input_ids)
        cache = self.pad_cache(compact)
        return _greedy_tokens(self, logits, cache, self.prompt_length, steps, sync_each_step)

    def save(self, prefix: str | Path) -> tuple[Path, Path]:
        path = Path(prefix)
        if self.rows is not None:
            self.rows.save(path.with_name(path.name + ".rows.aoto"))
        return (
            self.prefill.save(path.with_name(path.name + ".prefill.aoto")),
            self.decode.save(path.with_name(path.name + ".decode.aoto")),
        )

    # -- memory --------------------------------------------------------------
    def _cache_tensor_type(self) -> TensorType:
        expected = (self.num_layers, 2, 1, self.num_key_value_heads, self.cache_capacity, self.head_dim)
        graph = self.decode.plan.graph
        for value_id in graph.inputs:
            spec = graph.value(value_id).type
            if spec.shape == expected:
                return spec
        raise IRValidationError(f"the decode plan has no {expected} cache input")

    def memory_footprint(self) -> DecoderMemoryFootprint:
        cache_bytes = tensor_nbytes(self._cache_tensor_type())
        seen: dict[int, int] = {}
        for plan in (self.prefill, self.decode, self.rows):
            if plan is None:
                continue
            for tensor in plan._state_values:
                seen[id(tensor)] = tensor.numel() * tensor.element_size()
        weights = sum(seen.values())
        scratch = max(self.prefill.plan.footprint.activation_bytes, self.decode.plan.footprint.activation_bytes)
        masks = self._prefill_mask.numel() * self._prefill_mask.element_size() + self.cache_capacity
        resident = weights + cache_bytes + masks
        return DecoderMemoryFootprint(weights, cache_bytes, scratch, masks, resident + scratch)

    def check_memory_budget(self, budget_bytes: int) -> DecoderMemoryFootprint:
        footprint = self.memory_footprint()
        if footprint.step_peak_bytes > budget_bytes:
            raise MemoryBudgetError(
                f"one step needs {_mb(footprint.step_peak_bytes)} but the budget is "
                f"{_mb(budget_bytes)} ({footprint.describe()})",
                hint="shorten prompt_length + max_new_tokens or raise the budget",
            )
        return footprint


def _greedy_tokens(
    runtime: DecoderStaticCacheRuntime,
    logits: torch.Tensor,
    cache: torch.Tensor,
    valid_length: int,
    steps: int,
    sync_each_step: bool,
) -> torch.Tensor:
    """The greedy loop over one bucket, starting from the prefill result.

    ``valid_length`` is the real prompt length (not the bucket width). With
    ``sync_each_step`` the loop runs one plan call per token and synchronises
    after each, as a host that inspects every token would; otherwise the whole
    remainder of the sequence is handed to the device-resident stepper
    (:mod:`aotolith_b200.models.session`) and read back once.
    """

    from .. import ops

    token = ops.argmax(logits[:, -1, :]).reshape(1, 1)
    if steps == 1:
        return token.reshape(1, 1)
    if not sync_each_step:
        from .session import decode_session

        rest = decode_session(runtime).run(token, cache, valid_length, steps - 1)
        return torch.cat((token.reshape(1, 1), rest.reshape(1, -1)), dim=1)
    torch.cuda.synchronize(runtime.device)
    generated = [token.reshape(-1)]
    for _ in range(steps - 1):
        valid_length += 1
        logits, cache = runtime.decode_token(token, cache, valid_length, verify_token=False)
        token = ops.argmax(logits[:, -1, :]).reshape(1, 1)
        torch.cuda.synchronize(runtime.device)
        generated.append(token.reshape(-1))
    return torch.stack(generated, dim=1)


def _check_quantize_bits(quantize: int | None, quantize_bits: int) -> None:
    if quantize_bits not in (4, 8):
        raise CompilationError(
            f"quantize_bits must be 4 or 8, got {quantize_bits!r}",
            hint="four bits packs eight codes a word, eight bits packs four",
        )
    if quantize is None and quantize_bits != 4:
        raise CompilationError(
            "quantize_bits is only meaningful with quantize=<group size>",
            hint="pass quantize=64 (or another group size)",
        )


def _compile_bucket(
    model: torch.nn.Module,
    *,
    prompt_length: int,
    max_new_tokens: int,
    codegen_matmul: bool = False,
    codegen_attention: bool = False,
    autotune: bool = False,
    quantize: int | None = None,
    quantize_bits: int = 4,
    family: str | None = None,
    target: str = DEFAULT_TARGET,
    memory: str = "latency",
    decode_rows: int = 0,
    _packed_from: Any = None,
) -> DecoderStaticCacheRuntime:
    if memory not in MEMORY_POLICIES:
        raise CompilationError(
            f"unknown memory policy {memory!r}", hint="choose one of: " + ", ".join(MEMORY_POLICIES)
        )
    if prompt_length <= 0 or max_new_tokens < 0:
        raise CompilationError(
            "prompt_length must be positive and max_new_tokens non-negative",
            hint="both are compile-time constants of the plan pair",
        )
    if getattr(model, "training", False):
        raise CompilationError(
            "compile_decoder_static_cache requires model.eval()",
            hint="call model.eval() first",
        )
    capacity = prompt_length + max_new_tokens
    if decode_rows < 0 or decode_rows == 1 or decode_rows > max(max_new_tokens, 0):
        raise CompilationError(
            f"decode_rows must be 0 (no multi-row step) or in [2, max_new_tokens], got {decode_rows}",
            hint="the number of tokens a step consumes is a compile-time constant of its plan",
        )
    if capacity > int(model.config.max_position_embeddings):
        raise DynamicShapeError(
            "prompt_length + max_new_tokens exceeds the model's maximum position embeddings "
            f"({model.config.max_position_embeddings})",
            hint="shorten the prompt or the generation",
        )
    _check_quantize_bits(quantize, quantize_bits)
    if quantize is None:
        # dense bf16 weights: the adapters read the model's own tensors (no packing, no shared packing)
        if next(model.parameters()).dtype != torch.bfloat16:
            raise UnsupportedModelError("the cuda-sm100 kernels compute in bfloat16", hint="convert the model with .bfloat16()")
        prefill_module = DecoderPrefillModule(model, cache_capacity=capacity, require=family).eval()
        decode_module = DecoderDecodeModule(model, cache_capacity=capacity, require=family).eval()
        rows_module = DecoderRowsModule(model, cache_capacity=capacity, require=family).eval() if decode_rows else None
    else:
        settings = dict(cache_capacity=capacity, group_size=quantize, weight_bits=quantize_bits, require=family)
        prefill_module = QuantizedDecoderPrefillModule(model, packed_from=_packed_from, **settings).eval()
        decode_module = QuantizedDecoderDecodeModule(model, packed_from=prefill_module, **settings).eval()
        rows_module = (QuantizedDecoderRowsModule(model, packed_from=prefill_module, **settings).eval()
                       if decode_rows else None)
    if isinstance(_packed_from, list):
        _packed_from.append(prefill_module)
    options = dict(codegen_matmul=codegen_matmul, codegen_attention=codegen_attention,
                   autotune=autotune, target=target)
    mask = torch.from_numpy(prefill_mask(prompt_length, prompt_length))
    prefill = compile_module(
        prefill_module,
        (
            torch.zeros((1, prompt_length), dtype=torch.int64),
            torch.arange(prompt_length, dtype=torch.int64)[None, :],
            mask,
        ),
        **options,
    )
    dtype = next(model.parameters()).dtype
    decode = compile_module(
        decode_module,
        (
            torch.zeros((1, 1), dtype=torch.int64),
            torch.zeros((1, 1), dtype=torch.int64),
            torch.ones((1, 1, 1, capacity), dtype=torch.bool),
            torch.zeros(
                (prefill_module.num_layers, 2, 1, prefill_module.num_key_value_heads, capacity,
                 prefill_module.head_dim),
                dtype=dtype,
            ),
        ),
        **options,
    )
    rows = None
    if rows_module is not None:
        rows = compile_module(
            rows_module,
            (
                torch.zeros((1, decode_rows), dtype=torch.int64),
                torch.zeros((1, decode_rows), dtype=torch.int64),
                torch.ones((1, 1, decode_rows, capacity), dtype=torch.bool),
                torch.zeros(
                    (prefill_module.num_layers, 2, 1, prefill_module.num_key_value_heads, capacity,
                     prefill_module.head_dim),
                    dtype=dtype,
                ),
            ),
            **options,
        )
        prefill, decode, rows = share_plan_state([prefill, decode, rows])
    else:
        prefill, decode = share_plan_state([prefill, decode])
    device = torch.device(decode.plan.device)
    runtime = DecoderStaticCacheRuntime(
        prefill=prefill,
        decode=decode,
        prompt_length=prompt_length,
        max_new_tokens=max_new_tokens,
        cache_capacity=capacity,
        num_layers=prefill_module.num_layers,
        num_key_value_heads=prefill_module.num_key_value_heads,
        head_dim=prefill_module.head_dim,
        family=prefill_module.family.name,
        memory=memory,
        _prefill_mask=mask.to(device) if torch.cuda.is_available() else mask,
        _sessions={},
        rows=rows,
        decode_rows=decode_rows if rows is not None else 0,
    )
    del prefill_module, decode_module, rows_module
    return runtime


def compile_decoder_static_cache(model: torch.nn.Module, *, prompt_length: int, max_new_tokens: int,
                                 **options: Any) -> DecoderStaticCacheRuntime:
    """Compile a supported causal LM for greedy single-request generation.

    Keyword options: ``codegen_matmul``, ``codegen_attention``, ``autotune``,
    ``quantize`` (group size), ``quantize_bits``, ``family``, ``target``,
    ``memory`` - the reference's (``decoder.py:1090-1145``).

    ``decode_rows=m`` (no reference counterpart: the plan shape its ``docs/host-runtime.md:186-208``
    names as the next step) adds a third plan that consumes ``m`` tokens a step and returns ``m``
    rows of logits: :meth:`DecoderStaticCacheRuntime.decode_tokens`.

    ``tensor_parallel`` (a process group, or ``True`` for the default one; no reference
    counterpart) shards the packed decoder over the group's GPUs instead and returns the
    generation calls of the runtime over the shards (``tensor_parallel.TensorParallelRuntime``).
    """

    sharded = options.pop("tensor_parallel", None)
    if sharded is not None and sharded is not False:
        from ..tensor_parallel import compile_tensor_parallel

        unknown = set(options) - {"quantize", "quantize_bits", "family", "target", "device"}
        if unknown:
            raise CompilationError(f"options {sorted(unknown)} do not apply to a tensor-parallel compilation")
        if options.get("target", DEFAULT_TARGET) != DEFAULT_TARGET:
            raise CompilationError(f"unknown target {options['target']!r}", hint=f"the target is {DEFAULT_TARGET!r}")
        return compile_tensor_parallel(
            model, prompt_length=prompt_length, max_new_tokens=max_new_tokens, quantize=options.get("quantize"),
            quantize_bits=options.get("quantize_bits", 4), family=options.get("family"),
            tensor_parallel=sharded, device=options.get("device"))
    return _compile_bucket(model, prompt_length=prompt_length, max_new_tokens=max_new_tokens, **options)


@dataclass(frozen=True, slots=True)
class DecoderBucketedRuntime:
    """One runtime per prompt-length bucket; a request runs in the smallest that fits."""

    buckets: tuple[DecoderStaticCacheRuntime, ...]
    max_new_tokens: int

    def __post_init__(self) -> None:
        if not self.buckets:
            raise CompilationError("at least one bucket is required")
        widths = [bucket.prompt_length for bucket in self.buckets]
        if widths != sorted(set(widths)):
            raise CompilationError(f"buckets must be strictly increasing, got {widths}")
        for bucket in self.buckets:
            if bucket.max_new_tokens != self.max_new_tokens:
                raise CompilationError("every bucket must share one max_new_tokens")

    @property
    def prompt_lengths(self) -> tuple[int, ...]:
        return tuple(bucket.prompt_length for bucket in self.buckets)

    @property
    def family(self) -> str:
        return self.buckets[0].family

    @property
    def max_prompt_length(self) -> int:
        return self.buckets[-1].prompt_length

    def bucket_for(self, prompt_length: int) -> DecoderStaticCacheRuntime:
        if prompt_length <= 0:
            raise PlanInputError(f"prompt length must be positive, got {prompt_length}")
        for bucket in self.buckets:
            if prompt_length <= bucket.prompt_length:
                return bucket
        raise BucketRangeError(
            f"prompt length {prompt_length} exceeds the largest bucket ({self.max_prompt_length}); "
            "compile another bucket or truncate"
        )

    def prefill_ids(self, input_ids: Any) -> tuple[torch.Tensor, torch.Tensor]:
        ids = _as_input_ids(input_ids, self.buckets[0].device)
        if ids.shape[0] != 1:
            raise PlanInputError(f"expected batch size 1, got {ids.shape[0]}")
        bucket = self.bucket_for(int(ids.shape[1]))
        logits, compact = bucket.prefill_padded(ids)
        return logits, bucket.pad_cache(compact)

    def greedy_generate(self, input_ids: Any, *, max_new_tokens: int | None = None,
                        sync_each_step: bool = False) -> torch.Tensor:
        steps = self.max_new_tokens if max_new_tokens is None else max_new_tokens
        if steps < 0 or steps > self.max_new_tokens:
            raise PlanInputError(f"max_new_tokens must be in [0, {self.max_new_tokens}], got {steps}")
        ids = _as_input_ids(input_ids, self.buckets[0].device)
        if steps == 0:
            return torch.zeros((1, 0), dtype=torch.int64, device=ids.device)
        if ids.shape[0] != 1:
            raise PlanInputError(f"expected batch size 1, got {ids.shape[0]}")
        length = int(ids.shape[1])
        bucket = self.bucket_for(length)
        logits, compact = bucket.prefill_padded(ids)
        cache = bucket.pad_cache(compact)
        return _greedy_tokens(bucket, logits, cache, length, steps, sync_each_step)

    def save(self, prefix: str | Path) -> tuple[Path, ...]:
        path = Path(prefix)
        saved: list[Path] = []
        for bucket in self.buckets:
            saved.extend(bucket.save(path.with_name(f"{path.name}.{bucket.prompt_length}")))
        return tuple(saved)


def compile_decoder_bucketed(
    model: torch.nn.Module,
    *,
    prompt_lengths: Sequence[int],
    max_new_tokens: int,
    **options: Any,
) -> DecoderBucketedRuntime:
    """One plan pair per prompt-length bucket, all sharing one copy of the weights."""

    widths = [int(width) for width in prompt_lengths]
    if not widths:
        raise CompilationError("prompt_lengths must name at least one bucket")
    if any(width <= 0 for width in widths):
        raise CompilationError(f"bucket widths must be positive, got {widths}")
    if widths != sorted(set(widths)):
        raise CompilationError(f"bucket widths must be strictly increasing, got {widths}")
    runtimes = []
    packed = None
    for width in widths:
        holder: list = []
        runtimes.append(
            _compile_bucket(
                model, prompt_length=width, max_new_tokens=max_new_tokens,
                _packed_from=packed if packed is not None else holder, **options,
            )
        )
        if packed is None:
            packed = holder[0]
    shared = share_plan_state([plan for rt in runtimes for plan in (rt.prefill, rt.decode)])
    buckets = tuple(
        replace(rt, prefill=shared[2 * i], decode=shared[2 * i + 1]) for i, rt in enumerate(runtimes)
    )
    return DecoderBucketedRuntime(buckets=buckets, max_new_tokens=max_new_tokens)
