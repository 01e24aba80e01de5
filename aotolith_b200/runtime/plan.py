"""Executable plans on CUDA tensors.

A ``CompiledPlan`` holds a lowered graph, one ``KernelSelection`` per
operation and one callable per operation (keyed by the operation's first
output id). Calling it validates the inputs, then runs the operations in graph
order on torch's current CUDA stream. The contract is the reference's
(``src/aotolith/runtime/plan.py:199-260``, ``:511-583``): inputs are never
mutated, outputs are fresh tensors, a shape mismatch raises ``PlanInputError``
and a dtype mismatch ``PlanDTypeError``, and the plan may be called from
several host threads.

Where the reference wraps the straight-line body in ``mx.compile`` under the
``"latency"`` memory policy, this runtime records it once into a CUDA graph and
replays it: the per-operation host cost (argument marshalling, launch) is paid
at capture, and a step becomes one graph launch. Inputs that change per call
are staged into graph-owned buffers; outputs are cloned out of the graph's
memory so the functional contract holds.
"""

from __future__ import annotations

import threading
from contextvars import ContextVar
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..errors import DeviceError, IndexBoundsError, PlanDTypeError, PlanInputError
from ..ir import DType, Graph
from ..planning import StoragePlan
from ..selection import KernelSelection

MEMORY_POLICIES = ("latency", "balanced", "minimal")
DEFAULT_MEMORY = "balanced"

TORCH_DTYPES = {
    DType.F16: torch.float16,
    DType.BF16: torch.bfloat16,
    DType.F32: torch.float32,
    DType.BOOL: torch.bool,
    DType.I32: torch.int32,
    DType.I64: torch.int64,
}


@dataclass(frozen=True, slots=True)
class KernelArtifact:
    """What was selected for one operation: an entry point of the kernel library and its variant.

    The reference's record carries generated Metal source
    (``src/aotolith/codegen/msl.py:648-690``); kernels here are precompiled, so
    ``source`` is empty and ``name`` is the C-ABI symbol plus variant.
    """

    name: str
    kind: str
    input_ids: tuple[str, ...]
    output_ids: tuple[str, ...]
    source: str = ""
    header: str = ""
    params: tuple[tuple[str, Any], ...] = ()


@dataclass(frozen=True, slots=True)
class PlanFootprint:
    input_bytes: int
    activation_bytes: int
    output_bytes: int
    peak_live_bytes: int
    arena_bytes: int

    def describe(self) -> str:
        return (
            f"inputs {self.input_bytes} B, activations {self.activation_bytes} B, "
            f"outputs {self.output_bytes} B, peak {self.peak_live_bytes} B"
        )


class CallContext:
    """Per-call state the operation callables may use.

    ``buffers`` lets a producer place its result inside a buffer a later
    operation returns (the per-layer cache pairs are written straight into the
    next cache, so the closing ``cat`` copies nothing); ``bad_index`` is the
    device flag gathers report an out-of-range index through.
    """

    __slots__ = ("buffers", "bad_index", "device")

    def __init__(self, device: torch.device, verify: bool, buffers: dict[str, torch.Tensor] | None = None):
        self.device = device
        self.buffers: dict[str, torch.Tensor] = dict(buffers or {})
        self.bad_index = torch.zeros(1, dtype=torch.int64, device=device) if verify else None


_CONTEXT: ContextVar[CallContext | None] = ContextVar("aotolith_b200_call_context", default=None)


def current_context() -> CallContext | None:
    return _CONTEXT.get()


@dataclass(slots=True)
class CompiledPlan:
    graph: Graph
    kernels: tuple[KernelArtifact, ...]
    selections: tuple[KernelSelection, ...]
    _callables: dict[str, Callable[..., Any]]
    storage_plan: StoragePlan
    device: Any = None
    #: leading inputs that change between calls; the rest (bound state) are used in place
    dynamic_inputs: int | None = None
    #: the graph as a stage program of the persistent decode-step kernel, when it has that form
    step_program: Any = None
    _program: list | None = field(default=None, repr=False)
    _slots: dict[str, int] | None = field(default=None, repr=False)
    _lock: threading.Lock = field(default_factory=threading.Lock, repr=False)
    _graph_state: dict | None = field(default=None, repr=False)

    # -- structure -----------------------------------------------------------
    def _build(self) -> None:
        if self._program is not None:
            return
        with self._lock:
            if self._program is not None:
                return
            slots: dict[str, int] = {}
            for value in self.graph.inputs:
                slots[value] = len(slots)
            program = []
            for op in self.graph.ops:
                fn = self._callables.get(op.outputs[0])
                if fn is None:
                    raise DeviceError(
                        f"operation {op.op} -> {op.outputs[0]} has no implementation on this target"
                    )
                for out in op.outputs:
                    slots[out] = len(slots)
                program.append((fn, tuple(slots[v] for v in op.inputs), tuple(slots[v] for v in op.outputs), op.op))
            self._slots = slots
            self._program = program

    def prepare(self, memory: str = DEFAULT_MEMORY) -> PlanFootprint:
        """Build the runner now instead of on the first call."""

        if memory not in MEMORY_POLICIES:
            raise PlanInputError(f"unknown memory policy {memory!r}; choose one of {MEMORY_POLICIES}")
        self._build()
        return self.footprint

    @property
    def footprint(self) -> PlanFootprint:
        lifetimes = self.storage_plan.lifetimes
        events: dict[int, int] = {}
        for life in lifetimes:
            if life.is_input:
                continue
            events[life.start] = events.get(life.start, 0) + life.size_bytes
            events[life.end] = events.get(life.end, 0) - life.size_bytes
        live = peak = 0
        for index in sorted(events):
            live += events[index]
            peak = max(peak, live)
        return PlanFootprint(
            input_bytes=sum(l.size_bytes for l in lifetimes if l.is_input),
            activation_bytes=peak,
            output_bytes=sum(l.size_bytes for l in lifetimes if l.is_output),
            peak_live_bytes=self.storage_plan.peak_live_bytes,
            arena_bytes=self.storage_plan.arena_size_bytes,
        )

    # -- input handling --------------------------------------------------------
    def _device(self) -> torch.device:
        if self.device is None:
            raise DeviceError("this plan is not bound to a CUDA device")
        return torch.device(self.device)

    def _coerce(self, inputs: tuple[Any, ...]) -> list[torch.Tensor]:
        graph = self.graph
        if len(inputs) != len(graph.inputs):
            raise PlanInputError(
                f"expected {len(graph.inputs)} inputs, received {len(inputs)}",
                hint="plan.graph.inputs names them in order",
            )
        device = self._device()
        ready: list[torch.Tensor] = []
        for position, (value_id, given) in enumerate(zip(graph.inputs, inputs)):
            spec = graph.value(value_id).type
            if not isinstance(given, torch.Tensor):
                try:
                    given = torch.as_tensor(given)
                except Exception as error:  # noqa: BLE001
                    raise PlanInputError(f"input {position} is not a tensor: {error}") from error
            if tuple(given.shape) != spec.shape:
                raise PlanInputError(
                    f"input {position} ({value_id}) has shape {tuple(given.shape)}, expected {spec.shape}"
                )
            if given.dtype != TORCH_DTYPES[spec.dtype]:
                raise PlanDTypeError(
                    f"input {position} ({value_id}) has dtype {given.dtype}, expected {spec.dtype.value}"
                )
            if given.device != device:
                given = given.to(device, non_blocking=True)
            ready.append(given)
        return ready

    # -- execution ---------------------------------------------------------------
    def _run(self, inputs: list[torch.Tensor], context: CallContext) -> tuple[torch.Tensor, ...]:
        self._build()
        env: list[Any] = [None] * len(self._slots)
        env[: len(inputs)] = inputs
        token = _CONTEXT.set(context)
        try:
            for fn, in_slots, out_slots, name in self._program:
                result = fn(*[env[i] for i in in_slots])
                if len(out_slots) == 1:
                    env[out_slots[0]] = result
                else:
                    if not isinstance(result, (tuple, list)) or len(result) != len(out_slots):
                        raise DeviceError(f"{name} returned {type(result).__name__}, expected {len(out_slots)} values")
                    for slot, value in zip(out_slots, result):
                        env[slot] = value
        finally:
            _CONTEXT.reset(token)
        return tuple(env[self._slots[v]] for v in self.graph.outputs)

    def run_eager(
        self,
        inputs: list[torch.Tensor],
        *,
        verify_index_bounds: bool = False,
        buffers: dict[str, torch.Tensor] | None = None,
    ) -> tuple[torch.Tensor, ...]:
        """Run already-validated device tensors; ``buffers`` pre-places named values."""

        context = CallContext(self._device(), verify_index_bounds, buffers)
        outputs = self._run(inputs, context)
        if context.bad_index is not None:
            seen = int(context.bad_index.item())  # one sync per verified call
            if seen:
                raise IndexBoundsError(
                    f"index out of range at gather position {seen - 1}",
                    hint="pass verify_index_bounds=False when the indices are known good "
                    "(an argmax result, for example)",
                )
        return outputs

    def __call__(
        self,
        *inputs: Any,
        verify_index_bounds: bool = True,
        memory: str = DEFAULT_MEMORY,
    ) -> tuple[torch.Tensor, ...]:
        if memory not in MEMORY_POLICIES:
            raise PlanInputError(f"unknown memory policy {memory!r}; choose one of {MEMORY_POLICIES}")
        # the kernels launch on the CURRENT device's stream: make the plan's device current
        with torch.cuda.device(self._device()):
            ready = self._coerce(inputs)
            if memory == "latency":
                return self._replay(ready, verify_index_bounds)
            return self.run_eager(ready, verify_index_bounds=verify_index_bounds)

    # -- CUDA-graph stepper --------------------------------------------------------
    def _replay(self, inputs: list[torch.Tensor], verify_index_bounds: bool = False) -> tuple[torch.Tensor, ...]:
        """Replay the recorded plan. The recording always carries the gathers' bounds flag (it is
        cleared at the head of the graph); it is read back - one synchronisation, as in an eager
        verified call - only when the caller asks for verification."""

        with self._lock_graph():
            state = self._graph_state
            if state is None:
                state = self._capture(inputs)
                self._graph_state = state
            dynamic = state["dynamic"]
            for position in range(len(inputs)):
                if position < dynamic:
                    state["staging"][position].copy_(inputs[position], non_blocking=True)
                elif inputs[position].data_ptr() != state["pointers"][position]:
                    # bound state was replaced: the recorded graph no longer applies
                    self._graph_state = None
                    return self._replay(inputs, verify_index_bounds)
            state["graph"].replay()
            outputs = tuple(out.clone() for out in state["outputs"])
            if verify_index_bounds:
                seen = int(state["bad_index"].item())
                if seen:
                    raise IndexBoundsError(
                        f"index out of range at gather position {seen - 1}",
                        hint="pass verify_index_bounds=False when the indices are known good "
                        "(an argmax result, for example)",
                    )
            return outputs

    def _lock_graph(self):
        return _GRAPH_LOCK

    def _capture(self, inputs: list[torch.Tensor]) -> dict:
        device = self._device()
        dynamic = len(inputs) if self.dynamic_inputs is None else self.dynamic_inputs
        staging = [torch.empty_like(t) for t in inputs[:dynamic]]
        for buffer, given in zip(staging, inputs[:dynamic]):
            buffer.copy_(given)
        static = staging + list(inputs[dynamic:])
        # warm up on a side stream (allocator, lazy module loads), then record
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            self.run_eager(static, verify_index_bounds=False)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        context = CallContext(device, True)
        with torch.cuda.graph(graph):
            context.bad_index.zero_()
            outputs = self._run(static, context)
        return {
            "graph": graph,
            "bad_index": context.bad_index,
            "staging": staging,
            "outputs": outputs,
            "dynamic": dynamic,
            "pointers": [t.data_ptr() for t in static],
            "keep": static,
        }


_GRAPH_LOCK = threading.RLock()
