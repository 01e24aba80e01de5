"""The compile driver: capture -> rewrite -> backend -> executable plan.

Public surface and argument meaning follow ``src/aotolith/compiler.py`` of the
reference: ``compile_graph`` / ``compile_callable`` return a
``CompilationResult``; ``compile_module`` returns a ``CompiledModulePlan`` whose
graph inputs are the positional inputs, then promoted tensor keywords, then the
module state in ``named_parameters(remove_duplicate=False)`` +
``named_buffers(remove_duplicate=False)`` order, then one ``<constant N>`` entry
per tensor the trace captured (``compiler.py:458-533``). State is moved to the
device once, and tensors that alias share one device tensor (``:762-791``).
"""

from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from dataclasses import dataclass
from os import PathLike
from pathlib import Path
from typing import Any

import torch

from .backends import APPLE_TARGET, CUDA_TARGET, REFERENCE_TARGET, TARGETS, Backend, CudaBackend
from .capture import capture_fx
from .errors import CompilationError, PlanInputError, PlatformError
from .ir import Graph
from .passes import rewrite
from .runtime.plan import DEFAULT_MEMORY, CompiledPlan

DEFAULT_TARGET = CUDA_TARGET


@dataclass(frozen=True, slots=True)
class CompilationResult:
    plan: CompiledPlan
    input_graph: Graph
    lowered_graph: Graph
    codegen_matmul: bool = False
    codegen_attention: bool = False
    autotune: bool = False
    autotune_warmup: int = 2
    autotune_iterations: int = 7
    target: str = DEFAULT_TARGET

    def prepare(self, memory: str = DEFAULT_MEMORY) -> Any:
        return self.plan.prepare(memory)

    def save(self, path: str | PathLike[str]) -> Path:
        from .artifact import save_compiled

        return save_compiled(self, path)


@dataclass(frozen=True, slots=True)
class CompiledModulePlan:
    """An executable plan with the module's parameters and buffers bound as state."""

    compilation: CompilationResult
    input_count: int
    state_names: tuple[str, ...]
    _state_values: tuple[torch.Tensor, ...]
    tensor_kwarg_names: tuple[str, ...] = ()
    tensor_kwarg_templates: tuple[Any, ...] = ()

    @property
    def plan(self) -> CompiledPlan:
        return self.compilation.plan

    @property
    def target(self) -> str:
        return self.compilation.target

    @property
    def input_graph(self) -> Graph:
        return self.compilation.input_graph

    @property
    def lowered_graph(self) -> Graph:
        return self.compilation.lowered_graph

    def prepare(self, memory: str = DEFAULT_MEMORY) -> Any:
        return self.plan.prepare(memory)

    def save(self, path: str | PathLike[str]) -> Path:
        from .artifact import save_compiled

        return save_compiled(self, path)

    def __call__(self, *inputs: Any, verify_index_bounds: bool = True,
                 memory: str = DEFAULT_MEMORY, **tensor_kwargs: Any):
        if len(inputs) != self.input_count:
            raise PlanInputError(
                f"expected {self.input_count} inputs, received {len(inputs)}",
                hint="positional inputs come first, then promoted tensor keywords, then the state",
            )
        missing = [name for name in self.tensor_kwarg_names if name not in tensor_kwargs]
        if missing:
            raise PlanInputError("missing tensor keyword inputs: " + ", ".join(missing))
        unexpected = sorted(set(tensor_kwargs) - set(self.tensor_kwarg_names))
        if unexpected:
            raise PlanInputError(
                "unexpected keyword inputs: " + ", ".join(unexpected),
                hint="only tensor-valued keywords are promoted to graph inputs",
            )
        return self.plan(
            *inputs,
            *(tensor_kwargs[name] for name in self.tensor_kwarg_names),
            *self._state_values,
            verify_index_bounds=verify_index_bounds,
            memory=memory,
        )


def backend_for(
    target: str,
    *,
    codegen_matmul: bool = False,
    codegen_attention: bool = False,
    autotune: bool = False,
    autotune_warmup: int = 2,
    autotune_iterations: int = 7,
) -> Backend:
    """The backend a target name selects.

    ``cuda-sm100`` always generates (selects) kernels for the operations it
    covers, so ``codegen_matmul`` / ``codegen_attention`` are accepted and mean
    nothing more; its kernels have one variant per shape class chosen by rule,
    so ``autotune`` is refused rather than silently ignored. The two Apple
    targets cannot be built on this platform.
    """

    if target == CUDA_TARGET:
        if autotune:
            raise CompilationError(
                f"target {target!r} selects kernel variants by shape rule and has nothing to autotune",
                hint="drop autotune=True",
            )
        return CudaBackend(codegen_matmul=codegen_matmul, codegen_attention=codegen_attention)
    if target in (APPLE_TARGET, REFERENCE_TARGET):
        raise PlatformError(
            f"target {target!r} needs Apple silicon with MLX, which this installation does not have",
            hint=f"compile with target={CUDA_TARGET!r} on an NVIDIA B200",
        )
    raise CompilationError(
        f"unsupported target: {target}",
        hint="supported targets are: " + ", ".join(TARGETS),
    )


def compile_graph(
    graph: Graph,
    *,
    target: str = DEFAULT_TARGET,
    codegen_matmul: bool = False,
    codegen_attention: bool = False,
    autotune: bool = False,
    autotune_warmup: int = 2,
    autotune_iterations: int = 7,
    autotune_inputs: Sequence[Any] | None = None,
) -> CompilationResult:
    backend = backend_for(
        target, codegen_matmul=codegen_matmul, codegen_attention=codegen_attention,
        autotune=autotune, autotune_warmup=autotune_warmup, autotune_iterations=autotune_iterations,
    )
    # Packed projections absorb their norm regardless; dense single-row ones would need a dense
    # GEMV with a norm prologue, which this target does not have.
    lowered = rewrite(graph, native_matmul=False)
    plan = backend.compile(lowered, tune_inputs=autotune_inputs)
    return CompilationResult(
        plan=plan, input_graph=graph, lowered_graph=lowered,
        codegen_matmul=codegen_matmul, codegen_attention=codegen_attention, autotune=autotune,
        autotune_warmup=autotune_warmup, autotune_iterations=autotune_iterations, target=target,
    )


def _stand_in(tensor: torch.Tensor) -> torch.Tensor:
    """A CPU tensor of the same shape/dtype for shape-only tracing (no data is read)."""

    if tensor.device.type == "cpu":
        return tensor
    return torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu")


def compile_callable(
    fn: Callable[..., Any],
    example_inputs: Sequence[Any],
    *,
    target: str = DEFAULT_TARGET,
    codegen_matmul: bool = False,
    codegen_attention: bool = False,
    autotune: bool = False,
    autotune_warmup: int = 2,
    autotune_iterations: int = 7,
) -> CompilationResult:
    examples = tuple(_stand_in(t) if isinstance(t, torch.Tensor) else t for t in example_inputs)
    return compile_graph(
        capture_fx(fn, examples), target=target, codegen_matmul=codegen_matmul,
        codegen_attention=codegen_attention, autotune=autotune,
        autotune_warmup=autotune_warmup, autotune_iterations=autotune_iterations,
        autotune_inputs=example_inputs if autotune else None,
    )


def _module_state(module: torch.nn.Module) -> tuple[list[str], list[torch.Tensor]]:
    names: list[str] = []
    values: list[torch.Tensor] = []
    for name, value in module.named_parameters(remove_duplicate=False):
        names.append(name)
        values.append(value.detach())
    for name, value in module.named_buffers(remove_duplicate=False):
        names.append(name)
        values.append(value.detach())
    return names, values


def _to_device_once(values: Sequence[torch.Tensor], device: torch.device) -> tuple[torch.Tensor, ...]:
    """Move state to the device; tensors sharing storage share one device tensor."""

    moved: dict[tuple, torch.Tensor] = {}
    result = []
    for value in values:
        key = (value.data_ptr(), tuple(value.shape), tuple(value.stride()), value.dtype, str(value.device))
        if key not in moved:
            moved[key] = value.contiguous().to(device)
        result.append(moved[key])
    return tuple(result)


def _tensor_leaves(value: Any) -> list[torch.Tensor] | None:
    """Tensors of a nested tuple/list in reading order (``None`` entries dropped); None if anything else is in it."""

    found: list[torch.Tensor] = []
    for item in value:
        if item is None:
            continue
        if isinstance(item, torch.Tensor):
            found.append(item)
        elif isinstance(item, (tuple, list)):
            inner = _tensor_leaves(item)
            if inner is None:
                return None
            found.extend(inner)
        else:
            return None
    return found


def select_module_output(output: Any, output_key: str | None) -> Any:
    """What a compiled module returns for the module's raw ``output``.

    The reference's rule (``src/aotolith/compiler.py:843-889``): ``output_key`` names a mapping
    entry or an attribute; without it a tensor is itself, an object with ``.logits`` (a Hugging Face
    model output) is its logits, a mapping with one entry is that entry, and a tuple or list is
    the flat tuple of its tensor leaves.
    """

    chosen = output
    if output_key is not None:
        if isinstance(output, Mapping):
            if output_key not in output:
                raise KeyError(f"module output has no key {output_key!r}")
            chosen = output[output_key]
        elif hasattr(output, output_key):
            chosen = getattr(output, output_key)
        else:
            raise ValueError(f"module output has no attribute {output_key!r}")
    elif not isinstance(output, torch.Tensor):
        if hasattr(output, "logits"):
            chosen = output.logits
        elif isinstance(output, Mapping) and len(output) == 1:
            chosen = next(iter(output.values()))
    if isinstance(chosen, (tuple, list)):
        leaves = _tensor_leaves(chosen)
        if not leaves:
            raise ValueError("a module's sequence output must be a non-empty tuple or list whose leaves are tensors")
        return tuple(leaves)
    if not isinstance(chosen, torch.Tensor):
        raise ValueError("module output must be a tensor, a tuple/list of tensors, or expose one through output_key")
    return chosen


def compile_module(
    module: torch.nn.Module,
    example_inputs: Sequence[Any],
    *,
    example_kwargs: Mapping[str, Any] | None = None,
    output_key: str | None = None,
    target: str = DEFAULT_TARGET,
    codegen_matmul: bool = False,
    codegen_attention: bool = False,
    autotune: bool = False,
    autotune_warmup: int = 2,
    autotune_iterations: int = 7,
    device: str | torch.device | None = None,
) -> CompiledModulePlan:
    """Compile ``module.forward`` with its parameters and buffers bound as state.

    Tensor-valued ``example_kwargs`` become named graph inputs the caller passes
    per call; other keyword values are baked in at compile time.
    """

    from torch.func import functional_call

    if getattr(module, "training", False):
        raise CompilationError(
            "compile_module requires module.eval()",
            hint="the traced graph would hold dropout and other train-mode state",
        )
    backend_for(target, codegen_matmul=codegen_matmul, codegen_attention=codegen_attention,
                autotune=autotune)  # refuse a bad target before tracing
    kwargs = dict(example_kwargs or {})
    for reserved in ("verify_index_bounds", "memory"):
        if isinstance(kwargs.get(reserved), torch.Tensor):
            raise CompilationError(f"{reserved!r} is reserved by the plan call and cannot name a tensor input")
    tensor_kwarg_names = tuple(name for name, value in kwargs.items() if isinstance(value, torch.Tensor))
    static_kwargs = {name: value for name, value in kwargs.items() if name not in tensor_kwarg_names}
    state_names, state_values = _module_state(module)
    positional = tuple(example_inputs)
    n_inputs, n_kwargs = len(positional), len(tensor_kwarg_names)
    last_name: dict[tuple, str] = {}
    for name, value in zip(state_names, state_values):
        last_name[(value.data_ptr(), value.dtype, tuple(value.shape), tuple(value.stride()))] = name
    tied = {}
    for name, value in zip(state_names, state_values):
        last = last_name[(value.data_ptr(), value.dtype, tuple(value.shape), tuple(value.stride()))]
        if last != name and value.numel():
            tied[name] = last

    def traced(*flat):
        call_kwargs = dict(static_kwargs)
        call_kwargs.update(zip(tensor_kwarg_names, flat[n_inputs : n_inputs + n_kwargs]))
        state = dict(zip(state_names, flat[n_inputs + n_kwargs :]))
        # A tied tensor (an LM head that is the embedding) stays one graph input per name, as in the
        # reference's plans, and every use reads the input of the last name it is reachable by
        # (reference: src/aotolith/compiler.py:485-503, whose functional call ties them the same way).
        for name, last in tied.items():
            state[name] = state[last]
        return select_module_output(functional_call(module, state, tuple(flat[:n_inputs]), call_kwargs), output_key)

    examples = [*positional, *(kwargs[name] for name in tensor_kwarg_names), *state_values]
    examples = [_stand_in(t) if isinstance(t, torch.Tensor) else t for t in examples]
    constants: list[Any] = []
    graph = capture_fx(traced, examples, promoted_constants=constants)
    compilation = compile_graph(
        graph, target=target, codegen_matmul=codegen_matmul, codegen_attention=codegen_attention,
        autotune=autotune, autotune_warmup=autotune_warmup, autotune_iterations=autotune_iterations,
    )
    where = torch.device(device) if device is not None else torch.device(compilation.plan.device)
    all_names = tuple(state_names) + tuple(f"<constant {i}>" for i in range(len(constants)))
    all_values = list(state_values) + [c.detach() for c in constants]
    if torch.cuda.is_available():
        bound = _to_device_once(all_values, where)
    else:
        # No device to bind to (a compile-only host): keep the host tensors so the
        # plan can be inspected and saved; calling it raises DeviceError.
        bound = tuple(all_values)
    compilation.plan.device = str(where)
    compilation.plan.dynamic_inputs = n_inputs + n_kwargs
    return CompiledModulePlan(
        compilation=compilation,
        input_count=n_inputs,
        state_names=all_names,
        _state_values=bound,
        tensor_kwarg_names=tensor_kwarg_names,
        tensor_kwarg_templates=(),
    )
