"""Backends and the target registry.

``TARGETS`` keeps the reference's two names (``src/aotolith/backends/__init__.py:38``)
and adds ``"cuda-sm100"``. On this platform only the new target can compile:
the other two need Apple hardware / MLX and are refused with ``PlatformError``
by :func:`aotolith_b200.compiler.backend_for`.
"""

from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

from ..ir import Graph
from ..runtime.plan import CompiledPlan, KernelArtifact
from .cuda import TARGET as CUDA_TARGET
from .cuda import CudaBackend

REFERENCE_TARGET = "mlx-reference"
APPLE_TARGET = "apple-metal"

#: every target name the compiler, the CLI and the artifact loader accept
TARGETS: tuple[str, ...] = (APPLE_TARGET, REFERENCE_TARGET, CUDA_TARGET)


@runtime_checkable
class Backend(Protocol):
    """``compile(graph, *, tune_inputs=None) -> CompiledPlan`` and nothing else."""

    def compile(self, graph: Graph, *, tune_inputs: Any = None) -> CompiledPlan: ...


__all__ = [
    "APPLE_TARGET", "CUDA_TARGET", "REFERENCE_TARGET", "TARGETS",
    "Backend", "CompiledPlan", "CudaBackend", "KernelArtifact",
]
