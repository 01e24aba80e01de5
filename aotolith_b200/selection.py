"""Kernel-selection records: what runs each operation of a plan, and why.

One ``KernelSelection`` per graph operation, in order (``op_index`` is the
position). Field names follow ``src/aotolith/selection.py:18-34`` of the
reference; this target adds the implementation values

* ``"cuda_kernel"`` - a hand-written sm_100a kernel behind the C ABI
  (``artifact_name`` is the entry point and variant),
* ``"view"`` - a layout operation that moves no data,
* ``"copy"`` - a layout operation that has to materialise (``cat`` of strided
  parts), done by the tensor library's device copy,

and ``is_native`` is true for the first.
"""

from __future__ import annotations

from dataclasses import dataclass

CUDA_KERNEL = "cuda_kernel"
VIEW = "view"
COPY = "copy"


@dataclass(frozen=True, slots=True)
class KernelBenchmark:
    candidate: str
    artifact_name: str | None
    warmup_iterations: int
    iterations: int
    samples_seconds: tuple[float, ...]
    median_seconds: float | None
    min_seconds: float | None
    error: str | None = None


@dataclass(frozen=True, slots=True)
class KernelSelection:
    op_index: int
    op: str
    output_id: str
    implementation: str
    kind: str
    reason: str
    artifact_name: str | None = None
    benchmarks: tuple[KernelBenchmark, ...] = ()
    autotuned: bool = False
    device_name: str | None = None
    device_architecture: str | None = None

    @property
    def is_native(self) -> bool:
        return self.implementation in (CUDA_KERNEL, "metal_kernel")
