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


#: implementation values that mean "a compiled kernel runs this operation" (the second is the
#: reference's own, kept so that selections read from one of its artifacts answer correctly)
NATIVE_IMPLEMENTATIONS = (CUDA_KERNEL, "metal_kernel")


@dataclass(frozen=True, slots=True)
class KernelBenchmark:
    """One timed candidate of an autotuned selection (never produced by this target, which picks
    variants by shape rule; the record exists because selections of other targets carry it)."""

    candidate: str                          # "native" / the fallback's name
    artifact_name: str | None               # kernel the candidate would run, if it has one
    warmup_iterations: int                  # untimed runs before the samples
    iterations: int                         # timed runs
    samples_seconds: tuple[float, ...]      # one entry per timed run
    median_seconds: float | None            # None when the candidate failed
    min_seconds: float | None
    error: str | None = None                # why the candidate failed, if it did


@dataclass(frozen=True, slots=True)
class KernelSelection:
    """What runs one operation of a plan, and why."""

    op_index: int                           # position of the operation in graph.ops
    op: str                                 # its name in the IR ("addmm", "attention", ...)
    output_id: str                          # first output value: the key of the plan's callable
    implementation: str                     # CUDA_KERNEL, VIEW, COPY (other targets: their own values)
    kind: str                               # kernel family; the operation name on this target
    reason: str                             # one sentence a person can read in a report
    artifact_name: str | None = None        # C-ABI entry point and variant, e.g. aoto_sm100_qmatmul[qgemv_mma]
    benchmarks: tuple[KernelBenchmark, ...] = ()
    autotuned: bool = False                 # always False here
    device_name: str | None = None          # GPU the plan was compiled on, if one was visible
    device_architecture: str | None = None  # "sm_100a"

    @property
    def is_native(self) -> bool:
        return self.implementation in NATIVE_IMPLEMENTATIONS

    def describe(self) -> str:
        """``#12 addmm -> aoto_sm100_qmatmul[qgemv_mma]: streamed packed words, ...``"""

        target = self.artifact_name or self.implementation
        return f"#{self.op_index} {self.op} -> {target}: {self.reason}"
