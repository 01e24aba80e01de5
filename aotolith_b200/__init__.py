"""aotolith_b200: the ``cuda-sm100`` compile target for the Aotolith static-KV-cache decoder path.

The compile pipeline (FX capture -> typed IR -> rewrite passes -> kernel
selection) is Python; every operation of a compiled plan runs a hand-written
sm_100a kernel through the C ABI in ``include/aoto_sm100.h``. The public names
are the reference compiler's: ``compile_module`` / ``compile_callable`` /
``compile_graph``, ``plan.selections``, ``compile_qwen2_static_cache`` /
``compile_llama_static_cache`` / ``*_bucketed`` and ``greedy_generate``.
"""

from ._version import __version__
from .artifact import ABI_VERSION, FORMAT_VERSION, load_compiled_module, read_artifact_manifest, save_compiled
from .backends import TARGETS, Backend, CudaBackend
from .compiler import (
    CompilationResult,
    CompiledModulePlan,
    backend_for,
    compile_callable,
    compile_graph,
    compile_module,
)
from .errors import *  # noqa: F401,F403
from .ir import DType, Graph, Operation, TensorType, Value
from .models import (
    compile_llama_bucketed,
    compile_llama_static_cache,
    compile_qwen2_bucketed,
    compile_qwen2_static_cache,
)
from .selection import KernelBenchmark, KernelSelection
from .tensor_parallel import StreamedTensorParallelDecoder, TensorParallelDecoder

__all__ = [
    "TensorParallelDecoder", "StreamedTensorParallelDecoder", "ABI_VERSION", "FORMAT_VERSION", "load_compiled_module", "read_artifact_manifest", "save_compiled",
    "TARGETS", "Backend", "CudaBackend", "CompilationResult", "CompiledModulePlan", "DType",
    "Graph", "KernelBenchmark", "KernelSelection", "Operation", "TensorType", "Value",
    "backend_for", "compile_callable", "compile_graph", "compile_llama_bucketed",
    "compile_llama_static_cache", "compile_module", "compile_qwen2_bucketed",
    "compile_qwen2_static_cache", "__version__",
]
