"""The backend seam: target names, the one-method protocol, selections and kernel records.

After the reference's tests/test_reference_backend.py and tests/test_selection.py. The drop-in
boundary of this target is the reference's own seam - a target name resolved to an object with
``compile(graph, *, tune_inputs=None) -> CompiledPlan`` - so the checks here are that the names
and refusals are the reference's, that every operation of a compiled plan is accounted for by a
selection, and that native selections name the C-ABI entry point they call.
"""

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.backends import APPLE_TARGET, CUDA_TARGET, REFERENCE_TARGET, TARGETS, Backend, CudaBackend
from aotolith_b200.capture import capture_fx
from aotolith_b200.compiler import DEFAULT_TARGET, backend_for
from aotolith_b200.errors import CompilationError, PlatformError, UnsupportedOperationError
from aotolith_b200.models.synthetic import tiny_decoder
from aotolith_b200.runtime.plan import CompiledPlan
from aotolith_b200 import _native as N


def test_the_target_names_are_part_of_the_public_surface():
    assert TARGETS == ("apple-metal", "mlx-reference", "cuda-sm100")
    assert (APPLE_TARGET, REFERENCE_TARGET, CUDA_TARGET) == TARGETS
    assert DEFAULT_TARGET == "cuda-sm100"


def test_an_unknown_target_lists_the_ones_that_exist():
    with pytest.raises(CompilationError) as refused:
        backend_for("vulkan")
    for name in TARGETS:
        assert name in (refused.value.hint or "") + str(refused.value)


@pytest.mark.parametrize("target", [APPLE_TARGET, REFERENCE_TARGET])
def test_the_apple_targets_are_refused_on_this_platform_by_name(target):
    with pytest.raises(PlatformError, match=target):
        backend_for(target)
    model = tiny_decoder("qwen2", seed=1)
    with pytest.raises(PlatformError):
        aoto.compile_qwen2_static_cache(model, prompt_length=8, max_new_tokens=2, quantize=16, target=target)


def test_the_backend_satisfies_the_protocol():
    backend = backend_for(CUDA_TARGET)
    assert isinstance(backend, CudaBackend) and isinstance(backend, Backend)
    assert backend.target == CUDA_TARGET
    # the reference's kernel options are accepted and change nothing: this target always selects kernels
    assert isinstance(backend_for(CUDA_TARGET, codegen_matmul=True, codegen_attention=True), CudaBackend)


def test_autotuning_is_refused_rather_than_ignored():
    with pytest.raises(CompilationError, match="autotune"):
        backend_for(CUDA_TARGET, autotune=True)


def test_compile_returns_a_plan_with_one_selection_per_operation():
    def call(value, weight):
        return torch.nn.functional.rms_norm(value, (value.shape[-1],), weight, 1e-6)

    value = torch.randn(1, 4, 64).bfloat16()
    weight = torch.randn(64).bfloat16()
    graph = aoto.passes.rewrite(capture_fx(call, (value, weight)))
    plan = backend_for(CUDA_TARGET).compile(graph)
    assert isinstance(plan, CompiledPlan)
    assert [s.op_index for s in plan.selections] == list(range(len(graph.ops)))
    assert {s.output_id for s in plan.selections} == {op.outputs[0] for op in graph.ops}
    (norm,) = [s for s in plan.selections if s.op == "rms_norm"]
    assert norm.is_native and norm.implementation == "cuda_kernel"
    assert norm.artifact_name == "aoto_sm100_rms_norm" and norm.device_architecture == "sm_100a"
    assert norm.reason
    # every native selection names an entry point the library exports
    for selection in plan.selections:
        if selection.is_native:
            assert selection.artifact_name.split("[")[0] in N.EXPORTS
    # ... and is mirrored by a kernel record with the operands it binds
    (record,) = [k for k in plan.kernels if k.name == "aoto_sm100_rms_norm"]
    assert record.kind == "rms_norm" and len(record.input_ids) == 2 and abs(dict(record.params)["eps"] - 1e-6) < 1e-9


def test_a_decoder_plan_is_entirely_native_views_or_copies():
    model = tiny_decoder("llama", seed=2)
    runtime = aoto.compile_llama_static_cache(model, prompt_length=8, max_new_tokens=3, quantize=16)
    for plan in (runtime.prefill.plan, runtime.decode.plan):
        kinds = {s.implementation for s in plan.selections}
        assert kinds <= {"cuda_kernel", "view", "copy"}, kinds        # no interpreter fallback exists on this target
        assert len(plan.selections) == len(plan.graph.ops)
        for selection in plan.selections:
            if selection.is_native:
                assert selection.artifact_name.split("[")[0] in N.EXPORTS, selection.artifact_name


def test_an_operation_without_a_kernel_is_refused_by_name():
    def call(value):
        return torch.softmax(value, dim=-1)

    with pytest.raises(UnsupportedOperationError) as refused:
        aoto.compile_callable(call, (torch.randn(2, 8).bfloat16(),))
    assert "softmax" in str(refused.value)


def test_a_model_that_is_not_bfloat16_is_refused():
    from aotolith_b200.errors import UnsupportedDTypeError

    def call(value, weight):
        return torch.nn.functional.rms_norm(value, (value.shape[-1],), weight, 1e-6)

    with pytest.raises(UnsupportedDTypeError):
        aoto.compile_callable(call, (torch.randn(1, 4, 64), torch.randn(64)))
