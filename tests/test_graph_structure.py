"""The rewrite pipeline reproduces the reference's lowered graphs.

``golden/lowered_graphs.json`` holds what the reference's own ``capture_fx`` +
``rewrite`` produce for its quantized adapters on two toy decoders. The graphs
compiled here must be the same programs: same operations in the same order,
same operand wiring, same attributes, same shapes (value names aside, dead
operations aside).
"""

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.passes import PIPELINE
from tests.golden_util import GROUP, NEW, PROMPT, canonical_graph, eager_fixture, lowered_graphs


@pytest.fixture(scope="module", params=["qwen2", "llama"])
def compiled(request):
    model, _ = eager_fixture(request.param)
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, family=request.param
    )
    return request.param, runtime


def _strip(graph: dict) -> dict:
    # group-size attribute name of the custom operator is the same; nothing to strip today
    return graph


@pytest.mark.parametrize("which", ["decode", "prefill"])
def test_lowered_graph_matches_reference(compiled, which):
    family, runtime = compiled
    golden = lowered_graphs()[family][which]
    mine = canonical_graph(getattr(runtime, which).plan.graph)
    assert mine["inputs"] == golden["inputs"]
    assert [op["op"] for op in mine["ops"]] == [op["op"] for op in golden["ops"]]
    for index, (a, b) in enumerate(zip(mine["ops"], golden["ops"])):
        assert a == b, f"operation {index} ({a['op']}) differs from the reference's"
    assert mine["outputs"] == golden["outputs"]


def test_state_names_follow_the_reference(compiled):
    family, runtime = compiled
    golden = lowered_graphs()[family]
    assert list(runtime.decode.state_names) == golden["decode_state"]
    assert list(runtime.prefill.state_names) == golden["prefill_state"]
    # no dense projection weight survives into the plan state
    for name, tensor in zip(runtime.decode.state_names, runtime.decode._state_values):
        if name.endswith("_packed"):
            assert tensor.dtype == torch.int32
    assert not any(name.endswith("proj.weight") for name in runtime.decode.state_names)


def test_decode_structure_counts(compiled):
    _, runtime = compiled
    graph = runtime.decode.plan.graph
    layers = runtime.num_layers
    kinds = [op.op for op in graph.ops]
    assert kinds.count("rope_kv_cache_append") == layers          # one cache op per layer
    assert kinds.count("attention") == layers
    paired = [op for op in graph.ops if op.attrs.get("epilogue") == "silu_mul_paired"]
    assert len(paired) == layers
    assert all("weight_group_size" in op.attrs for op in graph.ops if op.op in ("matmul", "addmm"))
    assert "dequantize_i4" not in kinds and "rms_norm" not in kinds and "rope" not in kinds
    prefill = runtime.prefill.plan.graph
    assert not any(op.attrs.get("epilogue") == "silu_mul_paired" for op in prefill.ops)
    # the LM head of the prefill graph reads one row, so it is folded
    assert sum(1 for op in prefill.ops if "weight_group_size" in op.attrs) == 1


def test_pipeline_order():
    assert [name for name, _ in PIPELINE] == [
        "fuse_kv_cache_update", "simplify_layouts", "canonicalize_batched_matmul", "fuse_attention",
        "fold_matmul_input_layouts", "fold_quantized_weights", "fuse_norm_scale", "fuse_rope",
        "fuse_rope_into_kv_cache_update", "fuse_residual_epilogue", "fuse_pointwise",
        "fuse_gate_up_projection", "fuse_activation_epilogue", "eliminate_common_subexpressions",
        "fuse_rms_norm_epilogue", "collapse_trailing_layouts",
    ]


def test_selections_cover_every_operation(compiled):
    _, runtime = compiled
    for plan in (runtime.prefill.plan, runtime.decode.plan):
        assert len(plan.selections) == len(plan.graph.ops)
        for index, (selection, op) in enumerate(zip(plan.selections, plan.graph.ops)):
            assert selection.op_index == index and selection.op == op.op
            assert selection.output_id == op.outputs[0] and selection.reason
            assert selection.device_architecture == "sm_100a"
        compute = [s for s in plan.selections if s.kind in ("matmul", "addmm", "attention", "rope_kv_cache_append", "rms_norm", "rope", "embedding")]
        assert compute and all(s.is_native and s.implementation == "cuda_kernel" for s in compute)
