"""The stage program of the persistent decode-step kernel, built on the CPU.

The lowered decode graph of a packed decoder is a chain of five stages per layer
(q/k/v, attention, o, gate/up, down) and the LM head. The builder must recognise it
for both families, fold the token gather into the first stage, route the residual
stream through stamped addends, and place every intermediate in its own region of
the arena. A graph with an operation outside that chain has no program.
"""

import ctypes

import pytest

import aotolith_b200 as aoto
from aotolith_b200 import _native as N
from aotolith_b200.ir import Graph, Operation
from aotolith_b200.models.synthetic import SyntheticDecoder
from aotolith_b200.runtime import step_program as sp


@pytest.fixture(scope="module", params=["qwen2", "llama"])
def runtime(request):
    # the smallest shape the kernel's stages take: group 64, every K a multiple of 128
    qwen = request.param == "qwen2"
    model = SyntheticDecoder(
        model_type=request.param, vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
        num_attention_heads=2, num_key_value_heads=1, head_dim=64, max_position_embeddings=64,
        rope_theta=1e6 if qwen else 5e5, attention_bias=qwen, tie_word_embeddings=qwen, seed=2,
    )
    compile_fn = aoto.compile_qwen2_static_cache if qwen else aoto.compile_llama_static_cache
    return compile_fn(model, prompt_length=8, max_new_tokens=4, quantize=64)


def test_program_is_five_stages_a_layer_and_the_head(runtime):
    program = runtime.decode.plan.step_program
    assert program is not None
    kinds = [stage.kind for stage in program.stages]
    layer = [N.STAGE_GEMV, N.STAGE_ATTENTION, N.STAGE_GEMV, N.STAGE_GEMV, N.STAGE_GEMV]
    assert kinds == layer * runtime.num_layers + [N.STAGE_GEMV]
    assert program.capacity == runtime.cache_capacity and program.vocab == 512
    # the token gather is folded into the first projection; nothing else gathers its input
    assert program.stages[0].flags & N.STAGE_FLAG_X_GATHER
    assert not any(stage.flags & N.STAGE_FLAG_X_GATHER for stage in program.stages[1:])
    # the last stage writes plain logits into the output buffer
    head = program.stages[-1]
    assert head.flags & N.STAGE_FLAG_OUT_PLAIN and head.refs["out"].space == "output" and head.refs["out"].key == 0
    # every operation of the graph belongs to exactly one stage or is a view / table gather
    covered = sorted(i for stage in program.stages for i in stage.op_indices)
    assert len(covered) == len(set(covered))
    ops = runtime.decode.plan.graph.ops
    compute = {i for i, op in enumerate(ops) if op.op in ("matmul", "addmm", "attention", "rope_kv_cache_append")}
    assert compute <= set(covered)


def test_residual_stream_and_epilogues(runtime):
    program = runtime.decode.plan.step_program
    gemv = [stage for stage in program.stages if stage.kind == N.STAGE_GEMV]
    per_layer = 4
    for index in range(runtime.num_layers):
        qkv, o, gate_up, down = gemv[index * per_layer:(index + 1) * per_layer]
        assert "norm_weight" in qkv.refs and "norm_weight" in gate_up.refs
        assert gate_up.ints["epilogue"] == N.EPILOGUE_SILU_MUL_PAIRED and "packed2" in gate_up.refs
        # o and down add the residual; it is the gathered embedding row in layer 0, a stamped
        # intermediate afterwards
        first = index == 0
        assert o.ints["addend_mode"] == (N.STAGE_ADDEND_GATHER if first else N.STAGE_ADDEND_STAMPED)
        assert down.ints["addend_mode"] == N.STAGE_ADDEND_STAMPED
        assert o.ints["N"] == down.ints["N"] == 128 and gate_up.ints["N"] == 256 and down.ints["K"] == 256
    assert "norm_weight" in gemv[-1].refs and gemv[-1].ints["N"] == 512


def test_arena_regions_do_not_overlap(runtime):
    program = runtime.decode.plan.step_program
    graph = runtime.decode.plan.graph
    regions = []
    for value_id, offset in program.arena_offsets.items():
        numel = 1
        for dim in graph.value(value_id).type.shape:
            numel *= dim
        regions.append((offset, offset + N.load().aoto_sm100_stamped_bytes(numel)))
    regions.sort()
    for (a0, a1), (b0, b1) in zip(regions, regions[1:]):
        assert a1 <= b0
    assert regions[-1][1] <= program.arena_bytes
    assert all(offset % 16 == 0 for offset, _ in regions)


def test_stage_array_binds_and_the_library_accepts_it(runtime):
    program = runtime.decode.plan.step_program

    def resolve(ref):  # distinct, aligned fake addresses: nothing is dereferenced on the host
        base = {"input": 0x10000000, "arena": 0x20000000, "output": 0x30000000}[ref.space]
        key = ref.key if isinstance(ref.key, int) else (abs(hash(ref.key)) % 4096)
        return base + key * 0x100000 + ref.offset + (program.arena_offsets.get(ref.key, 0) if ref.space == "arena" else 0)

    greedy = dict(token=0x40000000, generated=0x40001000, counters=0x40002000, generated_capacity=4)
    array = sp.stage_array(program, resolve, greedy=greedy)
    assert len(array) == len(program.stages) + 1
    assert array[len(array) - 1].kind == N.STAGE_PICK
    assert array[len(array) - 2].flags & N.STAGE_FLAG_ARGMAX
    assert all(array[i].flags & N.STAGE_FLAG_WINDOW for i in range(len(array)) if array[i].kind == N.STAGE_ATTENTION)
    assert ctypes.sizeof(array) == len(array) * N.load().aoto_sm100_decode_step_stage_size()
    assert sp.supported(array)
    assert sp.scratch_bytes(array) >= 4096


def test_a_graph_with_a_foreign_operation_has_no_program(runtime):
    graph = runtime.decode.plan.graph
    ops = list(graph.ops)
    # replace a packed projection by an operation the kernel has no stage for
    index = next(i for i, op in enumerate(ops) if op.op == "addmm" or op.op == "matmul")
    ops[index] = Operation("erf", ops[index].inputs[:1], ops[index].outputs, {})
    foreign = Graph(graph.inputs, graph.values, tuple(ops), graph.outputs)
    assert sp.build_step_program(foreign) is None
