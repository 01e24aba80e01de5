"""Storage planning: lifetimes, slot reuse, arena size.

After the reference's tests/test_planning.py: a hand-built graph with a known answer, then the
properties any plan must have, checked on the decode plan of a toy decoder - tenants of one slot
never live at the same time, every slot is aligned and holds its largest tenant, the arena
covers the last slot, and nothing is released before its last reader or released twice.
"""

import aotolith_b200 as aoto
from aotolith_b200.ir import DType, Graph, Operation, TensorType, Value
from aotolith_b200.models.synthetic import tiny_decoder
from aotolith_b200.planning import BUFFER_ALIGNMENT, plan_storage, tensor_nbytes


def test_storage_plan_tracks_lifetimes_and_reuses_a_dead_buffer():
    tensor_type = TensorType((4,), DType.F32)
    values = {name: Value(name, tensor_type) for name in ("x", "y", "z", "dead", "live", "out")}
    graph = Graph(
        ("x", "y", "z"),
        values,
        (
            Operation("add", ("x", "y"), ("dead",)),
            Operation("neg", ("x",), ("live",)),
            Operation("add", ("live", "z"), ("out",)),
        ),
        ("out",),
    )
    plan = plan_storage(graph)
    lifetime = {item.value_id: item for item in plan.lifetimes}
    assert tensor_nbytes(tensor_type) == 16
    assert (lifetime["dead"].start, lifetime["dead"].end) == (0, 1)
    assert (lifetime["live"].start, lifetime["live"].end) == (1, 3)
    assert lifetime["out"].is_output and lifetime["x"].is_input
    assert plan.peak_live_bytes >= 3 * 16
    assert "dead" in plan.release_after_op[0]
    assert "x" in plan.release_after_op[1]
    assert {"live", "z"} <= set(plan.release_after_op[2])
    (slot,) = [slot for slot in plan.slots if "dead" in slot.value_ids]
    assert slot.value_ids == ("dead", "live")          # the dead value's bytes are reused by the next intermediate
    assert plan.arena_size_bytes >= slot.size_bytes and plan.arena_size_bytes % BUFFER_ALIGNMENT == 0


def test_a_decoder_plan_has_the_properties_every_plan_must_have():
    runtime = aoto.compile_qwen2_static_cache(tiny_decoder("qwen2", seed=3), prompt_length=8, max_new_tokens=4, quantize=16)
    for compiled in (runtime.prefill, runtime.decode):
        graph, plan = compiled.plan.graph, compiled.plan.storage_plan
        lifetime = {item.value_id: item for item in plan.lifetimes}
        assert set(lifetime) == set(graph.inputs) | {out for op in graph.ops for out in op.outputs}
        # producers and readers bracket every lifetime
        for index, op in enumerate(graph.ops):
            for out in op.outputs:
                assert lifetime[out].start == index
            for value in op.inputs:
                assert lifetime[value].start < index + 1 <= lifetime[value].end
        for value in graph.outputs:
            assert lifetime[value].is_output and lifetime[value].end == len(graph.ops) + 1
        # slots: aligned, large enough, tenants disjoint in time, no value in two slots
        seen = set()
        end = 0
        for slot in plan.slots:
            assert slot.offset_bytes % BUFFER_ALIGNMENT == 0 and slot.offset_bytes >= end
            end = slot.offset_bytes + slot.size_bytes
            tenants = [lifetime[v] for v in slot.value_ids]
            assert all(t.size_bytes <= slot.size_bytes and not t.is_input and not t.is_output for t in tenants)
            for i, a in enumerate(tenants):
                for b in tenants[i + 1:]:
                    assert a.end <= b.start or b.end <= a.start, (a.value_id, b.value_id)
            assert not seen & set(slot.value_ids)
            seen |= set(slot.value_ids)
        assert plan.arena_size_bytes >= end
        intermediates = {v for v, l in lifetime.items() if not l.is_input and not l.is_output}
        assert seen == intermediates
        # releases: once, after the last reader, never an output
        released = [value for values in plan.release_after_op for value in values]
        assert len(released) == len(set(released)) and not set(released) & set(graph.outputs)
        for index, values in enumerate(plan.release_after_op):
            for value in values:
                assert lifetime[value].end == index + 1
        # reuse pays: the arena is smaller than the sum of the intermediates
        assert plan.arena_size_bytes < sum(lifetime[v].size_bytes for v in intermediates)
        assert plan.peak_live_bytes >= max(l.size_bytes for l in lifetime.values())
        assert compiled.plan.footprint.activation_bytes > 0
