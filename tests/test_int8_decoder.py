"""Decoders packed with eight bits, without a GPU.

The reference ships the eight-bit path beside the four-bit one (``quantize_bits=8``,
tests/test_quantized_qwen2.py:240-298). ``golden/lowered_graphs_int8.json`` and
``golden/adapter_eager_int8_<family>.npz`` hold what the reference's own capture, rewrite and
eager adapter modules produce for the toy decoders packed that way. Here: the graphs compiled
for the CUDA target are the same programs, the oracle run over them reproduces the reference's
logits and tokens, and every projection is bound to an eight-bit kernel.
"""

import json

import numpy as np
import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.errors import CompilationError
from oracle.interp import OracleRuntime
from tests.golden_util import GOLDEN, GROUP, NEW, PROMPT, canonical_graph, eager_fixture

TOL = 2e-2


@pytest.fixture(scope="module", params=["qwen2", "llama"])
def case(request):
    model, _ = eager_fixture(request.param)   # the same weights as the four-bit fixtures
    data = np.load(GOLDEN / f"adapter_eager_int8_{request.param}.npz")
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, quantize_bits=8, family=request.param
    )
    return request.param, runtime, data


def _close(actual, expected):
    expected = torch.from_numpy(np.asarray(expected)).float()
    scale = float(expected.abs().max())
    return float((actual.float() - expected).abs().max()) <= TOL * scale


@pytest.mark.parametrize("which", ["decode", "prefill"])
def test_lowered_graph_matches_reference(case, which):
    family, runtime, _ = case
    golden = json.loads((GOLDEN / "lowered_graphs_int8.json").read_text())[family][which]
    mine = canonical_graph(getattr(runtime, which).plan.graph)
    assert mine["inputs"] == golden["inputs"]
    assert [op["op"] for op in mine["ops"]] == [op["op"] for op in golden["ops"]]
    for index, (a, b) in enumerate(zip(mine["ops"], golden["ops"])):
        assert a == b, f"operation {index} ({a['op']}) differs from the reference's"
    assert mine["outputs"] == golden["outputs"]


def test_packed_state_is_four_codes_a_word(case):
    _, runtime, _ = case
    hidden = None
    for name, tensor in zip(runtime.decode.state_names, runtime.decode._state_values):
        if name == "final_norm":
            hidden = tensor.shape[0]
    for name, tensor in zip(runtime.decode.state_names, runtime.decode._state_values):
        if name.startswith("o_proj_") and name.endswith("_packed"):
            assert tensor.dtype == torch.int32 and tensor.shape == (hidden, hidden // 4)


def test_projections_are_bound_to_the_eight_bit_kernels(case):
    _, runtime, _ = case
    decode = [s for s in runtime.decode.plan.selections if s.op in ("matmul", "addmm")]
    assert decode and all(s.artifact_name == "aoto_sm100_qmatmul[qgemv_i8]" for s in decode)
    kernels = [k for k in runtime.decode.plan.kernels if k.kind in ("matmul", "addmm")]
    assert kernels and all(dict(k.params)["weight_bits"] == 8 for k in kernels)
    prefill = [s for s in runtime.prefill.plan.selections if s.op in ("matmul", "addmm")]
    # the LM head of the prefill graph reads one row, the layer projections the whole prompt
    assert {s.artifact_name for s in prefill} == {"aoto_sm100_qmatmul[qgemm_i8_rows]", "aoto_sm100_qmatmul[qgemv_i8]"}
    unpacks = [s for s in runtime.prefill.plan.selections if s.op == "dequantize_i8"]
    assert unpacks and all(s.artifact_name == "aoto_sm100_qmatmul[weight operand]" for s in unpacks)
    # the persistent step kernel streams four-bit blocks only: eight-bit plans run operation by operation
    assert runtime.decode.plan.step_program is None


def test_oracle_over_the_compiled_graphs_matches_the_reference_adapters(case):
    _, runtime, data = case
    tokens, trace, cache = OracleRuntime(runtime).greedy(data["prompt"], NEW)
    assert _close(trace[0], data["prefill_logits"])
    for step, logits in enumerate(trace[1:]):
        assert _close(logits, data["step_logits"][step]), f"decode step {step}"
    assert tokens == data["tokens"].tolist()
    assert _close(cache, data["final_cache"])
    short = torch.from_numpy(data["prompt"])[:, : PROMPT - 3]
    logits, _ = OracleRuntime(runtime).prefill(short)
    assert _close(logits, data["padded_prefill_logits"])


def test_bit_width_refusals():
    model, _ = eager_fixture("qwen2")
    with pytest.raises(CompilationError):
        aoto.models.compile_decoder_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP,
                                                 quantize_bits=3)
    with pytest.raises(CompilationError):
        aoto.models.compile_decoder_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=None,
                                                 quantize_bits=8)


def test_artifact_round_trip_keeps_the_bit_width(case, tmp_path):
    _, runtime, _ = case
    _, decode_path = runtime.save(tmp_path / "eight")
    loaded = aoto.load_compiled_module(decode_path)
    assert [s.artifact_name for s in loaded.plan.selections] == [s.artifact_name for s in runtime.decode.plan.selections]
    assert [(o.op, dict(o.attrs).get("weight_bits")) for o in loaded.plan.graph.ops] == \
           [(o.op, dict(o.attrs).get("weight_bits")) for o in runtime.decode.plan.graph.ops]
    for a, b in zip(loaded._state_values, runtime.decode._state_values):
        assert torch.equal(a.cpu().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
