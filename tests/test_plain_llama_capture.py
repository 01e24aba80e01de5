"""A plain Hugging Face Llama through ``compile_module``'s front half (the reference's quick start).

The reference compiles ``LlamaForCausalLM(LlamaConfig(vocab 128, hidden 32, ...))`` as it is - no
adapter, no packing, fp32 (``README.md:67-84``). ``golden/lowered_graph_plain_llama.json`` holds
what the REFERENCE's ``capture_fx`` + ``rewrite`` make of that model (145 captured, 70 lowered
operations; written by ``golden/make_fixtures.py plain``), ``golden/plain_llama_eager.npz`` the
model's own logits. Here the same model goes through this repository's capture and rewrite: the
lowered graph must be the reference's operation for operation, and the oracle over it must give
the model's logits (the reference's own tolerance for this check, ``tests/test_reference_backend.py:326-367``).
The cuda-sm100 target has no fp32 kernels and says so.
"""

import json

import numpy as np
import pytest
import torch
from torch.func import functional_call

import aotolith_b200 as aoto
from aotolith_b200.capture import capture_fx
from aotolith_b200.compiler import select_module_output
from aotolith_b200.errors import UnsupportedDTypeError
from aotolith_b200.passes import rewrite
from oracle.interp import run_graph
from tests.golden.make_fixtures import module_state, plain_llama
from tests.golden_util import GOLDEN, canonical_graph


@pytest.fixture(scope="module")
def captured():
    model, ids = plain_llama()
    names, values = module_state(model)

    def traced(tokens, *state):
        return select_module_output(functional_call(model, dict(zip(names, state)), (tokens,), {}), None)

    constants: list = []
    graph = capture_fx(traced, [ids, *values], promoted_constants=constants)
    return model, ids, names, values, constants, graph, rewrite(graph)


def test_lowered_graph_is_the_references(captured):
    _, _, names, _, constants, _, lowered = captured
    golden = json.loads((GOLDEN / "lowered_graph_plain_llama.json").read_text())
    assert not constants and golden["constants"] == 0
    assert len(golden["graph"]["ops"]) == 68  # of the reference's 70 lowered operations, the live ones
    assert names == golden["state_names"]
    mine = canonical_graph(lowered)
    assert mine["inputs"] == golden["graph"]["inputs"]
    assert [op["op"] for op in mine["ops"]] == [op["op"] for op in golden["graph"]["ops"]]
    for index, (a, b) in enumerate(zip(mine["ops"], golden["graph"]["ops"])):
        assert a == b, f"operation {index} ({a['op']}) differs from the reference's"
    assert mine["outputs"] == golden["graph"]["outputs"]


def test_oracle_over_the_lowered_graph_gives_the_models_logits(captured):
    model, ids, _, values, constants, _, lowered = captured
    stored = np.load(GOLDEN / "plain_llama_eager.npz")
    assert np.array_equal(stored["ids"], ids.numpy())
    (logits,) = run_graph(lowered, [ids, *values, *constants])
    assert tuple(logits.shape) == (1, 4, 128)
    want = torch.from_numpy(stored["logits"])
    assert torch.allclose(logits, want, atol=2e-3, rtol=1e-3)
    with torch.no_grad():
        assert torch.allclose(model(ids).logits, want, atol=1e-6)


def test_the_cuda_target_refuses_an_fp32_graph_by_name(captured):
    model, ids, *_ = captured
    with pytest.raises(UnsupportedDTypeError, match="bfloat16"):
        aoto.compile_module(model, (ids,), codegen_matmul=True, codegen_attention=True)


def test_output_selection_follows_the_reference():
    from types import SimpleNamespace

    tensor, other = torch.zeros(2), torch.ones(3)
    assert select_module_output(tensor, None) is tensor
    assert select_module_output(SimpleNamespace(logits=tensor, past=object()), None) is tensor
    assert select_module_output({"only": tensor}, None) is tensor
    assert select_module_output({"a": tensor, "b": other}, "b") is other
    assert select_module_output(SimpleNamespace(hidden=other), "hidden") is other
    flat = select_module_output((tensor, (other, None, [tensor])), None)
    assert isinstance(flat, tuple) and [t is u for t, u in zip(flat, (tensor, other, tensor))] == [True] * 3
    with pytest.raises(KeyError):
        select_module_output({"a": tensor}, "missing")
    with pytest.raises(ValueError):
        select_module_output(SimpleNamespace(hidden=other), "missing")
    with pytest.raises(ValueError):
        select_module_output((tensor, "text"), None)
    with pytest.raises(ValueError):
        select_module_output(object(), None)
