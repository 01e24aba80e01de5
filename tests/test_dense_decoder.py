"""Dense (``quantize=None``) decoders, without a GPU.

The reference's dense adapters (``src/aotolith/models/decoder.py:282-520``) read the model's own
bf16 weights; only q/k/v are concatenated per layer. ``golden/lowered_graphs_dense.json`` and
``golden/adapter_eager_dense_<family>.npz`` hold what the reference's own capture, rewrite and
eager adapter modules produce for the toy decoders (``golden/make_fixtures.py dense``). Here: the
graphs compiled for the CUDA target are the same programs with the same state names, the oracle
run over them reproduces the reference's logits and tokens, every projection is bound to the dense
kernel of the library, and a decode graph without packed weights has no stage program (it runs
operation by operation).
"""

import json

import numpy as np
import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.errors import UnsupportedModelError
from oracle.interp import OracleRuntime
from tests.golden_util import GOLDEN, NEW, PROMPT, canonical_graph, eager_fixture

TOL = 2e-2


@pytest.fixture(scope="module", params=["qwen2", "llama"])
def case(request):
    model, _ = eager_fixture(request.param)   # the same weights as the four-bit fixtures
    data = np.load(GOLDEN / f"adapter_eager_dense_{request.param}.npz")
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, family=request.param
    )
    return request.param, runtime, data


def _close(actual, expected):
    expected = torch.from_numpy(np.asarray(expected)).float()
    scale = float(expected.abs().max())
    return float((actual.float() - expected).abs().max()) <= TOL * scale


@pytest.mark.parametrize("which", ["decode", "prefill"])
def test_lowered_graph_matches_reference(case, which):
    family, runtime, _ = case
    golden = json.loads((GOLDEN / "lowered_graphs_dense.json").read_text())[family]
    mine = canonical_graph(getattr(runtime, which).plan.graph)
    assert mine["inputs"] == golden[which]["inputs"]
    assert [op["op"] for op in mine["ops"]] == [op["op"] for op in golden[which]["ops"]]
    for index, (a, b) in enumerate(zip(mine["ops"], golden[which]["ops"])):
        assert a == b, f"operation {index} ({a['op']}) differs from the reference's"
    assert mine["outputs"] == golden[which]["outputs"]
    assert list(getattr(runtime, which).state_names) == golden[f"{which}_state"]


def test_every_projection_is_bound_to_the_dense_kernel(case):
    _, runtime, _ = case
    # one row: the tensor-pipe GEMV (K = 64 or 128 here); the prompt's rows: the row-staging kernel,
    # and the LM head of the prompt pass reads one row again
    for plan, variant in ((runtime.decode.plan, "dgemv_mma"), (runtime.prefill.plan, "dgemm_rows")):
        chosen = [s for s in plan.selections if s.kind in ("matmul", "addmm")]
        assert chosen and all(s.is_native and s.artifact_name in (f"aoto_sm100_qmatmul[{variant}]", "aoto_sm100_qmatmul[dgemv_mma]")
                              for s in chosen)
        assert any(s.artifact_name == f"aoto_sm100_qmatmul[{variant}]" for s in chosen)
        assert all(s.is_native for s in plan.selections if s.kind in ("attention", "rms_norm", "rope_kv_cache_append"))
    # a decode graph without packed weights is not a stage program: it runs operation by operation
    assert runtime.decode.plan.step_program is None
    # the model's projection weights are plan state as they are; nothing is packed
    names = list(runtime.decode.state_names)
    assert "model.model.layers.0.mlp.down_proj.weight" in names and not any(n.endswith("_packed") for n in names)


def test_oracle_reproduces_reference_logits_and_tokens(case):
    _, runtime, data = case
    oracle = OracleRuntime(runtime)
    prompt = torch.from_numpy(data["prompt"])
    tokens, trace, cache = oracle.greedy(prompt, NEW)
    assert tokens == data["tokens"].tolist()
    assert _close(trace[0], data["prefill_logits"])
    for step in range(NEW - 1):
        assert _close(trace[step + 1], data["step_logits"][step]), step
    assert _close(cache, data["final_cache"])


def test_left_padded_prefill_matches_reference(case):
    _, runtime, data = case
    oracle = OracleRuntime(runtime)
    short = torch.from_numpy(data["prompt"])[:, : PROMPT - 3]
    logits, _ = oracle.prefill(short)
    assert _close(logits, data["padded_prefill_logits"])


def test_a_dense_model_must_be_bfloat16():
    from aotolith_b200.models.synthetic import tiny_decoder

    with pytest.raises(UnsupportedModelError, match="bfloat16"):
        aoto.compile_llama_static_cache(tiny_decoder("llama", seed=1).float(), prompt_length=4, max_new_tokens=2)
