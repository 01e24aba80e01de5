"""Pin the CPU oracle against the reference's own torch adapter modules.

``golden/adapter_eager_<family>.npz`` holds what the reference's
``QuantizedDecoderPrefillModule`` / ``QuantizedDecoderDecodeModule`` compute
eagerly (PyTorch CPU bf16) for a seeded toy decoder. The oracle interpreter, run
over the graphs compiled here, must reproduce those logits within bf16
tolerance and the same greedy tokens.

Tolerance: both sides round to bf16 after every operation but not at the same
points (the eager adapter multiplies by a materialised weight inside
``F.linear``, the interpreter follows the MLX fallback's op-by-op rounding), so
logits are compared at ``2e-2 * max|logit|``.
"""

import numpy as np
import pytest
import torch

import aotolith_b200 as aoto
from oracle.interp import OracleRuntime, run_module_plan
from aotolith_b200.models.decoder import prefill_mask
from tests.golden_util import GROUP, NEW, PROMPT, eager_fixture

TOL = 2e-2


@pytest.fixture(scope="module", params=["qwen2", "llama"])
def case(request):
    model, data = eager_fixture(request.param)
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, family=request.param
    )
    return runtime, data


def _close(actual, expected):
    expected = torch.from_numpy(np.asarray(expected)).float()
    scale = float(expected.abs().max())
    return float((actual.float() - expected).abs().max()) <= TOL * scale


def test_greedy_loop_matches_reference_adapters(case):
    runtime, data = case
    tokens, trace, cache = OracleRuntime(runtime).greedy(data["prompt"], NEW)
    assert _close(trace[0], data["prefill_logits"])
    for step, logits in enumerate(trace[1:]):
        assert _close(logits, data["step_logits"][step]), f"decode step {step}"
    assert tokens == data["tokens"].tolist()
    assert _close(cache, data["final_cache"])


def test_left_padded_prefill_matches_reference(case):
    runtime, data = case
    short = torch.from_numpy(data["prompt"])[:, : PROMPT - 3]
    logits, _ = OracleRuntime(runtime).prefill(short)
    assert _close(logits, data["padded_prefill_logits"])


def test_cache_roll_semantics(case):
    """Each step drops slot 0 and appends at the last slot; the input cache is not modified."""

    runtime, data = case
    oracle = OracleRuntime(runtime)
    _, cache = oracle.prefill(data["prompt"])
    before = cache.clone()
    token = torch.tensor([[5]])
    _, after = oracle.decode(token, cache, PROMPT + 1)
    assert torch.equal(cache, before)
    assert torch.equal(after[:, :, :, :, :-1], cache[:, :, :, :, 1:])
    _, again = oracle.decode(token, cache, PROMPT + 1)
    assert torch.equal(after, again)
    # left padding is zeros and stays outside the window the mask selects
    assert not cache[:, :, :, :, : NEW].any()


def test_position_is_valid_length_minus_one(case):
    """Feeding the step a wrong position changes the logits: the rotary index matters."""

    runtime, data = case
    oracle = OracleRuntime(runtime)
    _, cache = oracle.prefill(data["prompt"])
    capacity = runtime.cache_capacity
    mask = (torch.arange(capacity) >= capacity - (PROMPT + 1)).reshape(1, 1, 1, -1)
    token = torch.tensor([[9]])
    right, _ = run_module_plan(runtime.decode, token, torch.tensor([[PROMPT]]), mask, cache)
    wrong, _ = run_module_plan(runtime.decode, token, torch.tensor([[PROMPT - 1]]), mask, cache)
    expected, _ = oracle.decode(token, cache, PROMPT + 1)
    assert torch.equal(right, expected)
    assert not torch.equal(right, wrong)


def test_prefill_mask_tables():
    """``prefill_mask(2, 4)`` and the causal case (reference tests/test_qwen2_static_cache.py:507-520)."""

    table = prefill_mask(2, 4)[0, 0]
    assert table.tolist() == [
        [False, False, False, False],
        [False, False, False, False],
        [False, False, True, False],
        [False, False, True, True],
    ]
    assert np.array_equal(prefill_mask(5, 5)[0, 0], np.tril(np.ones((5, 5), dtype=bool)))
