"""A decode step over ``m`` tokens (``decode_rows=m``), without a GPU.

The reference names this plan shape as its next step and ships no interface for it
(``docs/host-runtime.md:186-208``: token and position inputs ``[m]`` wide, a mask of ``m`` rows, ``m``
rows of logits for a host that verifies proposed tokens), so the pin is a property the domain
offers: one step over ``m`` given tokens equals ``m`` one-token steps over the same tokens - row
``j`` of the logits is the ``j``-th step's logits and the final caches agree. The one-token step is
the one pinned to the reference's eager adapters elsewhere. Both sides are evaluated by the oracle
over the graphs compiled for the CUDA target; the eager module over the same inputs is the second
opinion.
"""

import numpy as np
import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.errors import CompilationError, PlanInputError
from aotolith_b200.models.decoder import decode_rows_mask
from oracle.interp import OracleRuntime
from tests.golden_util import GROUP, NEW, PROMPT, eager_fixture

ROWS = 3
TOL = 2e-2


def _rel(actual, expected):
    expected = expected.float()
    return float((actual.float() - expected).abs().max() / expected.abs().max().clamp_min(1e-6))


@pytest.fixture(scope="module", params=[("qwen2", GROUP, 4), ("llama", GROUP, 4), ("qwen2", GROUP, 8), ("llama", None, 4)],
                ids=["qwen2-int4", "llama-int4", "qwen2-int8", "llama-dense"])
def case(request):
    family, quantize, bits = request.param
    model, _ = eager_fixture(family)
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=quantize, quantize_bits=bits, family=family,
        decode_rows=ROWS,
    )
    return runtime


def test_mask_rows():
    # capacity 6, the cache holds 5 tokens after a step over 3: slots 1..5 are real, the new tokens sit in 3..5
    mask = decode_rows_mask(5, 6, 3)[0, 0]
    assert mask.astype(int).tolist() == [[0, 1, 1, 1, 0, 0], [0, 1, 1, 1, 1, 0], [0, 1, 1, 1, 1, 1]]
    # one row is the decode mask of the one-token step
    assert decode_rows_mask(4, 6, 1)[0, 0].astype(int).tolist() == [[0, 0, 1, 1, 1, 1]]
    # a step that fills the window from empty is the causal mask
    assert np.array_equal(decode_rows_mask(3, 3, 3)[0, 0], np.tril(np.ones((3, 3), dtype=bool)))
    with pytest.raises(PlanInputError):
        decode_rows_mask(2, 6, 3)        # fewer tokens than rows
    with pytest.raises(PlanInputError):
        decode_rows_mask(7, 6, 3)


def test_one_step_over_m_tokens_equals_m_steps(case):
    runtime = case
    oracle = OracleRuntime(runtime)
    generator = torch.Generator().manual_seed(5)
    vocab = runtime.decode.plan.graph.value(runtime.decode.plan.graph.outputs[0]).type.shape[-1]
    prompt = torch.randint(0, vocab, (1, PROMPT), generator=generator)
    _, cache = oracle.prefill(prompt)
    tokens = torch.randint(0, vocab, (1, ROWS), generator=generator)      # proposed tokens, not greedy ones
    single_logits, single_cache, valid = [], cache, PROMPT
    for j in range(ROWS):
        valid += 1
        logits, single_cache = oracle.decode(tokens[:, j : j + 1], single_cache, valid)
        single_logits.append(logits[:, -1, :])
    rows_logits, rows_cache = oracle.decode_rows(tokens, cache, PROMPT + ROWS)
    assert tuple(rows_logits.shape) == (1, ROWS, vocab)
    for j in range(ROWS):
        assert _rel(rows_logits[:, j, :], single_logits[j]) < TOL, f"row {j}"
        assert int(rows_logits[:, j, :].float().argmax()) == int(single_logits[j].float().argmax())
    assert tuple(rows_cache.shape) == tuple(single_cache.shape)
    assert _rel(rows_cache, single_cache) < TOL
    # a second step continues from the cache the first returned
    more = torch.randint(0, vocab, (1, ROWS), generator=generator)
    valid = PROMPT + ROWS
    for j in range(ROWS):
        valid += 1
        logits, single_cache = oracle.decode(more[:, j : j + 1], single_cache, valid)
    again, _ = oracle.decode_rows(more, rows_cache, PROMPT + 2 * ROWS)
    assert _rel(again[:, -1, :], logits[:, -1, :]) < TOL


def test_graph_and_kernels_of_the_step(case):
    runtime = case
    plan = runtime.rows.plan
    assert runtime.decode_rows == ROWS
    ids = plan.graph.value(plan.graph.inputs[0]).type
    assert tuple(ids.shape) == (1, ROWS)
    assert tuple(plan.graph.value(plan.graph.outputs[0]).type.shape)[:2] == (1, ROWS)
    projections = [s for s in plan.selections if s.kind in ("matmul", "addmm")]
    assert projections and all(s.is_native for s in projections)
    assert all(s.is_native for s in plan.selections if s.kind in ("attention", "rms_norm", "rope"))
    # the step shares every weight with the other two plans: nothing is packed or copied twice
    mine = {name: value for name, value in zip(runtime.rows.state_names, runtime.rows._state_values)}
    for name, value in zip(runtime.decode.state_names, runtime.decode._state_values):
        if name in mine and value.numel() and not name.endswith("_table"):
            assert mine[name] is value, name


def test_eager_module_agrees_with_the_oracle_over_the_graph():
    from aotolith_b200.models.adapters import QuantizedDecoderRowsModule
    from oracle.eager import register_cpu_dequantize

    register_cpu_dequantize()       # the eager unpack on the host is the oracle's, as for the other adapter modules
    model, _ = eager_fixture("qwen2")
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, family="qwen2", decode_rows=ROWS)
    module = QuantizedDecoderRowsModule(model, cache_capacity=PROMPT + NEW, group_size=GROUP, weight_bits=4,
                                        require="qwen2").eval()
    oracle = OracleRuntime(runtime)
    generator = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 100, (1, PROMPT), generator=generator)
    _, cache = oracle.prefill(prompt)
    tokens = torch.randint(0, 100, (1, ROWS), generator=generator)
    valid = PROMPT + ROWS
    mask = torch.from_numpy(decode_rows_mask(valid, PROMPT + NEW, ROWS))
    positions = torch.arange(valid - ROWS, valid)[None, :]
    with torch.no_grad():
        want_logits, want_cache = module(tokens, positions, mask, cache)
    got_logits, got_cache = oracle.decode_rows(tokens, cache, valid)
    assert _rel(got_logits, want_logits) < TOL
    assert _rel(got_cache, want_cache) < TOL


def test_refusals():
    model, _ = eager_fixture("qwen2")
    for rows in (1, -2, NEW + 1):
        with pytest.raises(CompilationError, match="decode_rows"):
            aoto.models.compile_decoder_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP,
                                                     decode_rows=rows)
    plain = aoto.models.compile_decoder_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP)
    assert plain.rows is None and plain.decode_rows == 0
    with pytest.raises(PlanInputError, match="multi-row"):
        plain.decode_tokens(torch.zeros((1, ROWS), dtype=torch.int64), None, PROMPT + ROWS)


def test_the_step_is_saved_and_loaded_with_the_runtime(case, tmp_path):
    runtime = case
    runtime.save(tmp_path / "decoder")
    loaded = aoto.load_compiled_module(tmp_path / "decoder.rows.aoto")
    assert [s.artifact_name for s in loaded.plan.selections] == [s.artifact_name for s in runtime.rows.plan.selections]
    assert list(loaded.state_names) == list(runtime.rows.state_names)
    assert tuple(loaded.plan.graph.value(loaded.plan.graph.inputs[0]).type.shape) == (1, ROWS)


def test_mask_rows_are_the_one_token_masks_of_the_steps_they_replace():
    """Row j admits what the j-th one-token step would: every token held so far, its own included -
    ``valid_length - rows + 1 + j`` contiguous slots that end at the row's own slot."""

    rng = np.random.default_rng(3)
    for _ in range(200):
        capacity = int(rng.integers(2, 40))
        rows = int(rng.integers(1, capacity + 1))
        valid = int(rng.integers(rows, capacity + 1))
        mask = decode_rows_mask(valid, capacity, rows)[0, 0]
        assert mask.shape == (rows, capacity)
        for j in range(rows):
            admitted = np.flatnonzero(mask[j])
            own = capacity - rows + j
            assert admitted.size == valid - rows + 1 + j
            assert admitted[-1] == own and np.array_equal(admitted, np.arange(own - admitted.size + 1, own + 1))
