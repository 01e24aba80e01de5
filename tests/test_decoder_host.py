"""Host logic of the static-cache runtimes, without a GPU.

After the reference's tests/test_qwen2_static_cache.py and tests/test_llama_static_cache.py:
which checkpoints the adapters accept and refuse (and with which coded error), what the masks
select, how the bucketed runtime picks, pads and shares, and what the memory report counts. Where
numbers are compared they are the oracle's over the compiled graphs against the ``transformers``
model's own forward pass.
"""

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.errors import (
    AotolithError, BucketRangeError, CompilationError, MemoryBudgetError, PlanInputError, UnsupportedModelError,
)
from aotolith_b200.models.decoder import prefill_mask
from oracle.interp import OracleRuntime, run_module_plan

transformers = pytest.importorskip("transformers")

GROUP, NEW = 16, 4
COMMON = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-6)


def _qwen2(**overrides):
    torch.manual_seed(11)
    config = transformers.Qwen2Config(**{**COMMON, "tie_word_embeddings": True, **overrides})
    return transformers.Qwen2ForCausalLM(config).to(torch.bfloat16).eval()


def _llama(**overrides):
    torch.manual_seed(12)
    config = transformers.LlamaConfig(**{**COMMON, "tie_word_embeddings": False, **overrides})
    return transformers.LlamaForCausalLM(config).to(torch.bfloat16).eval()


def _options(**extra):
    return dict(max_new_tokens=NEW, quantize=GROUP, **extra)


# ---------------------------------------------------------------------------
# what the adapters accept and refuse
# ---------------------------------------------------------------------------

def test_entry_points_refuse_the_other_family_and_the_shared_one_takes_either():
    with pytest.raises(UnsupportedModelError, match="llama"):
        aoto.compile_llama_static_cache(_qwen2(), prompt_length=8, **_options())
    with pytest.raises(UnsupportedModelError, match="qwen2"):
        aoto.compile_qwen2_static_cache(_llama(), prompt_length=8, **_options())
    for model, family in ((_qwen2(), "qwen2"), (_llama(), "llama")):
        runtime = aoto.models.compile_decoder_static_cache(model, prompt_length=8, **_options())
        assert runtime.family == family


def test_an_uncovered_model_type_lists_the_covered_families():
    model = _llama()
    model.config.model_type = "mistral"
    with pytest.raises(UnsupportedModelError) as refused:
        aoto.models.compile_decoder_static_cache(model, prompt_length=8, **_options())
    assert "Qwen2" in str(refused.value) and "Llama" in str(refused.value)
    # a coded error a program can branch on, and an ordinary NotImplementedError for everyone else
    assert isinstance(refused.value, AotolithError) and isinstance(refused.value, NotImplementedError)
    assert refused.value.code.startswith("AOTO-")


def test_an_mlp_activation_other_than_silu_is_refused():
    with pytest.raises(UnsupportedModelError, match="SiLU gated MLP"):
        aoto.compile_llama_static_cache(_llama(hidden_act="gelu"), prompt_length=8, **_options())


def test_sliding_window_attention_is_refused():
    model = _qwen2(use_sliding_window=True, sliding_window=4, max_window_layers=0)
    if not (getattr(model.model, "has_sliding_layers", False)
            or "sliding_attention" in (getattr(model.config, "layer_types", None) or [])):
        pytest.skip("this transformers version does not build sliding layers from these settings")
    with pytest.raises(UnsupportedModelError, match="sliding-window"):
        aoto.compile_qwen2_static_cache(model, prompt_length=8, **_options())


def test_scaled_rope_is_refused_with_the_family_named():
    model = _llama()
    scaled = {"rope_type": "linear", "factor": 2.0, "rope_theta": 10000.0}
    if isinstance(getattr(model.config, "rope_parameters", None), dict):
        model.config.rope_parameters = scaled
    else:
        model.config.rope_scaling = scaled
    with pytest.raises(UnsupportedModelError, match="Llama"):
        aoto.compile_llama_static_cache(model, prompt_length=8, **_options())


def test_bias_free_attention_is_not_given_a_zero_bias_and_qwen2_keeps_its_own():
    llama = aoto.compile_llama_static_cache(_llama(), prompt_length=8, **_options())
    assert not any(name.startswith("qkv_bias") for name in llama.decode.state_names)
    assert not any(op.op == "addmm" and "rms_norm_eps" in op.attrs and len(op.inputs) == 5
                   for op in llama.decode.plan.graph.ops)
    qwen = aoto.compile_qwen2_static_cache(_qwen2(), prompt_length=8, **_options())
    biases = [name for name in qwen.decode.state_names if name.startswith("qkv_bias")]
    assert len(biases) == 2
    index = list(qwen.decode.state_names).index(biases[0])
    assert tuple(qwen.decode._state_values[index].shape) == (64 + 2 * 32,)     # q + k + v rows of the packed projection


def test_the_rope_base_is_read_from_the_config():
    def table(theta):
        model = _llama()
        if isinstance(getattr(model.config, "rope_parameters", None), dict):
            model.config.rope_parameters = {**model.config.rope_parameters, "rope_theta": theta}
        else:
            model.config.rope_theta = theta
        runtime = aoto.compile_llama_static_cache(model, prompt_length=8, **_options())
        index = list(runtime.decode.state_names).index("cosine_table")
        return runtime.decode._state_values[index].float().cpu()

    low, high = table(10000.0), table(500000.0)
    assert low.shape == high.shape and not torch.equal(low, high)
    # position 1, slowest pair of a 16-wide head: cos(theta^(-14/16))
    expected = torch.cos(torch.tensor(500000.0 ** (-14 / 16)))
    assert abs(float(high[1, 7]) - float(expected)) < 1e-2


def test_compile_time_refusals():
    model = _qwen2()
    with pytest.raises(CompilationError, match="memory policy"):
        aoto.compile_qwen2_static_cache(model, prompt_length=8, **_options(memory="frugal"))
    with pytest.raises(CompilationError):
        aoto.compile_qwen2_static_cache(model, prompt_length=0, **_options())
    with pytest.raises(CompilationError):                                    # 8 + 60 > 64 positions
        aoto.compile_qwen2_static_cache(model, prompt_length=8, max_new_tokens=60, quantize=GROUP)
    with pytest.raises(CompilationError, match="eval"):
        aoto.compile_qwen2_static_cache(model.train(), prompt_length=8, **_options())
    with pytest.raises(UnsupportedModelError, match="bfloat16"):            # dense weights are read as they are
        aoto.compile_qwen2_static_cache(_qwen2().float(), prompt_length=8, max_new_tokens=NEW)


# ---------------------------------------------------------------------------
# masks
# ---------------------------------------------------------------------------

def test_prefill_mask_is_causal_at_full_width_and_hides_left_padding():
    full = torch.from_numpy(prefill_mask(6, 6)).reshape(6, 6)
    assert torch.equal(full, torch.ones(6, 6, dtype=torch.bool).tril())
    padded = torch.from_numpy(prefill_mask(4, 6)).reshape(6, 6)
    assert not padded[:, :2].any()                                           # nobody reads a pad key
    assert not padded[:2].any()                                              # pad rows admit nothing
    assert torch.equal(padded[2:, 2:], torch.ones(4, 4, dtype=torch.bool).tril())
    with pytest.raises(BucketRangeError):
        prefill_mask(7, 6)
    with pytest.raises(PlanInputError):
        prefill_mask(0, 6)


# ---------------------------------------------------------------------------
# the bucketed runtime
# ---------------------------------------------------------------------------

@pytest.fixture(scope="module")
def bucketed():
    model = _qwen2()
    runtime = aoto.compile_qwen2_bucketed(model, prompt_lengths=(4, 8, 16), **_options())
    return model, runtime


def test_the_smallest_fitting_bucket_is_picked(bucketed):
    _, runtime = bucketed
    assert runtime.prompt_lengths == (4, 8, 16) and runtime.max_prompt_length == 16 and runtime.family == "qwen2"
    assert [runtime.bucket_for(n).prompt_length for n in (1, 4, 5, 8, 9, 16)] == [4, 4, 8, 8, 16, 16]
    with pytest.raises(BucketRangeError):
        runtime.bucket_for(17)
    with pytest.raises(PlanInputError):
        runtime.bucket_for(0)


def test_bucket_widths_must_be_positive_sorted_and_unique():
    model = _qwen2()
    for widths in ((), (8, 4), (4, 4), (0, 4), (-2,)):
        with pytest.raises(CompilationError):
            aoto.compile_qwen2_bucketed(model, prompt_lengths=widths, **_options())


def test_the_buckets_share_one_copy_of_the_weights(bucketed):
    _, runtime = bucketed
    first = runtime.buckets[0]
    anchor = {name: tensor.data_ptr() for name, tensor in zip(first.decode.state_names, first.decode._state_values)
              if name.endswith(("_packed", "_scales")) or name == "embed_tokens_weight"}
    assert len(anchor) >= 2 * 5 * 2
    for bucket in runtime.buckets:
        for plan in (bucket.prefill, bucket.decode):
            for name, tensor in zip(plan.state_names, plan._state_values):
                if name in anchor:
                    assert tensor.data_ptr() == anchor[name], f"{name} was copied for bucket {bucket.prompt_length}"
    # the report of one bucket counts every tensor once, tied and shared ones included
    footprint = first.memory_footprint()
    unique = {}
    for plan in (first.prefill, first.decode):
        for tensor in plan._state_values:
            unique[tensor.data_ptr()] = tensor.numel() * tensor.element_size()
    assert footprint.weights_bytes == sum(unique.values())


@pytest.mark.parametrize("length", [1, 3, 5, 8, 11, 16])
def test_bucketed_prefill_matches_the_model_for_every_length(bucketed, length):
    """Left padding is invisible: the last-row logits are the model's for the unpadded prompt."""

    model, runtime = bucketed
    prompt = torch.randint(0, 128, (1, length), generator=torch.Generator().manual_seed(length))
    bucket = runtime.bucket_for(length)
    logits, _ = OracleRuntime(bucket).prefill(prompt)
    with torch.no_grad():
        want = model(prompt).logits[:, -1:, :]
    # the plan multiplies 4-bit weights, the model its dense ones: compare against the plan of
    # exactly this length too, which must agree far more closely
    exact = aoto.compile_qwen2_static_cache(model, prompt_length=length, **_options())
    same, _ = OracleRuntime(exact).prefill(prompt)
    scale = float(same.float().abs().max())
    assert float((logits.float() - same.float()).abs().max()) <= 2e-2 * scale
    assert int(logits.float().argmax()) == int(same.float().argmax()) or \
        float(same.float().topk(2).values.diff().abs()) < 2e-2 * scale
    assert float((logits.float() - want.float()).abs().max()) <= 0.35 * float(want.float().abs().max())


def test_bucketed_generation_matches_a_per_length_compile(bucketed):
    model, runtime = bucketed
    prompt = torch.randint(0, 128, (1, 6), generator=torch.Generator().manual_seed(6))
    wide = OracleRuntime(runtime.bucket_for(6))
    tokens, trace, _ = wide.greedy(prompt, NEW)
    exact = aoto.compile_qwen2_static_cache(model, prompt_length=6, **_options())
    want, want_trace, _ = OracleRuntime(exact).greedy(prompt, NEW)
    for step, (got, expected) in enumerate(zip(trace, want_trace)):
        scale = float(expected.float().abs().max())
        assert float((got.float() - expected.float()).abs().max()) <= 2e-2 * scale, f"step {step}"
    gaps = [float(t.float().reshape(-1).topk(2).values.diff().abs()) for t in want_trace]
    assert tokens == want or min(gaps) < 5e-2, f"tokens {tokens} vs {want}, top-2 gaps {gaps}"


# ---------------------------------------------------------------------------
# memory report
# ---------------------------------------------------------------------------

def test_the_memory_report_counts_the_cache_and_the_weights_once():
    runtime = aoto.compile_qwen2_static_cache(_qwen2(), prompt_length=8, **_options())
    assert runtime.memory == "latency"                                       # the default policy of a decode runtime
    footprint = runtime.memory_footprint()
    layers, kv_heads, head_dim, capacity = 2, 2, 16, 8 + NEW
    assert footprint.cache_bytes == layers * 2 * kv_heads * capacity * head_dim * 2
    assert footprint.weights_bytes > 0 and footprint.step_peak_bytes >= footprint.weights_bytes + footprint.cache_bytes
    assert "weights" in footprint.describe() and "cache" in footprint.describe()
    assert runtime.check_memory_budget(footprint.step_peak_bytes) == footprint
    with pytest.raises(MemoryBudgetError, match="budget"):
        runtime.check_memory_budget(footprint.step_peak_bytes - 1)


def test_decode_contract_checks_run_before_anything_is_launched():
    runtime = aoto.compile_qwen2_static_cache(_qwen2(), prompt_length=8, **_options())
    with pytest.raises(PlanInputError):
        runtime.greedy_generate(torch.zeros((1, 8), dtype=torch.int64), max_new_tokens=NEW + 1)
    with pytest.raises(PlanInputError):
        runtime.greedy_generate(torch.zeros((1, 8), dtype=torch.int64), max_new_tokens=-1)
    # the oracle over the decode plan accepts exactly the operands the plan declares
    mask = torch.ones((1, 1, 1, 8 + NEW), dtype=torch.bool)
    cache = torch.zeros((2, 2, 1, 2, 8 + NEW, 16), dtype=torch.bfloat16)
    logits, new_cache = run_module_plan(runtime.decode, torch.zeros((1, 1), dtype=torch.int64),
                                        torch.zeros((1, 1), dtype=torch.int64), mask, cache)
    assert logits.shape == (1, 1, 128) and new_cache.shape == cache.shape
