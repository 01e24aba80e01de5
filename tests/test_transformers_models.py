"""Real ``transformers`` decoders through the adapters, without a GPU.

The reference checks its quantized runtime against the checkpoint whose projection weights
were replaced by their own quantise/dequantise round trip and which then runs as the plain
``transformers`` model (tests/test_quantized_qwen2.py:76-124, :240-262). The same here: a tiny
``Qwen2ForCausalLM`` (q/k/v bias, tied embeddings) and a tiny ``LlamaForCausalLM`` are compiled for
the CUDA target, the oracle runs the lowered graphs on the CPU, and its logits are compared with
the round-tripped model's own forward pass - prefill, and every decode step with the tokens fed
back. This pins the adapters (rotary convention, grouped heads, bias packing, cache roll) against
an implementation that shares no code with this repository.
"""

import copy

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.quantize import dequantize_int4, dequantize_int8, quantize_int4, quantize_int8
from oracle.interp import OracleRuntime

transformers = pytest.importorskip("transformers")

GROUP, PROMPT, NEW = 16, 8, 5
TOL = 3e-2


def _build(kind: str) -> torch.nn.Module:
    torch.manual_seed(5)
    common = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-6)
    if kind == "qwen2":
        model = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**common, tie_word_embeddings=True))
    else:
        model = transformers.LlamaForCausalLM(transformers.LlamaConfig(**common, tie_word_embeddings=False))
    return model.to(torch.bfloat16).eval()


def _round_tripped(model: torch.nn.Module, bits: int) -> torch.nn.Module:
    """The model with every projection (and the LM head) replaced by its packed round trip."""

    quantize, dequantize = (quantize_int4, dequantize_int4) if bits == 4 else (quantize_int8, dequantize_int8)
    twin = copy.deepcopy(model)
    embedding = twin.model.embed_tokens.weight.detach().clone()
    with torch.no_grad():
        for module in twin.modules():
            if isinstance(module, torch.nn.Linear):
                packed, scales = quantize(module.weight.float().numpy(), GROUP)
                scales = torch.from_numpy(scales).bfloat16().float().numpy()   # the plan keeps bf16 scales
                restored = torch.from_numpy(dequantize(packed, scales, GROUP)).to(module.weight.dtype)
                module.weight = torch.nn.Parameter(restored)                   # unties a tied LM head
        twin.model.embed_tokens.weight = torch.nn.Parameter(embedding)         # the table stays as it was
    return twin


def _rel(actual, expected):
    expected = expected.float()
    return float((actual.float() - expected).abs().max() / expected.abs().max())


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("kind", ["qwen2", "llama"])
def test_oracle_over_compiled_graphs_matches_the_round_tripped_checkpoint(kind, bits):
    model = _build(kind)
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, quantize_bits=bits
    )
    assert runtime.family == kind
    twin = _round_tripped(model, bits)
    prompt = torch.randint(0, 128, (1, PROMPT), generator=torch.Generator().manual_seed(1))
    oracle = OracleRuntime(runtime)
    logits, cache = oracle.prefill(prompt)
    with torch.no_grad():
        want = twin(prompt).logits[:, -1:, :]
    assert logits.shape == (1, 1, 128)
    assert _rel(logits, want) < TOL
    ids, valid = prompt, PROMPT
    for step in range(NEW - 1):
        token = want[:, -1].float().argmax(dim=-1, keepdim=True)             # the checkpoint's own greedy token
        ids = torch.cat((ids, token), dim=1)
        valid += 1
        logits, cache = oracle.decode(token, cache, valid)
        with torch.no_grad():
            want = twin(ids).logits[:, -1:, :]
        assert _rel(logits, want) < TOL, f"decode step {step}"


def test_the_runtime_outlives_the_model_it_was_compiled_from():
    """The plan holds packed words and scales, not the dense checkpoint (tests/test_quantized_qwen2.py:156-175)."""

    import gc
    import weakref

    model = _build("qwen2")
    runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP)
    alive = weakref.ref(model)
    del model
    gc.collect()
    assert alive() is None
    names = set(runtime.decode.state_names)
    for layer in range(2):
        for name in ("qkv", "o_proj", "gate_proj", "up_proj", "down_proj"):
            assert f"{name}_{layer}_packed" in names and f"{name}_{layer}_scales" in names
    dense = [name for name in names
             if not name.endswith(("_packed", "_scales"))
             and name not in {"cosine_table", "sine_table", "embed_tokens_weight", "final_norm"}
             and not name.startswith(("qkv_bias", "input_norm", "post_attention_norm"))]
    assert dense == []
    tokens, _, _ = OracleRuntime(runtime).greedy(torch.zeros((1, PROMPT), dtype=torch.int64), 2)
    assert len(tokens) == 2


def test_quantizing_requires_a_group_size_that_divides_the_reduction():
    model = _build("qwen2")
    with pytest.raises(ValueError):
        aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=48)


def test_a_llama_model_is_refused_by_the_qwen2_entry_point():
    from aotolith_b200.errors import UnsupportedModelError

    with pytest.raises(UnsupportedModelError):
        aoto.compile_qwen2_static_cache(_build("llama"), prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP)


@pytest.mark.parametrize("kv_heads", [1, 2, 4])
def test_llama_accepts_grouped_and_plain_attention(kv_heads):
    """One kv head for all query heads, grouped, and one per query head
    (tests/test_llama_static_cache.py:170-192 of the reference)."""

    torch.manual_seed(20 + kv_heads)
    config = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=kv_heads,
                                      max_position_embeddings=64, rms_norm_eps=1e-6, tie_word_embeddings=False)
    model = transformers.LlamaForCausalLM(config).to(torch.bfloat16).eval()
    runtime = aoto.compile_llama_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP,
                                              quantize_bits=8)
    assert runtime.num_key_value_heads == kv_heads and runtime.head_dim == 16
    twin = _round_tripped(model, 8)
    prompt = torch.randint(0, 128, (1, PROMPT), generator=torch.Generator().manual_seed(3))
    oracle = OracleRuntime(runtime)
    logits, cache = oracle.prefill(prompt)
    with torch.no_grad():
        want = twin(prompt).logits[:, -1:, :]
    assert _rel(logits, want) < TOL
    token = want[:, -1].float().argmax(dim=-1, keepdim=True)
    logits, _ = oracle.decode(token, cache, PROMPT + 1)
    with torch.no_grad():
        want = twin(torch.cat((prompt, token), dim=1)).logits[:, -1:, :]
    assert _rel(logits, want) < TOL


def test_a_short_prompt_in_a_wide_bucket_matches_the_checkpoint():
    """Left padding is invisible to the model's answer: prompt of 5 in a bucket of 8, eight bits
    (close to lossless), against the round-tripped checkpoint on the unpadded prompt."""

    model = _build("qwen2")
    runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP,
                                              quantize_bits=8)
    twin = _round_tripped(model, 8)
    prompt = torch.randint(0, 128, (1, 5), generator=torch.Generator().manual_seed(9))
    oracle = OracleRuntime(runtime)
    logits, cache = oracle.prefill(prompt)
    with torch.no_grad():
        want = twin(prompt).logits[:, -1:, :]
    assert _rel(logits, want) < TOL
    ids, valid = prompt, 5
    for step in range(NEW - 1):
        token = want[:, -1].float().argmax(dim=-1, keepdim=True)
        ids = torch.cat((ids, token), dim=1)
        valid += 1
        logits, cache = oracle.decode(token, cache, valid)
        with torch.no_grad():
            want = twin(ids).logits[:, -1:, :]
        assert _rel(logits, want) < TOL, f"decode step {step}"
