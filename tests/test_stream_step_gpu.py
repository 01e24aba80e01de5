"""The streamed decode-step kernel against the kernel that reads the weights in place.

Both run the same stage program over the same weights; one takes them from per-warp
streams laid out by ``runtime/stream_plan.py``, the other from the reference's packed
format. Tokens must be identical; logits and caches agree to bf16 rounding (the two
kernels sum a row's blocks in different orders). Both are also held to the oracle.
"""

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200 import ops
from aotolith_b200.models import session as session_module
from aotolith_b200.models.session import DecodeSession
from aotolith_b200.models.synthetic import SyntheticDecoder, qwen25_05b_shaped
from oracle.interp import OracleRuntime

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


def rel_err(actual, expected):
    expected = expected.float().cpu().reshape(-1)
    return float((actual.float().cpu().reshape(-1) - expected).abs().max()) / max(float(expected.abs().max()), 1e-30)


def same_until(a, b) -> int:
    """Number of leading tokens two generations share."""

    a, b = a.tolist(), b.tolist()
    for index, (x, y) in enumerate(zip(a, b)):
        if x != y:
            return index
    return min(len(a), len(b))


def two_sessions(runtime):
    streamed = DecodeSession(runtime)
    session_module.STREAM_STEP_DISABLED = True
    try:
        in_place = DecodeSession(runtime)
    finally:
        session_module.STREAM_STEP_DISABLED = False
    assert streamed.kernel_name == "stream_step_kernel"
    assert in_place.kernel_name == "decode_step_kernel"
    return streamed, in_place


def start(runtime, prompt):
    logits, compact = runtime.prefill_ids(prompt)
    return ops.argmax(logits[:, -1, :]).reshape(1, 1), runtime.pad_cache(compact)


@pytest.mark.parametrize("layers,prompt_length,new_tokens", [(3, 24, 9), (2, 130, 40)])
def test_streamed_and_in_place_kernels_agree(cuda, layers, prompt_length, new_tokens):
    model = qwen25_05b_shaped(seed=8, layers=layers)
    runtime = aoto.compile_qwen2_static_cache(model, prompt_length=prompt_length, max_new_tokens=new_tokens, quantize=64)
    prompt = torch.randint(0, 151936, (1, prompt_length), generator=torch.Generator().manual_seed(15))
    token, cache = start(runtime, prompt)
    streamed, in_place = two_sessions(runtime)
    for steps in (1, new_tokens - 1):
        a = streamed.run(token, cache, prompt_length, steps).cpu()
        b = in_place.run(token, cache, prompt_length, steps).cpu()
        assert a.tolist() == b.tolist()
        assert rel_err(streamed.logits, in_place.logits) < REL_TOL
        assert rel_err(streamed.final_cache(steps), in_place.final_cache(steps)) < REL_TOL
    # the window is moved bit for bit: every slot but the last of the next cache is a copy
    streamed.run(token, cache, prompt_length, 1)
    in_place.run(token, cache, prompt_length, 1)
    assert torch.equal(streamed.final_cache(1)[:, :, :, :, :-1], cache[:, :, :, :, 1:])
    # the appended slot is a projection result: the kernels may round it an ulp apart
    assert rel_err(streamed.final_cache(1)[:, :, :, :, -1], in_place.final_cache(1)[:, :, :, :, -1]) < REL_TOL


def test_streamed_kernel_matches_oracle_step_by_step(cuda):
    model = qwen25_05b_shaped(seed=9, layers=2)
    runtime = aoto.compile_qwen2_static_cache(model, prompt_length=20, max_new_tokens=6, quantize=64)
    prompt = torch.randint(0, 151936, (1, 20), generator=torch.Generator().manual_seed(16))
    want_tokens, trace, _ = OracleRuntime(runtime).greedy(prompt, 6)
    token, cache = start(runtime, prompt)
    session = DecodeSession(runtime)
    assert session.kernel_name == "stream_step_kernel"
    valid = 20
    for step in range(5):
        picked = session.run(token, cache, valid, 1)
        assert rel_err(session.logits, trace[step + 1]) < REL_TOL, f"step {step}"
        assert int(picked[0]) == want_tokens[step + 1]
        cache, valid = session.final_cache(1), valid + 1
        token = torch.tensor([[want_tokens[step + 1]]], device=runtime.device)


def test_streamed_kernel_with_wide_heads_and_long_rows(cuda):
    """Head dim 128, K = 7168 (56 blocks a tile, several pieces per share), untied head."""

    model = SyntheticDecoder(
        model_type="llama", vocab_size=49152, hidden_size=1024, intermediate_size=7168, num_hidden_layers=2,
        num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=256, rope_theta=5e5,
        rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, seed=22,
    )
    runtime = aoto.compile_llama_static_cache(model, prompt_length=16, max_new_tokens=7, quantize=64)
    prompt = torch.randint(0, 49152, (1, 16), generator=torch.Generator().manual_seed(17))
    token, cache = start(runtime, prompt)
    streamed, in_place = two_sessions(runtime)
    a = streamed.run(token, cache, 16, 6).cpu()
    b = in_place.run(token, cache, 16, 6).cpu()
    assert a.tolist() == b.tolist()
    assert rel_err(streamed.logits, in_place.logits) < REL_TOL
    assert rel_err(streamed.final_cache(6), in_place.final_cache(6)) < REL_TOL
    want, _, _ = OracleRuntime(runtime).greedy(prompt, 7)
    assert runtime.greedy_generate(prompt).cpu()[0].tolist() == want


@pytest.mark.parametrize("head_dim,kv_heads,prompt_length,new_tokens",
                         [(64, 2, 280, 25), (128, 2, 300, 30), (64, 2, 1000, 40), (128, 2, 1000, 24), (128, 1, 700, 20),
                          (128, 8, 40, 300)])
def test_streamed_kernel_with_a_window_longer_than_its_buffers(cuda, head_dim, kv_heads, prompt_length, new_tokens):
    """More than sixteen keys a warp: every kv head's window is spread over many CTAs and merged.

    Capacities 305, 330, 1040, 1024, 720 and 340: groups of seven, four, four again (one kv head: as
    many slices as the window has runs of sixteen keys) and one query head per kv head; windows that
    are nearly full and one that starts at 41 of 340 slots (fewer slices than CTAs per kv head).
    The step's own key is the last slot and comes from shared memory. Held to the kernel that reads
    the weights in place over the whole generation, to the oracle on the first steps.
    """

    if head_dim == 64:
        model = qwen25_05b_shaped(seed=12, layers=2, max_position_embeddings=2048)
        compile_fn, vocab = aoto.compile_qwen2_static_cache, 151936
    else:
        model = SyntheticDecoder(
            model_type="llama", vocab_size=32000, hidden_size=1024, intermediate_size=2816, num_hidden_layers=2,
            num_attention_heads=4 if kv_heads == 1 else 8, num_key_value_heads=kv_heads, head_dim=128,
            max_position_embeddings=2048, rope_theta=5e5,
            rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, seed=23,
        )
        compile_fn, vocab = aoto.compile_llama_static_cache, 32000
    runtime = compile_fn(model, prompt_length=prompt_length, max_new_tokens=new_tokens, quantize=64)
    prompt = torch.randint(0, vocab, (1, prompt_length), generator=torch.Generator().manual_seed(18))
    token, cache = start(runtime, prompt)
    streamed, in_place = two_sessions(runtime)
    steps = new_tokens - 1
    a = streamed.run(token, cache, prompt_length, steps).cpu()
    b = in_place.run(token, cache, prompt_length, steps).cpu()
    same = same_until(a, b)
    if same == steps:
        assert rel_err(streamed.logits, in_place.logits) < REL_TOL
        assert rel_err(streamed.final_cache(steps), in_place.final_cache(steps)) < REL_TOL
    else:
        # a random model's best two logits can tie within rounding: the step where the kernels part must
        # be such a tie (both kernels are run up to it again: their logits there are what is compared)
        assert same >= 2
        streamed.run(token, cache, prompt_length, same + 1)
        in_place.run(token, cache, prompt_length, same + 1)
        assert rel_err(streamed.logits, in_place.logits) < REL_TOL
        logits = in_place.logits.float().reshape(-1)
        gap = float(logits[int(b[same])] - logits[int(a[same])])
        assert 0 <= gap <= REL_TOL * float(logits.abs().max()), (same, gap)
    streamed.run(token, cache, prompt_length, 1)
    assert torch.equal(streamed.final_cache(1)[:, :, :, :, :-1], cache[:, :, :, :, 1:])
    if prompt_length <= 300 and new_tokens <= 30:
        want_tokens, trace, _ = OracleRuntime(runtime).greedy(prompt, 3)
        assert a[:2].tolist() == want_tokens[1:3]
        streamed.run(token, cache, prompt_length, 1)
        # the oracle rounds to bf16 where the reference does, and one bf16 step of the largest logit is
        # already 0.4-0.8 % of it: the yardstick is the oracle's own distance from the unrounded evaluation
        exact, _ = OracleRuntime(runtime, unrounded=True).decode(token.cpu(), cache.cpu(), prompt_length + 1)
        rounded, _ = OracleRuntime(runtime).decode(token.cpu(), cache.cpu(), prompt_length + 1)
        floor = rel_err(rounded, exact)
        assert rel_err(streamed.logits, exact) <= max(REL_TOL, 1.25 * floor), (rel_err(streamed.logits, exact), floor)
        assert rel_err(streamed.logits, rounded) < 2.5 * REL_TOL
        assert rel_err(streamed.logits, trace[1]) < 2.5 * REL_TOL
