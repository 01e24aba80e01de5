"""Parity on the configurations the benchmark itself times.

* the full Qwen2.5-0.5B-shaped request exactly as ``bench.py`` builds it (24 layers,
  prompt 128, 64 greedy tokens, model seed 0, prompt seed 1): identical greedy tokens, every
  decode step's logits against the oracle interpreter (``KL <= 1e-3`` and a bound on the
  max-abs error that is explained where it is set), for the persistent step kernel and for the
  per-operation plan, and on three steps the distance of GPU and oracle from the same graph
  evaluated without intermediate rounding;
* every point of the packed-matmul sweep (``bench.SWEEP_SHAPES x bench.SWEEP_ROWS``) with
  weights from the reference packer, against the oracle;
* a two-layer cut of the Llama-3-8B shape (head dim 128, window 1280, K = 14 336) through the
  step kernel, every step against the oracle on the same incoming cache;
* a two-layer cut of the Qwen2.5-0.5B shape against what the REFERENCE's adapter modules
  computed for it (``golden/adapter_eager_qwen05b_cut.npz``), at the same bound.
"""

import pytest
import torch

import aotolith_b200 as aoto
import bench
from aotolith_b200.models.synthetic import llama3_8b_shaped
from oracle import ops_ref as ref
from oracle.interp import OracleRuntime
from tests.golden_util import real_shape_fixture
from tests.helpers import activations, exact_packed_matmul, packed_weight, rel_max_error

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2
KL_TOL = 1e-3


def rel_err(actual, expected):
    expected = expected.float().cpu().reshape(-1)
    return float((actual.float().cpu().reshape(-1) - expected).abs().max()) / max(float(expected.abs().max()), 1e-30)


def kl(expected, actual):
    p = torch.log_softmax(expected.float().cpu().reshape(-1), dim=-1)
    q = torch.log_softmax(actual.float().cpu().reshape(-1), dim=-1)
    return float((p.exp() * (p - q)).sum())


def top2_gap(logits):
    top = logits.float().reshape(-1).topk(2).values
    return float(top[0] - top[1])


def session_steps(runtime, session, first_token, cache, valid_length, forced_tokens):
    """Run the device-resident stepper one step at a time, feeding ``forced_tokens``.

    Returns the logits of every step and the tokens the stepper picked itself.
    """

    logits, picked = [], []
    token = first_token
    for forced in forced_tokens:
        out = session.run(token.reshape(1, 1), cache, valid_length, 1)
        picked.append(int(out[0]))
        logits.append(session.logits.reshape(-1).clone() if session.mode == "kernel" else None)
        cache = session.final_cache(1)
        valid_length += 1
        token = torch.tensor([[forced]], device=runtime.device)
    return logits, picked


# At the full depth of the benchmarked model two correct bf16 pipelines are farther apart than the
# target's 1e-2: the ORACLE sits 1.0-1.5e-2 of the logit scale away from the same graph evaluated
# without intermediate rounding (24 layers of one-ulp differences; measured on this model, every
# decode step). So the full-depth test holds the GPU to the sharper statement - it is at least as
# close to the unrounded evaluation as the oracle is - and to a sanity bound against the oracle;
# the 1e-2 bound itself is held where it can hold, on the two-layer cuts below.
FULL_DEPTH_SANITY = 2.5e-2
FLOOR_SLACK = 1.25


def test_benchmarked_request_matches_oracle(cuda):
    """BASELINE config 2 as the benchmark runs it: 24 layers, prompt 128, 64 greedy tokens."""

    from aotolith_b200 import ops
    from aotolith_b200.models.session import DecodeSession

    model, _ = bench.build_model("qwen25_05b", seed=0)
    runtime = aoto.compile_qwen2_static_cache(
        model, prompt_length=bench.PROMPT, max_new_tokens=bench.NEW_TOKENS, quantize=bench.GROUP
    )
    prompt = bench.seeded_prompt(model.config.vocab_size, 1)
    oracle = OracleRuntime(runtime)
    # the oracle's greedy loop, keeping the cache every step starts from
    valid = bench.PROMPT
    logits, cache = oracle.prefill(prompt)
    trace, caches = [logits], []
    token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
    want_tokens = [int(token)]
    for _ in range(bench.NEW_TOKENS - 1):
        valid += 1
        caches.append(cache)
        logits, cache = oracle.decode(token, cache, valid)
        trace.append(logits)
        token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        want_tokens.append(int(token))
    gaps = [top2_gap(t[:, -1]) for t in trace]

    # the public call, as the end-to-end arm of the benchmark makes it
    tokens = runtime.greedy_generate(prompt).cpu()[0].tolist()
    assert tokens == want_tokens, f"oracle top-2 gaps per step: {gaps}"

    logits, compact = runtime.prefill_ids(prompt)
    assert rel_err(logits[:, -1], trace[0][:, -1]) < FULL_DEPTH_SANITY and kl(trace[0][:, -1], logits[:, -1]) < KL_TOL
    cache = runtime.pad_cache(compact)
    first = ops.argmax(logits[:, -1, :]).reshape(1, 1)
    assert int(first) == want_tokens[0]

    # persistent step kernel: every step's logits, fed with the oracle's tokens
    kernel = DecodeSession(runtime)
    assert kernel.mode == "kernel"
    step_logits, picked = session_steps(runtime, kernel, first, cache, bench.PROMPT, want_tokens[1:])
    assert picked == want_tokens[1:], f"oracle top-2 gaps per step: {gaps}"
    for step, got in enumerate(step_logits):
        want = trace[step + 1]
        assert rel_err(got, want) < FULL_DEPTH_SANITY, f"kernel step {step}: {rel_err(got, want):.3e}"
        assert kl(want, got) < KL_TOL, f"kernel step {step}"

    # per-operation plan: the same steps through decode_token
    token, valid = first, bench.PROMPT
    plan_logits = []
    for step in range(bench.NEW_TOKENS - 1):
        valid += 1
        got, cache = runtime.decode_token(token, cache, valid, verify_token=False)
        want = trace[step + 1]
        assert rel_err(got, want) < FULL_DEPTH_SANITY, f"plan step {step}: {rel_err(got, want):.3e}"
        assert kl(want, got) < KL_TOL, f"plan step {step}"
        plan_logits.append(got.reshape(-1).clone())
        token = torch.tensor([[want_tokens[step + 1]]], device=runtime.device)

    # the yardstick: three steps evaluated without intermediate rounding from the oracle's own cache
    unrounded = OracleRuntime(runtime, unrounded=True)
    for step in (0, 31, 62):
        exact, _ = unrounded.decode(torch.tensor([[want_tokens[step]]]), caches[step], bench.PROMPT + 1 + step)
        floor = rel_err(trace[step + 1], exact)
        for name, got in (("kernel", step_logits[step]), ("plan", plan_logits[step])):
            error = rel_err(got, exact)
            assert error <= max(REL_TOL, FLOOR_SLACK * floor), (
                f"{name} step {step}: {error:.3e} from the unrounded evaluation, the oracle is {floor:.3e} from it")


@pytest.mark.parametrize("K,N,bias", bench.SWEEP_SHAPES)
def test_every_sweep_point_matches_oracle(cuda, K, N, bias):
    """The 15 timed points of the packed-matmul sweep, with real packed weights."""

    from aotolith_b200 import ops

    packed, scales = packed_weight(50 + N % 97, N, K, bench.GROUP)
    addend = activations(51, N, std=0.5) if bias else None
    packed_dev, scales_dev = packed.to(cuda), scales.to(cuda)
    addend_dev = addend.to(cuda) if bias else None
    for M in bench.SWEEP_ROWS:
        x = activations(52 + M, M, K)
        got = ops.qmatmul(x.to(cuda), packed_dev, scales_dev, group_size=bench.GROUP, addend=addend_dev).cpu()
        want = ref.packed_matmul(x, packed, scales, bench.GROUP, addend=addend)
        assert got.shape == (M, N)
        assert rel_max_error(got, want) < REL_TOL, f"M={M}: {ops.qmatmul_variant(M, N, K, bench.GROUP)}"
        exact = exact_packed_matmul(x, packed, scales, bench.GROUP)
        if bias:
            exact = exact + addend.double()
        assert rel_max_error(got, exact) < 4e-3, f"M={M}"


def test_llama_8b_shaped_layers_through_the_step_kernel(cuda):
    """Head dim 128, window 1280 (split attention form), K = 14 336 block lists."""

    from aotolith_b200 import ops
    from aotolith_b200.models.session import DecodeSession

    model = llama3_8b_shaped(seed=3, layers=2)
    runtime = aoto.compile_llama_static_cache(model, prompt_length=1024, max_new_tokens=256, quantize=64)
    assert runtime.cache_capacity == 1280
    prompt = torch.randint(0, 128256, (1, 1024), generator=torch.Generator().manual_seed(14))
    logits, compact = runtime.prefill_ids(prompt)
    cache = runtime.pad_cache(compact)
    token = ops.argmax(logits[:, -1, :]).reshape(1, 1)
    kernel = DecodeSession(runtime)
    assert kernel.mode == "kernel"
    oracle = OracleRuntime(runtime)
    unrounded = OracleRuntime(runtime, unrounded=True)
    valid = 1024
    floor = 0.0
    for step in range(4):
        valid += 1
        want_logits, want_cache = oracle.decode(token.cpu(), cache.cpu(), valid)
        picked = kernel.run(token, cache, valid - 1, 1)
        got_logits = kernel.logits.reshape(-1).clone()
        got_cache = kernel.final_cache(1)
        if step == 0:
            # rows of 4096 and 14 336 products: the oracle's own distance from the unrounded evaluation of
            # the same step says how close two bf16 pipelines can be expected to agree here
            exact, _ = unrounded.decode(token.cpu(), cache.cpu(), valid)
            floor = rel_err(want_logits, exact)
            assert rel_err(got_logits, exact) <= max(REL_TOL, FLOOR_SLACK * floor), (
                f"{rel_err(got_logits, exact):.3e} from the unrounded evaluation, the oracle is {floor:.3e} from it")
        bound = max(REL_TOL, 2 * floor)  # both sides carry their own rounding
        assert rel_err(got_logits, want_logits) < bound, f"step {step}: {rel_err(got_logits, want_logits):.3e} (floor {floor:.3e})"
        assert kl(want_logits, got_logits) < KL_TOL, f"step {step}"
        assert rel_err(got_cache, want_cache) < REL_TOL
        # 128 256 bf16 logits of a random-init model tie at the top (a top-2 gap of exactly 0 occurs): the
        # token must be the argmax of the kernel's own logits and sit within rounding of the oracle's maximum
        flat = want_logits.float().reshape(-1)
        assert int(picked[0]) == int(got_logits.float().argmax())
        assert float(flat[int(picked[0])]) >= float(flat.max()) - bound * float(flat.abs().max()), f"gap {top2_gap(want_logits)}"
        token, cache = picked.reshape(1, 1), got_cache


def test_real_shape_cut_matches_reference_adapters(cuda):
    """GPU against the reference's own adapter modules at the target's tolerance."""

    from aotolith_b200 import ops
    from aotolith_b200.models.session import DecodeSession

    model, data = real_shape_fixture()
    runtime = aoto.compile_qwen2_static_cache(
        model, prompt_length=data["prompt_length"], max_new_tokens=data["new_tokens"], quantize=data["group"]
    )
    prompt = torch.from_numpy(data["prompt"])
    want_tokens = data["tokens"].tolist()
    assert runtime.greedy_generate(prompt).cpu()[0].tolist() == want_tokens
    logits, compact = runtime.prefill_ids(prompt)
    assert rel_err(logits[:, -1], data["logits"][0]) < REL_TOL and kl(data["logits"][0], logits[:, -1]) < KL_TOL
    cache = runtime.pad_cache(compact)
    first = ops.argmax(logits[:, -1, :]).reshape(1, 1)
    kernel = DecodeSession(runtime)
    assert kernel.mode == "kernel"
    step_logits, picked = session_steps(runtime, kernel, first, cache, data["prompt_length"], want_tokens[1:])
    assert picked == want_tokens[1:]
    for step, got in enumerate(step_logits):
        want = data["logits"][step + 1]
        assert rel_err(got, want) < REL_TOL, f"step {step}: {rel_err(got, want):.3e}"
        assert kl(want, got) < KL_TOL
