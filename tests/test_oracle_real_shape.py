"""Pin the oracle to the reference at the size where the target's tolerance holds.

``golden/adapter_eager_qwen05b_cut.npz`` holds what the reference's quantized
adapter modules compute eagerly for a two-layer cut of the Qwen2.5-0.5B shape
(hidden 896, vocabulary 151 936, group 64). At this width a bf16 ulp is small
against the logit scale, so the oracle interpreter is held to the target's own
bound: ``1e-2 * max|logit|`` and a KL bound on the next-token distribution, for
the prefill and for every decode step, plus identical greedy tokens.
"""

import torch

import aotolith_b200 as aoto
from oracle.interp import OracleRuntime
from tests.golden_util import real_shape_fixture

REL_TOL = 1e-2
KL_TOL = 1e-3


def kl(expected, actual):
    p = torch.log_softmax(expected.float().reshape(-1), dim=-1)
    q = torch.log_softmax(actual.float().reshape(-1), dim=-1)
    return float((p.exp() * (p - q)).sum())


def test_oracle_matches_reference_adapters_on_the_real_shape():
    model, data = real_shape_fixture()
    runtime = aoto.compile_qwen2_static_cache(
        model, prompt_length=data["prompt_length"], max_new_tokens=data["new_tokens"], quantize=data["group"]
    )
    tokens, trace, cache = OracleRuntime(runtime).greedy(torch.from_numpy(data["prompt"]), data["new_tokens"])
    assert tokens == data["tokens"].tolist()
    for step, logits in enumerate(trace):
        want = data["logits"][step]
        got = logits[0, -1, :].float()
        error = float((got - want).abs().max()) / float(want.abs().max())
        assert error < REL_TOL, f"step {step}: {error:.3e}"
        assert kl(want, got) < KL_TOL, f"step {step}"
    want_cache = data["final_cache"]
    assert float((cache.float() - want_cache).abs().max()) <= REL_TOL * float(want_cache.abs().max())
