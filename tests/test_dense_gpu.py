"""Dense bf16 projections and dense decoders on the GPU, through the C ABI.

The products are compared with "accumulate in fp32, round once to bf16" over the same bf16 operands
(``1e-2 * max|expected|``) and with an unrounded float64 evaluation (``4e-3 * max|exact|``). The
decoders are the reference's dense adapters (src/aotolith/models/decoder.py:282-520) over the toy
weights; the tokens are the ones the reference's eager adapter modules produce.
"""

import numpy as np
import pytest
import torch

from tests.golden_util import GOLDEN
from tests.helpers import activations, rel_max_error

pytestmark = pytest.mark.gpu

ORACLE_TOL = 1e-2
EXACT_TOL = 4e-3


def _ops():
    import aotolith_b200.ops as ops

    return ops


def dense_weight(seed: int, n_rows: int, K: int, std: float = 0.02) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy((rng.standard_normal((n_rows, K)) * std).astype(np.float32)).bfloat16()


def _rounded(x, weight):
    return (x.float() @ weight.float().T).bfloat16()


def _check(got, rounded, exact):
    assert got.dtype == torch.bfloat16 and got.shape == rounded.shape
    assert rel_max_error(got, rounded) <= ORACLE_TOL
    assert rel_max_error(got.double(), exact) <= max(EXACT_TOL, 1.25 * rel_max_error(rounded.double(), exact))


# the benchmarked decoders' projection shapes (0.5B and 8B) beside ragged small ones
SHAPES = [(896, 1152), (896, 4864), (4864, 896), (4096, 6144), (14336, 4096), (64, 24), (8, 3), (72, 130), (1000, 17),
          (32, 16), (96, 19), (896, 18947), (32768, 40)]


@pytest.mark.parametrize("K,N", SHAPES)
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 13])
def test_dmatmul_plain(cuda, K, N, M):
    ops = _ops()
    x, weight = activations(3, M, K), dense_weight(4, N, K)
    got = ops.dmatmul(x.to(cuda), weight.to(cuda)).cpu()
    _check(got, _rounded(x, weight), x.double() @ weight.double().T)
    one_row = "dgemv_mma" if K % 32 == 0 and N >= 16 else "dgemv"
    assert ops.dmatmul_variant(M, N, K) == (one_row if M == 1 else "dgemm_rows")


@pytest.mark.parametrize("K,N", [(896, 1152), (4096, 4096), (64, 24), (72, 130)])
@pytest.mark.parametrize("M", [1, 4, 7])
def test_dmatmul_bias_residual_and_scales(cuda, K, N, M):
    ops = _ops()
    x, weight = activations(5, M, K), dense_weight(6, N, K)
    bias = dense_weight(7, 1, N, std=0.5).reshape(N)
    residual = activations(8, M, N)
    exact = x.double() @ weight.double().T
    got = ops.dmatmul(x.to(cuda), weight.to(cuda), addend=bias.to(cuda)).cpu()
    _check(got, (bias.float() + x.float() @ weight.float().T).bfloat16(), bias.double() + exact)
    got = ops.dmatmul(x.to(cuda), weight.to(cuda), addend=residual.to(cuda), alpha=0.5, beta=2.0).cpu()
    _check(got, (2.0 * residual.float() + 0.5 * (x.float() @ weight.float().T)).bfloat16(),
           2.0 * residual.double() + 0.5 * exact)


@pytest.mark.parametrize("K,N", [(896, 4864), (4096, 14336), (64, 24), (72, 130), (896, 18950), (96, 19)])
def test_dmatmul_paired_gate_up(cuda, K, N):
    """One row, two weights: ``silu(x W1^T) * (x W2^T)`` as runtime/mlx_ops/__init__.py:589-596 states it."""

    ops = _ops()
    x, first, second = activations(9, 1, K), dense_weight(10, N, K, std=0.05), dense_weight(11, N, K, std=0.05)
    got = ops.dmatmul(x.to(cuda), first.to(cuda), weight2=second.to(cuda)).cpu()
    gate, up = x.double() @ first.double().T, x.double() @ second.double().T
    exact = gate * (up / (1.0 + torch.exp(-gate)))
    product, other = _rounded(x, first), _rounded(x, second)
    rounded = product * (other / (1.0 + torch.exp(-product)))
    assert got.dtype == torch.bfloat16 and got.shape == (1, N)
    assert rel_max_error(got.double(), exact) <= max(EXACT_TOL, 1.25 * rel_max_error(rounded.double(), exact))
    assert ops.dmatmul_variant(1, N, K, paired=True) == ("dgemv_mma" if K % 32 == 0 and K < 2048 else "dgemv")


@pytest.mark.parametrize("M", [1, 6])
def test_dmatmul_gated_epilogue(cuda, M):
    ops = _ops()
    K, N = 896, 1152
    x, weight, gate = activations(12, M, K), dense_weight(13, N, K), activations(14, M, N)
    got = ops.dmatmul(x.to(cuda), weight.to(cuda), gate=gate.to(cuda)).cpu()
    exact = (x.double() @ weight.double().T) * (gate.double() / (1.0 + torch.exp(-gate.double())))
    rounded = _rounded(x, weight) * (gate / (1.0 + torch.exp(-gate)))
    assert rel_max_error(got.double(), exact) <= max(EXACT_TOL, 1.25 * rel_max_error(rounded.double(), exact))


def test_dmatmul_refuses_what_the_kernel_does_not_cover(cuda):
    from aotolith_b200.errors import PlanInputError

    ops = _ops()
    x = activations(1, 1, 12).to(cuda)                       # K is not a multiple of eight elements
    with pytest.raises((PlanInputError, RuntimeError)):
        ops.dmatmul(x, dense_weight(2, 8, 12).to(cuda))
    x = activations(1, 2, 64).to(cuda)                       # the paired form takes one row
    w = dense_weight(2, 8, 64).to(cuda)
    with pytest.raises((PlanInputError, RuntimeError)):
        ops.dmatmul(x, w, weight2=w)


# ---------------------------------------------------------------------------
# whole dense decoders
# ---------------------------------------------------------------------------

def _rel_err(actual, expected):
    expected = expected.float().cpu()
    return float((actual.float().cpu() - expected).abs().max() / expected.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("family", ["qwen2", "llama"])
def test_dense_decoder_matches_oracle_and_reference(cuda, family):
    """Prefill, decode steps and greedy tokens of a toy decoder compiled without quantisation."""

    import aotolith_b200 as aoto
    from oracle.interp import OracleRuntime
    from tests.golden_util import NEW, PROMPT, eager_fixture

    model, _ = eager_fixture(family)
    data = np.load(GOLDEN / f"adapter_eager_dense_{family}.npz")
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, family=family
    )
    oracle = OracleRuntime(runtime)
    prompt = torch.from_numpy(data["prompt"])
    logits, compact = runtime.prefill_ids(prompt)
    want_logits, want_cache = oracle.prefill(prompt)
    assert _rel_err(logits, want_logits) < 2e-2
    assert _rel_err(logits, torch.from_numpy(data["prefill_logits"])) < 3e-2   # the reference's eager adapters
    cache = runtime.pad_cache(compact)
    assert _rel_err(cache, want_cache) < 2e-2
    token = torch.tensor([[int(want_logits[:, -1].float().argmax())]])
    valid = PROMPT
    for step in range(NEW - 1):
        valid += 1
        logits, cache = runtime.decode_token(token, cache, valid)
        want_logits, want_cache = oracle.decode(token, want_cache, valid)
        assert _rel_err(logits, want_logits) < 2e-2, f"step {step}"
        assert _rel_err(cache, want_cache) < 2e-2
        token = torch.tensor([[int(want_logits[:, -1].float().argmax())]])
    tokens = runtime.greedy_generate(prompt).cpu()
    assert tokens.shape == (1, NEW)
    assert tokens[0].tolist() == data["tokens"].tolist()
    assert torch.equal(runtime.greedy_generate(prompt).cpu(), tokens)   # the stepper is reusable
