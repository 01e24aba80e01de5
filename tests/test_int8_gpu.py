"""Eight-bit packed projections on the GPU against the CPU oracle, through the C ABI.

The unpack is byte work and is bit-exact. The products are compared with the
oracle's "round the weight to bf16, accumulate in fp32, round once" at
``1e-2 * max|expected|`` and with an unrounded float64 evaluation of the same
bf16 weights at ``4e-3 * max|exact|``. Mirrors the reference's eight-bit cases
(tests/test_quantize.py:173-240, tests/test_quantized_matmul.py).
"""

import numpy as np
import pytest
import torch

from aotolith_b200.quantize import quantize_int8
from oracle import ops_ref as ref
from tests.golden_util import GOLDEN
from tests.helpers import activations, rel_max_error

pytestmark = pytest.mark.gpu

ORACLE_TOL = 1e-2
EXACT_TOL = 4e-3


def _ops():
    import aotolith_b200.ops as ops

    return ops


def packed_weight_i8(seed: int, n_rows: int, K: int, group: int, std: float = 0.02):
    rng = np.random.default_rng(seed)
    weight = torch.from_numpy((rng.standard_normal((n_rows, K)) * std).astype(np.float32)).bfloat16()
    packed, scales = quantize_int8(weight.float().numpy(), group)
    return torch.from_numpy(packed), torch.from_numpy(scales).bfloat16()


def exact_i8(x, packed, scales, group):
    """float64 product over the bf16 weights the unpack materialises."""

    return x.double() @ ref.dequantize_i8(packed, scales, group).double().T


@pytest.mark.parametrize("K,N,group", [(896, 1152, 64), (128, 48, 64), (64, 24, 16), (4096, 512, 64), (96, 40, 32), (8, 3, 8)])
def test_dequantize_i8_bit_exact(cuda, K, N, group):
    ops = _ops()
    packed, scales = packed_weight_i8(1, N, K, group)
    got = ops.dequantize_i8(packed.to(cuda), scales.to(cuda), group).cpu()
    want = ref.dequantize_i8(packed, scales, group)
    assert got.dtype == torch.bfloat16 and got.shape == (N, K)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_dequantize_i8_every_byte_value(cuda):
    """All 256 byte values, unit scale: the codes the reference's unpack gives for the same words."""

    ops = _ops()
    kat = np.load(GOLDEN / "quantize_int8_kat.npz")
    words = torch.from_numpy(kat["all_words"])
    scales = torch.ones((1, 1), dtype=torch.bfloat16)
    got = ops.dequantize_i8(words.to(cuda), scales.to(cuda), 256).cpu()
    assert got.float().reshape(-1).tolist() == kat["all_codes"].astype(np.float32).reshape(-1).tolist()


@pytest.mark.parametrize("K,N,group", [(896, 1152, 64), (896, 4864, 64), (4864, 896, 64), (4096, 6144, 64),
                                       (128, 16, 64), (64, 24, 16), (96, 17, 32)])
def test_qgemv_i8_plain(cuda, K, N, group):
    ops = _ops()
    packed, scales = packed_weight_i8(K + N, N, K, group)
    x = activations(7, 1, K)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, weight_bits=8).cpu()
    assert got.shape == (1, N)
    assert ops.qmatmul_variant(1, N, K, group, weight_bits=8) == "qgemv_i8"
    assert rel_max_error(got, ref.packed_matmul(x, packed, scales, group, weight_bits=8)) < ORACLE_TOL
    assert rel_max_error(got, exact_i8(x, packed, scales, group)) < EXACT_TOL


def test_qgemv_i8_extreme_codes(cuda):
    """Alternating +127 / -127 codes: every group on the edge of its range."""

    ops = _ops()
    K, N = 256, 32
    signs = torch.tensor([1.0, -1.0]).repeat(K // 2)
    weight = (signs[None, :] * torch.linspace(0.5, 2.0, N)[:, None]).bfloat16()
    packed_np, scales_np = quantize_int8(weight.float().numpy(), 64)
    packed, scales = torch.from_numpy(packed_np), torch.from_numpy(scales_np).bfloat16()
    assert set(ref.unpack_codes_i8(packed).reshape(-1).tolist()) == {127, -127}
    x = activations(11, 1, K)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8).cpu()
    exact = exact_i8(x, packed, scales, 64)
    # one bf16 rounding of the result plus cancellation slack of the fp32 sum
    bound = exact.abs() * 2.0 ** -8 + 1e-5 * (x.double().abs().sum() * scales.double().max() * 127)
    assert bool(((got.double() - exact).abs() <= bound).all())


@pytest.mark.parametrize("K,N", [(896, 1152), (4096, 1024), (64, 24)])
def test_qgemv_i8_bias_and_norm(cuda, K, N):
    ops = _ops()
    group = 64 if K % 64 == 0 and K >= 128 else 16
    packed, scales = packed_weight_i8(5, N, K, group)
    x = activations(12, 1, K)
    bias = activations(13, N, std=0.5)
    norm_w = activations(14, K, std=0.1) + 1.0
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, weight_bits=8,
                      addend=bias.to(cuda), norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6).cpu()
    want = ref.packed_matmul(x, packed, scales, group, addend=bias, norm_weight=norm_w, rms_norm_eps=1e-6,
                             weight_bits=8)
    assert rel_max_error(got, want) < ORACLE_TOL


def test_qgemv_i8_residual_and_paired(cuda):
    ops = _ops()
    K, N = 896, 4864
    gate_p, gate_s = packed_weight_i8(20, N, K, 64)
    up_p, up_s = packed_weight_i8(21, N, K, 64)
    x = activations(22, 1, K)
    norm_w = activations(23, K, std=0.1) + 1.0
    got = ops.qmatmul(x.to(cuda), gate_p.to(cuda), gate_s.to(cuda), group_size=64, weight_bits=8,
                      packed2=up_p.to(cuda), scales2=up_s.to(cuda),
                      norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6).cpu()
    want = ref.packed_matmul(x, gate_p, gate_s, 64, packed2=up_p, scales2=up_s,
                             norm_weight=norm_w, rms_norm_eps=1e-6, weight_bits=8)
    assert rel_max_error(got, want) < 2 * ORACLE_TOL  # the oracle itself rounds five times
    down_p, down_s = packed_weight_i8(24, K, N, 64)
    hidden = activations(25, 1, 1, N)
    resid = activations(26, 1, 1, K)
    got = ops.qmatmul(hidden.to(cuda), down_p.to(cuda), down_s.to(cuda), group_size=64, weight_bits=8,
                      addend=resid.to(cuda)).cpu()
    want = ref.packed_matmul(hidden, down_p, down_s, 64, addend=resid, weight_bits=8)
    assert got.shape == (1, 1, K)
    assert rel_max_error(got, want) < ORACLE_TOL


@pytest.mark.parametrize("M,K,N", [(2, 896, 1152), (5, 128, 40), (16, 896, 1152), (128, 896, 896), (37, 4864, 896),
                                   (9, 16384, 64)])
def test_qmatmul_i8_rows(cuda, M, K, N):
    """Several activation rows: rows staged per CTA in groups of 8, 4 or 2, ragged last group."""

    ops = _ops()
    packed, scales = packed_weight_i8(M + K, N, K, 64)
    x = activations(31, M, K)
    bias = activations(32, N, std=0.5)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8,
                      addend=bias.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, 64, addend=bias, weight_bits=8)
    assert ops.qmatmul_variant(M, N, K, 64, weight_bits=8) == "qgemm_i8_rows"
    assert got.shape == (M, N)
    assert rel_max_error(got, want) < ORACLE_TOL
    # every row equals the single-row kernel's result for that row (same weights, same order of sums)
    row = ops.qmatmul(x[M - 1:].to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8,
                      addend=bias.to(cuda)).cpu()
    assert torch.equal(row, got[M - 1:])


def test_qmatmul_i8_rows_gate_and_residual(cuda):
    ops = _ops()
    M, K, N = 24, 896, 4864
    packed, scales = packed_weight_i8(41, N, K, 64)
    x = activations(42, M, K)
    gate = activations(43, M, N)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8, gate=gate.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, 64, gate=gate, weight_bits=8)
    assert rel_max_error(got, want) < ORACLE_TOL
    resid = activations(44, M, N)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8, addend=resid.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, 64, addend=resid, weight_bits=8)
    assert rel_max_error(got, want) < ORACLE_TOL


def test_qmatmul_i8_refuses_what_it_cannot_do(cuda):
    from aotolith_b200.errors import AotolithError

    ops = _ops()
    packed, scales = packed_weight_i8(51, 32, 128, 64)
    x = activations(52, 4, 128)
    norm_w = activations(53, 128, std=0.1) + 1.0
    with pytest.raises(AotolithError):   # the norm prologue needs a single row
        ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64, weight_bits=8,
                    norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6)
    with pytest.raises(AotolithError):   # four codes a word: K = 4 * words
        ops.qmatmul(x.to(cuda), packed[:, :16].contiguous().to(cuda), scales.to(cuda), group_size=64, weight_bits=8)


# ---------------------------------------------------------------------------
# whole decoders packed with eight bits
# ---------------------------------------------------------------------------

def _rel_err(actual, expected):
    expected = expected.float().cpu()
    return float((actual.float().cpu() - expected).abs().max() / expected.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("family", ["qwen2", "llama"])
def test_int8_decoder_matches_oracle_and_reference(cuda, family):
    """Prefill, decode steps and greedy tokens of a toy decoder compiled with quantize_bits=8."""

    import aotolith_b200 as aoto
    from oracle.interp import OracleRuntime
    from tests.golden_util import GROUP, NEW, PROMPT, eager_fixture

    model, _ = eager_fixture(family)
    data = np.load(GOLDEN / f"adapter_eager_int8_{family}.npz")
    runtime = aoto.models.compile_decoder_static_cache(
        model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP, quantize_bits=8, family=family
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
