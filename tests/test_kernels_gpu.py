"""Parity of every sm_100a kernel with the CPU oracle, through the C ABI.

Tolerances: integer/byte/index work is bit-exact (dequantisation, cache roll,
gathers, masks, argmax, rotary embedding - whose bf16 rounding points are
reproduced). Floating-point reductions are compared with the oracle at
``1e-2 * max|expected|`` (the logit tolerance of the target) and with an
unrounded float64 evaluation at ``4e-3 * max|exact|`` (one bf16 rounding of the
result is 2^-9 relative).
"""

import math

import pytest
import torch

from oracle import ops_ref as ref
from tests.helpers import activations, exact_packed_matmul, packed_weight, rel_max_error

pytestmark = pytest.mark.gpu

ORACLE_TOL = 1e-2
EXACT_TOL = 4e-3

QWEN_SHAPES = [(896, 1152), (896, 896), (896, 4864), (4864, 896)]


def _ops():
    import aotolith_b200.ops as ops

    return ops


@pytest.mark.parametrize("K,N,group", [(896, 1152, 64), (128, 48, 64), (64, 24, 16), (4096, 512, 64), (96, 40, 32)])
def test_dequantize_bit_exact(cuda, K, N, group):
    ops = _ops()
    packed, scales = packed_weight(1, N, K, group)
    got = ops.dequantize_i4(packed.to(cuda), scales.to(cuda), group).cpu()
    want = ref.dequantize_i4(packed, scales, group)
    assert got.dtype == torch.bfloat16 and got.shape == (N, K)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("K,N", QWEN_SHAPES + [(4096, 6144), (14336, 4096), (128, 16), (256, 40), (384, 17)])
def test_qgemv_plain(cuda, K, N):
    ops = _ops()
    packed, scales = packed_weight(K + N, N, K, 64)
    x = activations(7, 1, K)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64).cpu()
    assert got.shape == (1, N)
    assert ops.qmatmul_variant(1, N, K, 64) == ("qgemv_stream" if N >= 65536 else "qgemv_mma")
    assert rel_max_error(got, ref.packed_matmul(x, packed, scales, 64)) < ORACLE_TOL
    assert rel_max_error(got, exact_packed_matmul(x, packed, scales, 64)) < EXACT_TOL


def test_qgemv_lm_head_shape(cuda):
    ops = _ops()
    K, N = 896, 151936
    packed, scales = packed_weight(3, N, K, 64)
    x = activations(8, 1, K)
    norm_w = (activations(9, K, std=0.1) + 1.0)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64,
                      norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6).cpu()
    want = ref.packed_matmul(x, packed, scales, 64, norm_weight=norm_w, rms_norm_eps=1e-6)
    assert rel_max_error(got, want) < ORACLE_TOL
    assert int(got.float().argmax()) == int(want.float().argmax())
    assert ops.qmatmul_variant(1, N, K, 64) == "qgemv_stream"


def test_qgemv_extreme_codes(cuda):
    """Alternating +7 / -7 codes: every group on the edge of its range.

    Mirrors the reference's extreme-code GEMV case (tests/test_quantized_matmul.py:75-113).
    """

    ops = _ops()
    K, N = 256, 32
    signs = torch.tensor([1.0, -1.0]).repeat(K // 2)
    weight = (signs[None, :] * torch.linspace(0.5, 2.0, N)[:, None]).bfloat16()
    from aotolith_b200.quantize import quantize_int4, unpack_codes

    packed_np, scales_np = quantize_int4(weight.float().numpy(), 64)
    assert set(unpack_codes(packed_np).reshape(-1).tolist()) == {7, -7}
    packed, scales = torch.from_numpy(packed_np), torch.from_numpy(scales_np).bfloat16()
    x = activations(11, 1, K)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=64).cpu()
    exact = exact_packed_matmul(x, packed, scales, 64)
    # one bf16 rounding of the result: 2^-8 relative per element plus cancellation slack
    bound = exact.abs() * 2.0 ** -8 + 1e-5 * (x.double().abs().sum() * scales.double().max() * 7)
    assert bool(((got.double() - exact).abs() <= bound).all())


@pytest.mark.parametrize("K,N", [(896, 1152), (4096, 6144), (64, 24)])
def test_qgemv_bias_and_norm(cuda, K, N):
    """The packed q/k/v projection: fused RMS-norm prologue and bias epilogue."""

    ops = _ops()
    group = 64 if K % 64 == 0 and K >= 128 else 16
    packed, scales = packed_weight(5, N, K, group)
    x = activations(12, 1, K)
    bias = activations(13, N, std=0.5)
    norm_w = activations(14, K, std=0.1) + 1.0
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group,
                      addend=bias.to(cuda), norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6).cpu()
    want = ref.packed_matmul(x, packed, scales, group, addend=bias, norm_weight=norm_w, rms_norm_eps=1e-6)
    assert rel_max_error(got, want) < ORACLE_TOL


@pytest.mark.parametrize("K,N", [(4864, 896), (896, 896), (14336, 4096), (48, 32)])
def test_qgemv_residual(cuda, K, N):
    ops = _ops()
    group = 64 if K % 128 == 0 else 16
    packed, scales = packed_weight(6, N, K, group)
    x = activations(15, 1, 1, K)
    resid = activations(16, 1, 1, N)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, addend=resid.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, group, addend=resid)
    assert got.shape == (1, 1, N)
    assert rel_max_error(got, want) < ORACLE_TOL


@pytest.mark.parametrize("K,N", [(896, 4864), (4096, 14336), (32, 64)])
def test_qgemv_paired_silu_mul(cuda, K, N):
    """gate/up pair with the SiLU-mul epilogue, norm folded in."""

    ops = _ops()
    group = 64 if K % 128 == 0 else 16
    gate_p, gate_s = packed_weight(20, N, K, group)
    up_p, up_s = packed_weight(21, N, K, group)
    x = activations(22, 1, K)
    norm_w = activations(23, K, std=0.1) + 1.0
    got = ops.qmatmul(x.to(cuda), gate_p.to(cuda), gate_s.to(cuda), group_size=group,
                      packed2=up_p.to(cuda), scales2=up_s.to(cuda),
                      norm_weight=norm_w.to(cuda), rms_norm_eps=1e-6).cpu()
    want = ref.packed_matmul(x, gate_p, gate_s, group, packed2=up_p, scales2=up_s,
                             norm_weight=norm_w, rms_norm_eps=1e-6)
    left = ref.matmul_norm_prologue(x, norm_w, 1e-6)
    g = exact_packed_matmul(left, gate_p, gate_s, group)
    u = exact_packed_matmul(left, up_p, up_s, group)
    exact = u * (g / (1 + torch.exp(-g)))
    assert rel_max_error(got, want) < 2 * ORACLE_TOL  # the oracle itself rounds five times
    assert rel_max_error(got, exact) < ORACLE_TOL


@pytest.mark.parametrize("M,K,N", [(2, 896, 1152), (16, 896, 1152), (128, 896, 1152), (200, 4864, 896),
                                   (37, 896, 4864), (130, 256, 1000), (5, 64, 24),
                                   (64, 896, 896), (256, 4864, 896), (128, 64, 72),
                                   # few rows: the kernel that shares K among the warps of a CTA
                                   (8, 896, 4864), (3, 4864, 896), (9, 4864, 896), (16, 128, 40), (7, 896, 18950),
                                   (4, 4096, 6144), (8, 14336, 4096), (12, 4864, 64), (24, 896, 1152)])
def test_qmatmul_rows(cuda, M, K, N):
    """Several activation rows (prefill semantics: dequantise, then multiply)."""

    ops = _ops()
    group = 64 if K % 128 == 0 else 16
    packed, scales = packed_weight(30, N, K, group)
    x = activations(31, M, K)
    bias = activations(32, N, std=0.5)
    if K % 128 == 0:
        staged = (8 if M <= 8 else 16) * (2 * K + 64) + 8 * (1 if M <= 8 else 2) * 4 * 32 * 4
        few = 2 <= M <= 16 and N >= 16 and staged <= 200 * 1024
        assert ops.qmatmul_variant(M, N, K, group) == (
            "qgemm_rows" if few else
            "gemm_tcgen05" if M >= 64 or (M >= 8 and (N >= 4096 or K >= 2048)) else "gemm_mma")
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, addend=bias.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, group, addend=bias)
    assert got.shape == (M, N)
    assert rel_max_error(got, want) < ORACLE_TOL
    assert rel_max_error(got, exact_packed_matmul(x, packed, scales, group) + bias.double()) < EXACT_TOL
    gate = activations(33, M, N)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, gate=gate.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, group, gate=gate)
    assert rel_max_error(got, want) < ORACLE_TOL
    resid = activations(34, M, N)
    got = ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=group, addend=resid.to(cuda)).cpu()
    want = ref.packed_matmul(x, packed, scales, group, addend=resid)
    assert rel_max_error(got, want) < ORACLE_TOL
    from aotolith_b200 import _native
    assert _native.load().aoto_sm100_qmatmul_take_timeout_flag() == 0


def test_qmatmul_rows_match_single_rows(cuda):
    """Every row of the multi-row product agrees with the decode kernel run on that row alone."""

    ops = _ops()
    M, K, N = 19, 896, 896
    packed, scales = packed_weight(35, N, K, 64)
    x = activations(36, M, K).to(cuda)
    packed, scales = packed.to(cuda), scales.to(cuda)
    together = ops.qmatmul(x, packed, scales, group_size=64).float()
    alone = torch.cat([ops.qmatmul(x[i:i + 1], packed, scales, group_size=64) for i in range(M)]).float()
    # the two kernels round the weight at different points (code*scale before / scale after the sum)
    assert float((together - alone).abs().max()) <= ORACLE_TOL * float(alone.abs().max())


def test_qgemv_deterministic(cuda):
    ops = _ops()
    packed, scales = packed_weight(40, 896, 4864, 64)
    x = activations(41, 1, 4864).to(cuda)
    packed, scales = packed.to(cuda), scales.to(cuda)
    first = ops.qmatmul(x, packed, scales, group_size=64)
    for _ in range(3):
        assert torch.equal(first, ops.qmatmul(x, packed, scales, group_size=64))


def test_qmatmul_refuses_bad_requests(cuda):
    from aotolith_b200.errors import DeviceError, PlanInputError

    ops = _ops()
    packed, scales = packed_weight(42, 16, 128, 64)
    x = activations(43, 1, 128)
    with pytest.raises(DeviceError):
        ops.qmatmul(x, packed, scales, group_size=64)  # CPU tensors: no CPU path
    with pytest.raises(PlanInputError):
        ops.qmatmul(x.to(cuda)[:, :64], packed.to(cuda), scales.to(cuda), group_size=64)
    with pytest.raises(DeviceError):
        ops.qmatmul(x.to(cuda), packed.to(cuda), scales.to(cuda), group_size=48)  # 48 does not divide 128


@pytest.mark.parametrize("rows,H", [(1, 896), (128, 896), (3, 4096), (5, 32)])
def test_rms_norm(cuda, rows, H):
    ops = _ops()
    x = activations(50, rows, H)
    w = activations(51, H, std=0.1) + 1.0
    got = ops.rms_norm(x.to(cuda), w.to(cuda), 1e-6).cpu()
    want = ref.rms_norm(x, w, 1e-6)
    # one rounding on both sides; statistics differ only in summation order
    assert rel_max_error(got, want) < 2.0 ** -7
    resid = activations(52, rows, H)
    got, total = ops.rms_norm(x.to(cuda), w.to(cuda), 1e-6, residual=resid.to(cuda), return_sum=True)
    assert torch.equal(total.cpu(), x + resid)
    assert rel_max_error(got.cpu(), ref.rms_norm(x + resid, w, 1e-6)) < 2.0 ** -7


@pytest.mark.parametrize("heads,T,D", [(14, 128, 64), (2, 1, 64), (32, 5, 128), (4, 3, 8)])
def test_rope_bit_exact(cuda, heads, T, D):
    ops = _ops()
    # strided operand: a transposed slice of a projection row, as the prefill graph has it
    row = activations(60, 1, T, heads * D + 16)
    x = row[:, :, 8 : 8 + heads * D].reshape(1, T, heads, D).transpose(1, 2)
    cos = activations(61, 1, 1, T, D, std=0.7)
    sin = activations(62, 1, 1, T, D, std=0.7)
    got = ops.rope(row.to(cuda)[:, :, 8 : 8 + heads * D].reshape(1, T, heads, D).transpose(1, 2),
                   cos.to(cuda), sin.to(cuda)).cpu()
    want = ref.rope(x, cos, sin)
    assert torch.equal(got.view(torch.int16), want.contiguous().view(torch.int16))


def test_embedding_and_bounds(cuda):
    ops = _ops()
    table = activations(70, 1000, 896)
    ids = torch.tensor([[0, 999, 17, 512]], dtype=torch.int64)
    got = ops.embedding(table.to(cuda), ids.to(cuda)).cpu()
    assert torch.equal(got, ref.embedding(table, ids))
    flag = torch.zeros(1, dtype=torch.int64, device=cuda)
    bad = torch.tensor([[3, 1000, -1]], dtype=torch.int64)
    got = ops.embedding(table.to(cuda), bad.to(cuda), bad_index=flag).cpu()
    assert int(flag.item()) == 2  # 1 + position of the first offending id
    assert torch.equal(got[0, 0], table[3]) and not got[0, 1].any() and not got[0, 2].any()
    narrow = activations(71, 16, 6)  # width not a multiple of 8: scalar path
    ids = torch.tensor([5, 0, 15], dtype=torch.int64)
    assert torch.equal(ops.embedding(narrow.to(cuda), ids.to(cuda)).cpu(), narrow[ids])


def test_mask_select(cuda):
    ops = _ops()
    mask = torch.arange(192) >= 192 - 129
    got = ops.mask_select(mask.reshape(1, 1, 1, 192).to(cuda), 0.0, float("-inf")).cpu()
    want = ref.mask_to_additive(mask.reshape(1, 1, 1, 192), torch.bfloat16)
    assert torch.equal(got, want)


def test_argmax_first_maximum(cuda):
    ops = _ops()
    logits = activations(80, 1, 151936)
    logits[0, 4000] = logits[0, 90000] = 50.0  # a tie: the first index wins
    got = ops.argmax(logits.to(cuda)).cpu()
    assert got.tolist() == [4000]
    many = activations(81, 5, 1000)
    assert torch.equal(ops.argmax(many.to(cuda)).cpu(), many.float().argmax(dim=-1))


@pytest.mark.parametrize("L,KVH,QH,C,D", [(24, 2, 14, 192, 64), (3, 8, 32, 40, 128), (2, 2, 4, 12, 8)])
def test_rope_kv_cache_append_exact(cuda, L, KVH, QH, C, D):
    ops = _ops()
    cache = activations(90, L, 2, 1, KVH, C, D)
    row = activations(91, 1, 1, (QH + 2 * KVH) * D)
    cos = activations(92, 1, 1, 1, D, std=0.7)
    sin = activations(93, 1, 1, 1, D, std=0.7)
    layer = L - 1
    attrs = dict(layer=layer, query_start=0, key_start=QH * D, value_start=(QH + KVH) * D, query_heads=QH)
    q, pair, keys, values = ops.rope_kv_cache_append(cache.to(cuda), row.to(cuda), cos.to(cuda), sin.to(cuda), **attrs)
    rq, rpair, rkeys, rvalues = ref.rope_kv_cache_append(cache, row, cos, sin, **attrs)
    assert torch.equal(q.cpu(), rq) and torch.equal(pair.cpu(), rpair)
    assert torch.equal(keys.cpu(), rkeys) and torch.equal(values.cpu(), rvalues)
    # the un-rotated form
    npair, nk, nv = ops.kv_cache_append(cache.to(cuda), rq[:, :KVH].contiguous().to(cuda), row.to(cuda),
                                        layer=0, value_start=(QH + KVH) * D)
    wpair, _, _ = ref.kv_cache_append(cache, rq[:, :KVH], row, layer=0, value_start=(QH + KVH) * D)
    assert torch.equal(npair.cpu(), wpair)


def test_cache_roll_invariants(cuda):
    """The window shifts by exactly one slot and the source cache is untouched."""

    ops = _ops()
    L, KVH, QH, C, D = 2, 2, 4, 16, 64
    cache = activations(95, L, 2, 1, KVH, C, D).to(cuda)
    before = cache.clone()
    row = activations(96, 1, 1, (QH + 2 * KVH) * D).to(cuda)
    cos = torch.ones(1, 1, 1, D, dtype=torch.bfloat16, device=cuda)
    sin = torch.zeros(1, 1, 1, D, dtype=torch.bfloat16, device=cuda)
    _, pair, _, _ = ops.rope_kv_cache_append(cache, row, cos, sin, layer=1, query_start=0,
                                             key_start=QH * D, value_start=(QH + KVH) * D, query_heads=QH)
    assert torch.equal(cache, before)
    assert torch.equal(pair[:, :, :, :-1], cache[1][:, :, :, 1:])
    assert torch.equal(pair[0, 0, :, -1].reshape(-1), row[0, 0, QH * D : (QH + KVH) * D])
    assert torch.equal(pair[1, 0, :, -1].reshape(-1), row[0, 0, (QH + KVH) * D :])


@pytest.mark.parametrize("QH,KVH,C,D,valid", [(14, 2, 192, 64, 129), (32, 8, 1280, 128, 1025),
                                               (4, 2, 12, 8, 5), (14, 2, 192, 64, 192), (8, 8, 2100, 64, 2100),
                                               (4, 2, 8200, 64, 8000)])  # the last: more splits than the staged merge holds
def test_attention_decode(cuda, QH, KVH, C, D, valid):
    ops = _ops()
    q = activations(100, 1, QH, 1, D)
    k = activations(101, 1, KVH, C, D)
    v = activations(102, 1, KVH, C, D)
    mask = ref.mask_to_additive((torch.arange(C) >= C - valid).reshape(1, 1, 1, C), torch.bfloat16)
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5).cpu()
    want = ref.attention(q, k, v, mask, scale=D ** -0.5)
    assert rel_max_error(got, want) < ORACLE_TOL
    got2 = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5).cpu()
    assert torch.equal(got, got2)


def test_attention_fully_masked_rows_are_zero(cuda):
    ops = _ops()
    QH, KVH, C, D = 4, 2, 40, 64
    q = activations(110, 1, QH, 1, D)
    k = activations(111, 1, KVH, C, D)
    v = activations(112, 1, KVH, C, D)
    mask = torch.full((1, 1, 1, C), float("-inf"), dtype=torch.bfloat16)
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5).cpu()
    assert not got.any()


@pytest.mark.parametrize("QH,KVH,C,D", [(14, 2, 192, 64), (4, 2, 40, 16), (8, 8, 1, 64)])
def test_attention_single_query_causal_sees_key_zero_only(cuda, QH, KVH, C, D):
    """Top-left aligned causal rule with one query row: only key 0 is admitted (the oracle's
    and the reference's ``_causal_mask``); the split-KV decode kernel must not serve this case."""

    ops = _ops()
    q = activations(140, 1, QH, 1, D)
    k = activations(141, 1, KVH, C, D)
    v = activations(142, 1, KVH, C, D)
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), None, scale=D ** -0.5, causal=True).cpu()
    want = ref.attention(q, k, v, None, scale=D ** -0.5, causal=True)
    assert rel_max_error(got, want) < ORACLE_TOL
    # with one admitted key the result is that key's value row, head by head
    group = QH // KVH
    for head in range(QH):
        assert torch.equal(got[0, head, 0], v[0, head // group, 0])


@pytest.mark.parametrize("QH,KVH,P,D,length", [(14, 2, 128, 64, 128), (14, 2, 64, 64, 37), (32, 8, 96, 128, 96), (4, 2, 7, 8, 3),
                                                  (8, 2, 200, 64, 131), (8, 4, 257, 128, 257), (2, 1, 16, 64, 16),
                                                  (8, 2, 512, 64, 300), (8, 2, 1024, 128, 1024), (4, 4, 384, 128, 65)])
def test_attention_prefill(cuda, QH, KVH, P, D, length):
    """Prefill with the left-padded bucket mask; pad query rows are fully masked -> zero."""

    ops = _ops()
    q = activations(120, 1, QH, P, D)
    k = activations(121, 1, KVH, P, D)
    v = activations(122, 1, KVH, P, D)
    query = torch.arange(P)[:, None]
    key = torch.arange(P)[None, :]
    allowed = (key <= query) & (key >= P - length)
    mask = ref.mask_to_additive(allowed.reshape(1, 1, P, P), torch.bfloat16)
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5).cpu()
    want = ref.attention(q, k, v, mask, scale=D ** -0.5)
    assert rel_max_error(got, want) < ORACLE_TOL
    if length < P:
        assert not got[:, :, : P - length].any()
    if length == P:
        causal = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), None, scale=D ** -0.5, causal=True).cpu()
        assert rel_max_error(causal, want) < ORACLE_TOL


@pytest.mark.parametrize("P,D,band", [(512, 64, 100), (320, 128, 1), (448, 64, 447)])
def test_attention_prefill_skips_only_tiles_without_admitted_keys(cuda, P, D, band):
    """A banded mask leaves whole key tiles without an admitted key before and after the band; the
    kernel passes over them, and over nothing else. Some query rows admit no key at all."""

    ops = _ops()
    QH, KVH = 4, 2
    q = activations(130, 1, QH, P, D)
    k = activations(131, 1, KVH, P, D)
    v = activations(132, 1, KVH, P, D)
    query = torch.arange(P)[:, None]
    key = torch.arange(P)[None, :]
    allowed = (key <= query) & (key > query - band) & ((query < 70) | (query >= 140))
    allowed[P - 1, 3] = True                      # a lone admitted key in a tile the band never reaches
    mask = ref.mask_to_additive(allowed.reshape(1, 1, P, P), torch.bfloat16)
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5).cpu()
    want = ref.attention(q, k, v, mask, scale=D ** -0.5)
    assert rel_max_error(got, want) < ORACLE_TOL
    assert not got[:, :, 70:140].any()
    # the workspace for the tile classes is optional: without it every tile is visited, same result
    plain = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), mask.to(cuda), scale=D ** -0.5, optional_workspace=False).cpu()
    assert torch.equal(plain, got)


def test_scratch_is_shared_between_kernels_and_shapes(cuda):
    """Attention splits of different shapes and wide argmax reuse one per-stream scratch buffer."""

    ops = _ops()
    logits = activations(130, 1, 151936)
    for C in (1280, 192, 700):
        q = activations(131, 1, 14, 1, 64)
        k = activations(132, 1, 2, C, 64)
        v = activations(133, 1, 2, C, 64)
        want = ref.attention(q, k, v, None, scale=0.125)
        got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), None, scale=0.125).cpu()
        assert rel_max_error(got, want) < ORACLE_TOL
        assert ops.argmax(logits.to(cuda)).cpu().tolist() == [int(logits.float().argmax())]


def test_greedy_pick_and_step_inputs(cuda):
    ops = _ops()
    counters = torch.tensor([130, 0], dtype=torch.int32, device=cuda)
    position = torch.zeros((1, 1), dtype=torch.int64, device=cuda)
    mask = torch.zeros((1, 1, 1, 192), dtype=torch.bool, device=cuda)
    token = torch.zeros((1, 1), dtype=torch.int64, device=cuda)
    generated = torch.full((8,), -1, dtype=torch.int64, device=cuda)
    picks = []
    for step in range(3):
        ops.step_inputs(counters, position, mask)
        assert int(position.item()) == 129 + step
        assert mask.reshape(-1).cpu().tolist() == [False] * (192 - 130 - step) + [True] * (130 + step)
        logits = activations(140 + step, 151936)
        picks.append(int(logits.float().argmax()))
        ops.greedy_pick(logits.to(cuda), token, generated, counters)
        assert int(token.item()) == picks[-1]
    assert generated.cpu().tolist()[:3] == picks and int(generated[3]) == -1
    assert counters.cpu().tolist() == [133, 3]
