"""The packed format: known-answer tests and equality with the reference packer's output.

The known-answer cases restate ``tests/test_quantize.py`` of the reference
(nibble order ``:66-74``, negatives ``:77-83``, scale rule ``:94-100``, zero group
``:103-107``, error bound ``:110-115``, group-size refusals ``:128-141``); the
fixture ``golden/quantize_kat.npz`` holds what the reference packer itself
produced on seeded matrices.
"""

import numpy as np
import pytest
import torch

from aotolith_b200 import quantize as Q
from aotolith_b200.models.quantized import pack_weight
from oracle import ops_ref as ref
from tests.golden_util import GOLDEN


def test_pack_shapes_and_dtypes():
    weight = np.random.default_rng(0).standard_normal((12, 128)).astype(np.float32)
    packed, scales = Q.quantize_int4(weight, 64)
    assert packed.shape == (12, 16) and packed.dtype == np.int32
    assert scales.shape == (12, 2) and scales.dtype == np.float32


def test_nibble_order_known_answer():
    # codes 1..7 and -7 (scale 1 when max|w| = 7): code k of a word sits at bit 4k
    weight = np.array([[1, 2, 3, 4, 5, 6, 7, -7]], dtype=np.float32)
    packed, scales = Q.quantize_int4(weight, 8)
    assert scales[0, 0] == pytest.approx(1.0)
    word = int(packed[0, 0]) & 0xFFFFFFFF
    assert [(word >> (4 * k)) & 0xF for k in range(8)] == [1, 2, 3, 4, 5, 6, 7, 9]
    assert Q.unpack_codes(packed).tolist() == [[1, 2, 3, 4, 5, 6, 7, -7]]
    # the most negative code is representable (8 -> -8) though never produced
    forced = np.array([[0x8 | (0xF << 4)]], dtype=np.int32)
    assert Q.unpack_codes(forced)[0, :2].tolist() == [-8, -1]


def test_scale_rule_zero_group_and_error_bound():
    rng = np.random.default_rng(1)
    weight = rng.standard_normal((7, 64)).astype(np.float32)
    weight[2, :16] = 0.0
    packed, scales = Q.quantize_int4(weight, 16)
    peaks = np.abs(weight.reshape(7, 4, 16)).max(axis=-1)
    expected = np.where(peaks > 0, peaks, 1.0) / 7
    assert np.allclose(scales, expected, rtol=1e-7)
    assert scales[2, 0] == pytest.approx(1.0 / 7)
    codes = Q.unpack_codes(packed)
    assert not codes[2, :16].any()
    assert codes.min() >= -7 and codes.max() <= 7
    restored = Q.dequantize_int4(packed, scales, 16)
    assert np.all(np.abs(restored - weight) <= np.repeat(scales, 16, axis=-1) / 2 + 1e-7)


def test_exact_code_round_trip():
    rng = np.random.default_rng(2)
    codes = rng.integers(-7, 8, size=(9, 32)).astype(np.float32)
    codes[:, 0] = 7.0  # pins the scale of every 32-wide group to exactly 1
    packed, scales = Q.quantize_int4(codes, 32)
    assert np.array_equal(Q.unpack_codes(packed), codes.astype(np.int8))
    assert np.allclose(scales, 1.0)


@pytest.mark.parametrize("group,inner", [(0, 64), (-8, 64), (12, 48), (48, 64)])
def test_group_size_refusals(group, inner):
    with pytest.raises(ValueError):
        Q.check_group_size(group, inner)
    with pytest.raises(ValueError):
        Q.quantize_int4(np.zeros((2, inner), dtype=np.float32), group)


def test_int8_layout():
    weight = np.array([[127, -127, 1, -1]], dtype=np.float32)
    packed, scales = Q.quantize_int8(weight, 4)
    word = int(packed[0, 0]) & 0xFFFFFFFF
    assert [(word >> (8 * k)) & 0xFF for k in range(4)] == [127, 129, 1, 255]
    assert Q.unpack_codes_int8(packed).tolist() == [[127, -127, 1, -1]]
    assert np.allclose(Q.dequantize_int8(packed, scales, 4), weight)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_matches_reference_packer_output(tag):
    kat = np.load(GOLDEN / "quantize_kat.npz")
    group = int(kat[f"{tag}_group"])
    packed, scales = Q.quantize_int4(kat[f"{tag}_weight"], group)
    assert np.array_equal(packed, kat[f"{tag}_packed"])
    assert np.array_equal(scales, kat[f"{tag}_scales"])
    assert np.array_equal(Q.unpack_codes(packed), kat[f"{tag}_codes"])
    assert np.array_equal(Q.dequantize_int4(packed, scales, group), kat[f"{tag}_dequant"])
    # the oracle's torch unpack agrees with the NumPy one
    assert np.array_equal(ref.unpack_codes(torch.from_numpy(packed)).numpy(), kat[f"{tag}_codes"])


def test_pack_weight_keeps_the_weight_dtype():
    weight = torch.randn(8, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    packed, scales = pack_weight(weight, 16)
    assert packed.dtype == torch.int32 and packed.shape == (8, 8)
    assert scales.dtype == torch.bfloat16 and scales.shape == (8, 4)
    want = ref.dequantize_i4(packed, scales, 16)
    assert want.dtype == torch.bfloat16
    # bf16(code) * bf16(scale), one rounding: compare with an explicit fp32 product
    codes = ref.unpack_codes(packed).float()
    explicit = (codes * scales.float().repeat_interleave(16, dim=-1)).bfloat16()
    assert torch.equal(want, explicit)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_int8_matches_reference_packer_output(tag):
    """Eight-bit packer, unpack and dequantise against the reference's own outputs."""

    kat = np.load(GOLDEN / "quantize_int8_kat.npz")
    group = int(kat[f"{tag}_group"])
    packed, scales = Q.quantize_int8(kat[f"{tag}_weight"], group)
    assert np.array_equal(packed, kat[f"{tag}_packed"])
    assert np.array_equal(scales, kat[f"{tag}_scales"])
    assert np.array_equal(Q.unpack_codes_int8(packed), kat[f"{tag}_codes"])
    assert np.array_equal(Q.dequantize_int8(packed, scales, group), kat[f"{tag}_dequant"])
    # the oracle's torch unpack and its bf16 dequantise agree with the reference's torch operator
    assert np.array_equal(ref.unpack_codes_i8(torch.from_numpy(packed)).numpy(), kat[f"{tag}_codes"])
    low = ref.dequantize_i8(torch.from_numpy(packed), torch.from_numpy(scales).bfloat16(), group)
    assert low.dtype == torch.bfloat16
    assert np.array_equal(low.float().numpy(), kat[f"{tag}_dequant_bf16"])


def test_int8_unpack_of_every_byte_value():
    kat = np.load(GOLDEN / "quantize_int8_kat.npz")
    assert np.array_equal(Q.unpack_codes_int8(kat["all_words"]), kat["all_codes"])
    assert np.array_equal(ref.unpack_codes_i8(torch.from_numpy(kat["all_words"])).numpy(), kat["all_codes"])
    assert kat["all_codes"].reshape(-1).tolist() == [b if b < 128 else b - 256 for b in range(256)]


def test_oracle_int8_packed_matmul_is_dequantise_then_matmul():
    rng = np.random.default_rng(4)
    weight = (rng.standard_normal((12, 64)) * 0.05).astype(np.float32)
    packed_np, scales_np = Q.quantize_int8(weight, 16)
    packed, scales = torch.from_numpy(packed_np), torch.from_numpy(scales_np).bfloat16()
    x = torch.from_numpy(rng.standard_normal((3, 64)).astype(np.float32)).bfloat16()
    bias = torch.from_numpy(rng.standard_normal(12).astype(np.float32)).bfloat16()
    got = ref.packed_matmul(x, packed, scales, 16, addend=bias, weight_bits=8)
    dense = ref.dequantize_i8(packed, scales, 16)
    want = 1.0 * bias + 1.0 * (x.float() @ dense.float().T).bfloat16()
    assert got.dtype == torch.bfloat16 and torch.equal(got, want)
    # eight bits are far closer to the weight than four (tests/test_quantize.py:205-214 of the reference)
    four = Q.dequantize_int4(*Q.quantize_int4(weight, 16), 16)
    eight = Q.dequantize_int8(packed_np, scales_np, 16)
    assert np.abs(eight - weight).max() < np.abs(four - weight).max() / 8


def test_torch_packer_is_bit_identical_to_the_numpy_packer():
    """``quantize_torch`` (used when a model lives on the device) against ``quantize_int4/int8``."""

    import torch

    from aotolith_b200.quantize import quantize_int4, quantize_int8, quantize_torch

    rng = np.random.default_rng(11)
    for rows, inner, group in ((7, 128, 64), (5, 96, 32), (3, 64, 16)):
        weight = (rng.standard_normal((rows, inner)) * 0.05).astype(np.float32)
        weight[0, :group] = 0.0                                   # an all-zero group
        weight[1, :] = np.where(np.arange(inner) % 2 == 0, 1.0, -1.0) * 0.75
        weight[2, 3] = weight[2, :group].max() * 0.5              # a value exactly half way between codes
        for bits, reference in ((4, quantize_int4), (8, quantize_int8)):
            want_words, want_scales = reference(weight, group)
            words, scales = quantize_torch(torch.from_numpy(weight), group, bits)
            assert np.array_equal(words.numpy(), want_words)
            assert np.array_equal(scales.numpy().view(np.int32), want_scales.view(np.int32))
    bf16 = torch.from_numpy((rng.standard_normal((6, 256)) * 0.02).astype(np.float32)).bfloat16()
    words, scales = quantize_torch(bf16, 64, 4)
    want_words, want_scales = quantize_int4(bf16.float().numpy(), 64)
    assert np.array_equal(words.numpy(), want_words) and np.array_equal(scales.numpy(), want_scales)
