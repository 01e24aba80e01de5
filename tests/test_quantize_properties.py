"""Properties of the packed weight format over random shapes, group sizes and values.

The known answers of the reference's packer are pinned in tests/test_quantize.py; here the
rules it states (``src/aotolith/quantize.py:1-60, 95-200``) are checked as properties: codes stay
inside the symmetric range, the scale is the group magnitude over 7 (127), an all-zero group
is scaled as if its magnitude were one and gets zero codes, packing is a bijection on codes, the reconstruction error is at
most half a step per weight, and the oracle's torch unpack agrees with the NumPy one.
"""

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from aotolith_b200 import quantize as Q
from oracle import ops_ref as ref

BITS = {4: (Q.quantize_int4, Q.unpack_codes, Q.dequantize_int4, ref.unpack_codes, 7, 8),
        8: (Q.quantize_int8, Q.unpack_codes_int8, Q.dequantize_int8, ref.unpack_codes_i8, 127, 4)}


@st.composite
def weights(draw):
    bits = draw(st.sampled_from([4, 8]))
    per_word = BITS[bits][5]
    group = per_word * draw(st.integers(1, 8))
    groups = draw(st.integers(1, 4))
    rows = draw(st.integers(1, 6))
    seed = draw(st.integers(0, 2**31 - 1))
    scale = draw(st.sampled_from([1e-3, 0.05, 1.0, 300.0]))
    rng = np.random.default_rng(seed)
    weight = (rng.standard_normal((rows, group * groups)) * scale).astype(np.float32)
    if draw(st.booleans()):
        weight[0, :group] = 0.0                                   # an all-zero group
    return bits, group, weight


@settings(max_examples=60, deadline=None)
@given(weights())
def test_format_rules_hold(case):
    bits, group, weight = case
    quantize, unpack, dequantize, torch_unpack, magnitude, per_word = BITS[bits]
    packed, scales = quantize(weight, group)
    rows, inner = weight.shape
    assert packed.dtype == np.int32 and packed.shape == (rows, inner // per_word)
    assert scales.dtype == np.float32 and scales.shape == (rows, inner // group)
    codes = unpack(packed)
    assert codes.dtype == np.int8 and codes.shape == weight.shape
    assert codes.min() >= -magnitude and codes.max() <= magnitude             # symmetric: the most negative code is unused
    grouped = np.abs(weight).reshape(rows, inner // group, group).max(axis=-1)
    expected_scale = (np.where(grouped > 0, grouped, 1.0) / magnitude).astype(np.float32)
    assert np.allclose(scales, expected_scale, rtol=1e-6, atol=0)
    zero_groups = grouped == 0
    assert not codes.reshape(rows, inner // group, group)[zero_groups].any()
    # reconstruction: at most half a step away from every weight
    restored = dequantize(packed, scales, group)
    step = np.repeat(scales, group, axis=-1)
    assert np.all(np.abs(restored - weight) <= 0.5 * step * (1 + 1e-5) + 1e-12)
    # the largest weight of every group lands on the edge of the range
    edge = np.abs(codes).reshape(rows, inner // group, group).max(axis=-1)
    assert np.all(edge[~zero_groups] == magnitude)
    # the oracle's torch unpack is the same function
    assert np.array_equal(torch_unpack(torch.from_numpy(packed)).numpy(), codes)


@settings(max_examples=40, deadline=None)
@given(st.sampled_from([4, 8]), st.integers(1, 5), st.integers(1, 6), st.integers(0, 2**31 - 1))
def test_packing_is_a_bijection_on_codes(bits, rows, words, seed):
    quantize, unpack, _, _, magnitude, per_word = BITS[bits]
    rng = np.random.default_rng(seed)
    codes = rng.integers(-magnitude, magnitude + 1, size=(rows, words * per_word)).astype(np.float32)
    codes[:, 0] = magnitude                                       # pins every row's scale to exactly one
    packed, scales = quantize(codes, words * per_word)
    assert np.allclose(scales, 1.0)
    assert np.array_equal(unpack(packed), codes.astype(np.int8))
    # word j holds codes j*per_word .. (j+1)*per_word - 1, code k at bit k*bits, two's complement
    word = int(packed[0, 0]) & 0xFFFFFFFF
    fields = [(word >> (bits * k)) & ((1 << bits) - 1) for k in range(per_word)]
    signed = [f - (1 << bits) if f >= (1 << (bits - 1)) else f for f in fields]
    assert signed == codes[0, :per_word].astype(int).tolist()
