"""The normalisation folds: the scale into the norm, the norm into the packed projection.

After the reference's tests/test_passes_norm.py. PyTorch writes RMSNorm as an fp32 upcast, the
normalisation, a scaled multiply and a narrowing cast; ``fuse_norm_scale`` turns that chain into
one weighted ``rms_norm`` and must not move a bit; ``fuse_rms_norm_epilogue`` then moves the norm
into the single-row packed projections that read it, and must back off when the row has another
reader or the product has several rows. The numbers are the oracle's over the graphs.
"""

import numpy as np
import torch

from aotolith_b200.capture import capture_fx
from aotolith_b200.models.quantized import dequantize_i4
from aotolith_b200.passes import rewrite
from aotolith_b200.passes.fusion import fuse_norm_scale
from aotolith_b200.quantize import quantize_int4
from oracle.interp import run_graph

EPS = 1e-6
GROUP = 32


def _rms_norm_scale(value, weight):
    """The spelling Qwen and Llama use."""

    upcast = value.to(torch.float32)
    variance = upcast.pow(2).mean(-1, keepdim=True)
    normalized = upcast * torch.rsqrt(variance + EPS)
    return (weight * normalized).to(value.dtype)


def _counts(graph):
    counts = {}
    for op in graph.ops:
        counts[op.op] = counts.get(op.op, 0) + 1
    return counts


def _case(hidden, *, seed=0, rows=(1, 1)):
    generator = torch.Generator().manual_seed(seed)
    value = torch.randn(*rows, hidden, generator=generator).bfloat16()
    weight = torch.randn(hidden, generator=generator).bfloat16()
    return value, weight


def test_the_captured_normalization_is_a_chain_of_casts_norm_and_scale():
    # the premise of the pass: casts around the row (and, depending on how the frontend spells the
    # promotion, on the weight), the normalisation, and the scale multiply
    counts = _counts(capture_fx(_rms_norm_scale, _case(64)))
    assert counts.get("rms_norm") == 1 and counts.get("mul") == 1 and counts.get("cast") in (2, 3)


def test_the_fold_leaves_one_weighted_normalization():
    graph = rewrite(capture_fx(_rms_norm_scale, _case(64)))
    counts = _counts(graph)
    assert counts == {"rms_norm": 1}
    (norm,) = graph.ops
    assert len(norm.inputs) == 2 and norm.attrs["has_weight"] is True


def test_the_folded_normalization_is_bit_identical():
    for seed in range(4):
        value, weight = _case(128, seed=seed, rows=(2, 3))
        graph = capture_fx(_rms_norm_scale, (value, weight))
        folded = fuse_norm_scale(graph)
        assert len(folded.ops) < len(graph.ops)
        (expected,) = run_graph(graph, [value, weight])
        (actual,) = run_graph(folded, [value, weight])
        assert torch.equal(actual, expected), seed
        with torch.no_grad():
            eager = _rms_norm_scale(value, weight)
        assert float((actual.float() - eager.float()).abs().max()) < 1e-2


def test_the_fold_keeps_the_normalized_row_when_it_has_two_readers():
    def two_readers(value, weight):
        upcast = value.to(torch.float32)
        variance = upcast.pow(2).mean(-1, keepdim=True)
        normalized = upcast * torch.rsqrt(variance + EPS)
        return ((weight * normalized) + normalized).to(value.dtype)

    graph = rewrite(capture_fx(two_readers, _case(64)))
    norms = [op for op in graph.ops if op.op == "rms_norm"]
    assert len(norms) == 1 and len(norms[0].inputs) == 1      # standalone form: the scale stayed outside


def _projection_case(rows, seed=1, hidden=128, out=64):
    rng = np.random.default_rng(seed)
    value = torch.from_numpy(rng.standard_normal((1, rows, hidden)).astype(np.float32)).bfloat16()
    weight = torch.from_numpy((rng.standard_normal(hidden) * 0.1 + 1).astype(np.float32)).bfloat16()
    packed, scales = quantize_int4((rng.standard_normal((out, hidden)) * 0.05).astype(np.float32), GROUP)
    return value, weight, torch.from_numpy(packed), torch.from_numpy(scales).bfloat16()


def _normed_projection(value, weight, packed, scales):
    return torch.nn.functional.linear(_rms_norm_scale(value, weight), dequantize_i4(packed, scales, GROUP))


def test_the_norm_moves_into_a_single_row_packed_projection():
    operands = _projection_case(rows=1)
    graph = rewrite(capture_fx(_normed_projection, operands))
    counts = _counts(graph)
    assert counts.get("matmul") == 1 and "rms_norm" not in counts and "dequantize_i4" not in counts
    matmul = next(op for op in graph.ops if op.op == "matmul")
    assert matmul.attrs["rms_norm_eps"] == EPS and matmul.attrs["weight_group_size"] == GROUP
    assert len(matmul.inputs) == 4                            # x, words, scales, norm weight


def test_the_fused_projection_matches_the_standalone_norm():
    operands = _projection_case(rows=1, seed=3)
    captured = capture_fx(_normed_projection, operands)
    (fused,) = run_graph(rewrite(captured), list(operands))
    (plain,) = run_graph(captured, list(operands))
    scale = float(plain.float().abs().max())
    assert float((fused.float() - plain.float()).abs().max()) <= 1e-2 * scale


def test_a_projection_over_several_rows_keeps_its_norm():
    operands = _projection_case(rows=4)
    graph = rewrite(capture_fx(_normed_projection, operands))
    counts = _counts(graph)
    assert counts.get("rms_norm") == 1 and counts.get("dequantize_i4") == 1
    matmul = next(op for op in graph.ops if op.op == "matmul")
    assert "rms_norm_eps" not in matmul.attrs and "weight_group_size" not in matmul.attrs


def test_a_normalized_row_with_another_reader_keeps_its_norm():
    def shared(value, weight, packed, scales):
        row = _rms_norm_scale(value, weight)
        return torch.nn.functional.linear(row, dequantize_i4(packed, scales, GROUP)), row

    operands = _projection_case(rows=1)
    graph = rewrite(capture_fx(shared, operands))
    assert _counts(graph).get("rms_norm") == 1
    matmul = next(op for op in graph.ops if op.op == "matmul")
    assert "rms_norm_eps" not in matmul.attrs and matmul.attrs["weight_group_size"] == GROUP
