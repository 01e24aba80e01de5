"""Packed weights through the compiler: the fold, the kernel binding, and the numbers.

Mirrors the strategy of the reference's tests/test_quantized_matmul.py for the CUDA target,
without a GPU. There are two compiled shapes and they take different paths: a single-row matmul
(decode) is folded, ``matmul(x, Wp, S){weight_group_size, weight_bits}``, and no unpacked weight
exists in the graph; a wider matmul (prefill) keeps the explicit unpack as an operation, which
the backend binds as the weight operand of the multi-row kernel instead of materialising it.
The numbers are the oracle's, run over the lowered graph, against the same product evaluated
directly: ``x @ dequantize(Wp, S)^T`` with fp32 accumulation and one rounding.
"""

import numpy as np
import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.models.quantized import dequantize_i4, dequantize_i8
from aotolith_b200.quantize import quantize_int4, quantize_int8
from oracle import ops_ref as ref
from oracle.interp import run_graph

GROUP = 32
UNPACK = {4: (dequantize_i4, quantize_int4, ref.dequantize_i4), 8: (dequantize_i8, quantize_int8, ref.dequantize_i8)}


def _case(rows: int, inner: int, batch: int, seed: int, bits: int = 4):
    rng = np.random.default_rng(seed)
    weight = rng.standard_normal((rows, inner)).astype(np.float32)
    activation = torch.from_numpy(rng.standard_normal((batch, inner)).astype(np.float32)).bfloat16()
    packed, scales = UNPACK[bits][1](weight, GROUP)
    return activation, torch.from_numpy(packed), torch.from_numpy(scales).bfloat16()


def _direct(activation, packed, scales, bits: int = 4):
    weight = UNPACK[bits][2](packed, scales, GROUP)
    return (activation.float() @ weight.float().T).bfloat16()


def _compile(rows: int, inner: int, batch: int, seed: int, bits: int = 4):
    activation, packed, scales = _case(rows, inner, batch, seed, bits)
    unpack = UNPACK[bits][0]

    def call(activation, packed, scales):
        return torch.matmul(activation, unpack(packed, scales, GROUP).t())

    compiled = aoto.compile_callable(call, (activation, packed, scales))
    (actual,) = run_graph(compiled.plan.graph, [activation, packed, scales])
    return compiled, actual, _direct(activation, packed, scales, bits)


def _ops(compiled):
    return [op.op for op in compiled.plan.graph.ops]


def _matmul(compiled):
    return next(op for op in compiled.plan.graph.ops if op.op in ("matmul", "addmm"))


def _kernels(compiled):
    return [s.artifact_name for s in compiled.plan.selections]


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rows,inner", [(64, 128), (32, 256), (128, 64)])
def test_decode_matmul_matches_the_direct_product(rows, inner, bits):
    _, actual, expected = _compile(rows, inner, 1, seed=rows + inner, bits=bits)
    assert actual.dtype == torch.bfloat16 and actual.shape == (1, rows)
    assert torch.equal(actual, expected)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("batch", [2, 5, 64])
def test_prefill_matmul_matches_the_direct_product(batch, bits):
    _, actual, expected = _compile(64, 128, batch, seed=batch, bits=bits)
    assert actual.shape == (batch, 64)
    assert torch.equal(actual, expected)


@pytest.mark.parametrize("bits", [4, 8])
def test_a_single_row_matmul_keeps_no_unpacked_weight(bits):
    compiled, _, _ = _compile(64, 128, 1, seed=3, bits=bits)
    assert not any(name.startswith("dequantize") for name in _ops(compiled))
    matmul = _matmul(compiled)
    assert len(matmul.inputs) == 3
    assert "transpose_b" not in matmul.attrs
    # the packed words are an operand as they are: int32 [rows, inner * bits / 32]
    packed_type = compiled.plan.graph.value(matmul.inputs[1]).type
    assert packed_type.shape == (64, 128 * bits // 32)


@pytest.mark.parametrize("bits", [4, 8])
def test_a_wide_matmul_keeps_the_unpack(bits):
    compiled, _, _ = _compile(64, 128, 4, seed=4, bits=bits)
    assert _ops(compiled).count(f"dequantize_i{bits}") == 1
    assert "weight_group_size" not in _matmul(compiled).attrs
    # ... but the backend never materialises it: the unpack is the weight operand of the row kernel
    kernels = _kernels(compiled)
    assert "aoto_sm100_qmatmul[weight operand]" in kernels
    assert f"aoto_sm100_dequantize_i{bits}" not in kernels


@pytest.mark.parametrize("bits", [4, 8])
def test_group_size_and_width_survive_into_the_folded_matmul(bits):
    compiled, _, _ = _compile(64, 128, 1, seed=5, bits=bits)
    attrs = _matmul(compiled).attrs
    assert attrs["weight_group_size"] == GROUP and attrs["weight_bits"] == bits


def test_the_decode_matmul_is_bound_to_a_native_kernel():
    four, _, _ = _compile(64, 128, 1, seed=6, bits=4)
    (selection,) = [s for s in four.plan.selections if s.op == "matmul"]
    assert selection.implementation == "cuda_kernel" and selection.is_native
    assert selection.artifact_name == "aoto_sm100_qmatmul[qgemv_generic]"      # group 32: outside the fast variant
    assert selection.device_architecture == "sm_100a"
    eight, _, _ = _compile(64, 128, 1, seed=6, bits=8)
    (selection,) = [s for s in eight.plan.selections if s.op == "matmul"]
    assert selection.artifact_name == "aoto_sm100_qmatmul[qgemv_i8]"


def test_a_graph_that_returns_the_unpacked_matrix_keeps_the_unpack():
    from aotolith_b200.capture import capture_fx
    from aotolith_b200.errors import UnsupportedOperationError
    from aotolith_b200.passes import rewrite

    activation, packed, scales = _case(64, 128, 1, seed=7)

    def call(activation, packed, scales):
        weight = dequantize_i4(packed, scales, GROUP)
        return torch.matmul(activation, weight.t()), weight

    graph = rewrite(capture_fx(call, (activation, packed, scales)))
    assert [op.op for op in graph.ops].count("dequantize_i4") == 1
    matmul = next(op for op in graph.ops if op.op == "matmul")
    assert "weight_group_size" not in matmul.attrs            # the fold leaves a weight alone that is also a result
    product, weight = run_graph(graph, [activation, packed, scales])
    assert torch.equal(weight, ref.dequantize_i4(packed, scales, GROUP))
    assert torch.equal(product, _direct(activation, packed, scales))
    # The matmul now reads a materialised bf16 weight. This target has packed projections only,
    # and no interpreter to fall back to: the compile is refused and says why.
    with pytest.raises(UnsupportedOperationError, match="dense matmul"):
        aoto.compile_callable(call, (activation, packed, scales))


@pytest.mark.parametrize("bits", [4, 8])
def test_a_residual_folds_into_one_packed_addmm(bits):
    activation, packed, scales = _case(64, 128, 1, seed=8, bits=bits)
    residual = torch.from_numpy(np.random.default_rng(9).standard_normal((1, 64)).astype(np.float32)).bfloat16()
    unpack = UNPACK[bits][0]

    def call(activation, residual, packed, scales):
        return residual + torch.nn.functional.linear(activation, unpack(packed, scales, GROUP))

    compiled = aoto.compile_callable(call, (activation, residual, packed, scales))
    assert _ops(compiled) == ["addmm"]
    addmm = _matmul(compiled)
    assert addmm.attrs["weight_group_size"] == GROUP and addmm.attrs["weight_bits"] == bits
    (actual,) = run_graph(compiled.plan.graph, [activation, residual, packed, scales])
    expected = residual + _direct(activation, packed, scales, bits)
    assert torch.equal(actual, expected)


@pytest.mark.parametrize("bits", [4, 8])
def test_decode_mlp_pairs_two_packed_projections_into_one_launch(bits):
    """``silu(x Wg^T) * (x Wu^T)`` over one activation row: one paired matmul, one kernel."""

    rng = np.random.default_rng(10)
    inner, rows = 128, 96
    activation = torch.from_numpy(rng.standard_normal((1, inner)).astype(np.float32)).bfloat16()
    gate_p, gate_s = UNPACK[bits][1]((rng.standard_normal((rows, inner)) * 0.1).astype(np.float32), GROUP)
    up_p, up_s = UNPACK[bits][1]((rng.standard_normal((rows, inner)) * 0.1).astype(np.float32), GROUP)
    operands = (activation, torch.from_numpy(gate_p), torch.from_numpy(gate_s).bfloat16(),
                torch.from_numpy(up_p), torch.from_numpy(up_s).bfloat16())
    unpack = UNPACK[bits][0]

    def call(activation, gate_p, gate_s, up_p, up_s):
        gate = torch.nn.functional.linear(activation, unpack(gate_p, gate_s, GROUP))
        up = torch.nn.functional.linear(activation, unpack(up_p, up_s, GROUP))
        return torch.nn.functional.silu(gate) * up

    compiled = aoto.compile_callable(call, operands)
    assert _ops(compiled) == ["matmul"]
    paired = _matmul(compiled)
    assert paired.attrs["epilogue"] == "silu_mul_paired" and len(paired.inputs) == 5
    assert paired.attrs["weight_bits"] == bits
    (selection,) = compiled.plan.selections
    assert selection.artifact_name.startswith("aoto_sm100_qmatmul[")
    (actual,) = run_graph(compiled.plan.graph, list(operands))
    gate = _direct(activation, operands[1], operands[2], bits)
    up = _direct(activation, operands[3], operands[4], bits)
    expected = gate * (up / (1.0 + torch.exp(-gate)))   # the paired form of the oracle: gate first
    scale = float(expected.float().abs().max())
    assert float((actual.float() - expected.float()).abs().max()) <= 2e-2 * scale
