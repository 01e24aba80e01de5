"""Seeded input builders shared by the parity tests."""

from __future__ import annotations

import numpy as np
import torch

from aotolith_b200.quantize import quantize_int4


def packed_weight(seed: int, n_rows: int, K: int, group: int, std: float = 0.02):
    """bf16 ~N(0, std) weight, quantised with the reference packer.

    Returns ``(packed int32 [N,K/8], scales bf16 [N,K/group])`` as CPU tensors.
    """

    rng = np.random.default_rng(seed)
    weight = torch.from_numpy((rng.standard_normal((n_rows, K)) * std).astype(np.float32)).bfloat16()
    packed, scales = quantize_int4(weight.float().numpy(), group)
    return torch.from_numpy(packed), torch.from_numpy(scales).bfloat16()


def activations(seed: int, *shape: int, std: float = 1.0) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy((rng.standard_normal(shape) * std).astype(np.float32)).bfloat16()


def exact_packed_matmul(x, packed, scales, group):
    """float64 ``x @ (code*scale)^T`` with no intermediate rounding."""

    from oracle.ops_ref import unpack_codes

    weight = unpack_codes(packed).double() * scales.double().repeat_interleave(group, dim=-1)
    return x.double() @ weight.T


def rel_max_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    scale = float(expected.double().abs().max())
    return float((actual.double() - expected.double()).abs().max()) / max(scale, 1e-30)
