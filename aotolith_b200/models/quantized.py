"""The ``dequantize_i4`` / ``dequantize_i8`` torch operators and the weight packer.

Tracing needs the unpack of a packed weight to be ONE node (the rewrite
pipeline folds ``matmul(x, dequantize_i4(Wp, S))`` into a packed matmul), so it
is a ``torch.library`` operator with a fake (shape-only) implementation for
capture and a CUDA implementation that calls the sm_100a kernel. There is
deliberately no CPU implementation on this target.

Mirrors ``src/aotolith/models/quantized.py:40-163`` of the reference (operator
schema, packer contract: NumPy packs, torch carries the result, scales keep the
weight's dtype).
"""

from __future__ import annotations

import threading

import numpy as np

from ..quantize import check_group_size, quantize_int4, quantize_int8

NAMESPACE = "aotolith_b200"
DEQUANTIZE_I4 = f"{NAMESPACE}::dequantize_i4"
DEQUANTIZE_I8 = f"{NAMESPACE}::dequantize_i8"

_registered = False
_lock = threading.Lock()


def _register() -> None:
    global _registered
    if _registered:
        return
    with _lock:
        if _registered:
            return
        import torch
        from torch import Tensor

        torch.library.define(
            DEQUANTIZE_I4, "(Tensor packed, Tensor scales, int group_size) -> Tensor"
        )

        @torch.library.impl(DEQUANTIZE_I4, "CUDA")
        def _dequantize_cuda(packed: Tensor, scales: Tensor, group_size: int) -> Tensor:
            from .. import ops

            return ops.dequantize_i4(packed, scales, group_size)

        @torch.library.register_fake(DEQUANTIZE_I4)
        def _dequantize_fake(packed: Tensor, scales: Tensor, group_size: int) -> Tensor:
            if packed.dim() != 2:
                raise ValueError(f"packed int4 weights must be 2-D, got {packed.shape}")
            return packed.new_empty((packed.shape[0], packed.shape[1] * 8), dtype=scales.dtype)

        torch.library.define(
            DEQUANTIZE_I8, "(Tensor packed, Tensor scales, int group_size) -> Tensor"
        )

        @torch.library.impl(DEQUANTIZE_I8, "CUDA")
        def _dequantize_i8_cuda(packed: Tensor, scales: Tensor, group_size: int) -> Tensor:
            from .. import ops

            return ops.dequantize_i8(packed, scales, group_size)

        @torch.library.register_fake(DEQUANTIZE_I8)
        def _dequantize_i8_fake(packed: Tensor, scales: Tensor, group_size: int) -> Tensor:
            if packed.dim() != 2:
                raise ValueError(f"packed int8 weights must be 2-D, got {packed.shape}")
            return packed.new_empty((packed.shape[0], packed.shape[1] * 4), dtype=scales.dtype)

        _registered = True


def dequantize_i4(packed, scales, group_size: int):
    """``[N, K]`` weight in the scales' dtype from packed words (one traced node)."""

    _register()
    import torch

    return torch.ops.aotolith_b200.dequantize_i4(packed, scales, group_size)


def dequantize_i8(packed, scales, group_size: int):
    """Eight-bit twin of :func:`dequantize_i4` (``models/quantized.py:124-130`` of the reference)."""

    _register()
    import torch

    return torch.ops.aotolith_b200.dequantize_i8(packed, scales, group_size)


def pack_weight(weight, group_size: int, bits: int = 4):
    """Pack a ``[out, in]`` weight: ``(int32 words [out, in*bits/32], scales [out, in/group])``.

    ``weight`` is a torch tensor or array-like. Scales come back in the weight's
    dtype (cast after the codes were chosen with the fp32 scale).
    """

    import torch

    if isinstance(weight, torch.Tensor) and weight.is_cuda:
        # a model built on the device is packed there (the same arithmetic, bit for bit)
        from ..quantize import quantize_torch

        if weight.dim() != 2:
            raise ValueError(f"a quantized weight must be 2-D, got {tuple(weight.shape)}")
        if bits not in (4, 8):
            raise ValueError(f"bits must be 4 or 8, got {bits!r}")
        words, scales = quantize_torch(weight, group_size, bits)
        return words, scales.to(weight.dtype)
    if isinstance(weight, torch.Tensor):
        matrix = weight.detach().float().cpu().numpy()
        scale_dtype = weight.dtype
    else:
        matrix = np.asarray(weight, dtype=np.float32)
        scale_dtype = torch.float32
    if matrix.ndim != 2:
        raise ValueError(f"a quantized weight must be 2-D, got {matrix.shape}")
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits!r}")
    check_group_size(group_size, matrix.shape[-1], 32 // bits)
    packed, scales = (quantize_int8 if bits == 8 else quantize_int4)(matrix, group_size)
    return torch.from_numpy(packed), torch.from_numpy(scales).to(scale_dtype)
