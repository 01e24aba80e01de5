"""Weight-only group quantisation: the packed format and its host-side codecs.

The format is the reference compiler's (``src/aotolith/quantize.py:1-37``):

* a weight is ``[out, in]``; the ``in`` axis is cut into groups of
  ``group_size`` values that share one scale ``max|w| / magnitude`` (7 for four
  bits, 127 for eight); an all-zero group is scaled as if its magnitude were one
  (scale ``1 / magnitude``), which keeps the division finite and its codes zero;
* codes are ``clip(rint(w / scale), lowest, magnitude)`` (round half to even),
  stored two's complement;
* 32-bit words hold eight nibbles (or four bytes), code ``k`` of a word at bit
  ``4k`` (``8k``), word ``j`` of a row holding codes ``8j .. 8j+7``;
* scales are ``[out, in / group_size]``, float32 from the packer and cast to the
  model dtype by the caller *after* the codes were chosen with the fp32 scale.

These functions run at compile time on the host (packing a checkpoint) and in
tests; the device never calls them.
"""

from __future__ import annotations

import numpy as np

INT4_MIN, INT4_MAX, INT4_MAGNITUDE = -8, 7, 7
INT8_MIN, INT8_MAX, INT8_MAGNITUDE = -128, 127, 127
NIBBLES_PER_WORD = 8
BYTES_PER_WORD = 4


def check_group_size(group_size: int, inner: int, packed_width: int = NIBBLES_PER_WORD) -> int:
    """Validate a group size against a reduction length (``quantize.py:69-92``).

    Raises ``ValueError`` for a non-positive size, one that is not a multiple of
    the codes a word holds, or one that does not divide ``inner``.
    """

    if group_size <= 0:
        raise ValueError(f"quantization group size must be positive, got {group_size}")
    if group_size % packed_width:
        raise ValueError(
            f"quantization group size must be a multiple of {packed_width}, got {group_size}"
        )
    if inner % group_size:
        raise ValueError(
            f"quantization group size {group_size} does not divide the reduction length {inner}"
        )
    return group_size


def _quantize(weight, group_size: int, bits: int) -> tuple[np.ndarray, np.ndarray]:
    per_word = 32 // bits
    magnitude = (1 << (bits - 1)) - 1
    matrix = np.asarray(weight, dtype=np.float32)
    if matrix.ndim != 2:
        raise ValueError(f"quantization expects a 2-D weight, got {matrix.shape}")
    rows, inner = matrix.shape
    check_group_size(group_size, inner, per_word)
    grouped = matrix.reshape(rows, inner // group_size, group_size)
    peak = np.abs(grouped).max(axis=2)
    scale = (np.where(peak > 0.0, peak, np.float32(1.0)) / np.float32(magnitude)).astype(np.float32)
    codes = np.rint(grouped / scale[..., None])
    codes = np.clip(codes, -magnitude - 1, magnitude).astype(np.int64).reshape(rows, inner)
    fields = (codes & ((1 << bits) - 1)).reshape(rows, inner // per_word, per_word)
    shifts = (np.arange(per_word, dtype=np.int64) * bits)[None, None, :]
    words = (fields << shifts).sum(axis=2)  # disjoint bit fields: sum == or
    packed = (words & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
    return np.ascontiguousarray(packed), scale


def quantize_int4(weight, group_size: int = 64) -> tuple[np.ndarray, np.ndarray]:
    """``(packed int32 [out, in/8], scales float32 [out, in/group])``."""

    return _quantize(weight, group_size, 4)


def quantize_int8(weight, group_size: int = 64) -> tuple[np.ndarray, np.ndarray]:
    """``(packed int32 [out, in/4], scales float32 [out, in/group])``."""

    return _quantize(weight, group_size, 8)


def _unpack(packed, bits: int) -> np.ndarray:
    words = np.asarray(packed)
    if not np.issubdtype(words.dtype, np.integer):
        raise TypeError("unpack_codes needs integer words")
    if words.ndim != 2:
        raise ValueError(f"packed words must be 2-D, got {words.shape}")
    per_word = 32 // bits
    wide = words.astype(np.int64) & 0xFFFFFFFF
    shifts = (np.arange(per_word, dtype=np.int64) * bits)[None, None, :]
    fields = (wide[:, :, None] >> shifts) & ((1 << bits) - 1)
    signed = np.where(fields >= (1 << (bits - 1)), fields - (1 << bits), fields)
    return signed.astype(np.int8).reshape(words.shape[0], words.shape[1] * per_word)


def unpack_codes(packed) -> np.ndarray:
    """Signed 4-bit codes ``[out, in]`` (int8) of packed words."""

    return _unpack(packed, 4)


def unpack_codes_int8(packed) -> np.ndarray:
    """Signed 8-bit codes ``[out, in]`` (int8) of packed words."""

    return _unpack(packed, 8)


def dequantize_int4(packed, scales, group_size: int) -> np.ndarray:
    """float32 weights a packed 4-bit pair stands for."""

    spread = np.repeat(np.asarray(scales, dtype=np.float32), group_size, axis=-1)
    return unpack_codes(packed).astype(np.float32) * spread


def dequantize_int8(packed, scales, group_size: int) -> np.ndarray:
    """float32 weights a packed 8-bit pair stands for."""

    spread = np.repeat(np.asarray(scales, dtype=np.float32), group_size, axis=-1)
    return unpack_codes_int8(packed).astype(np.float32) * spread


def quantize_torch(weight, group_size: int = 64, bits: int = 4):
    """The same packer on a torch tensor, wherever it lives: ``(int32 words, float32 scales)``.

    Every step is the fp32 operation of :func:`_quantize` (``abs`` / ``max`` / divide /
    round-half-to-even / clip), so the words and scales are bit for bit those of the NumPy
    packer; ``tests/test_quantize.py`` holds the two against each other. Packing a model that
    was built on the GPU stays on the GPU.
    """

    import torch

    per_word = 32 // bits
    magnitude = (1 << (bits - 1)) - 1
    matrix = weight.detach().to(torch.float32)
    if matrix.dim() != 2:
        raise ValueError(f"quantization expects a 2-D weight, got {tuple(matrix.shape)}")
    rows, inner = matrix.shape
    check_group_size(group_size, inner, per_word)
    grouped = matrix.reshape(rows, inner // group_size, group_size)
    peak = grouped.abs().amax(dim=2)
    scale = torch.where(peak > 0, peak, torch.ones_like(peak)) / magnitude
    codes = torch.round(grouped / scale[..., None]).clamp_(-magnitude - 1, magnitude).to(torch.int64)
    fields = (codes.reshape(rows, inner // per_word, per_word) & ((1 << bits) - 1))
    shifts = torch.arange(per_word, dtype=torch.int64, device=matrix.device) * bits
    words = (fields << shifts).sum(dim=2)  # disjoint bit fields: sum == or
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words.contiguous(), scale.contiguous()
