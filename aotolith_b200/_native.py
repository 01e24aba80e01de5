"""ctypes binding of ``libaoto_sm100.so`` (declared in ``include/aoto_sm100.h``).

The library is the only way this package computes anything: there is no eager
or CPU substitute, and loading fails loudly (``DeviceError``) when the shared
object has not been built. The structures below mirror the C ones field for
field; ``EXPORTS`` lists every symbol the header declares so a test can check
that the built library exports them all.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

from .errors import DeviceError

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libaoto_sm100.so"

ABI_VERSION = 1

OK = 0
ERR_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_LAUNCH = -3
ERR_TIMEOUT = -4
ERR_TOO_LARGE = -5

ADDEND_NONE, ADDEND_VECTOR, ADDEND_FULL = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SILU_MUL, EPILOGUE_SILU_MUL_PAIRED = 0, 1, 2
FLAG_PDL = 1
FLAG_WEIGHT_BITS_8 = 2
FLAG_WEIGHT_DENSE = 4


class QMatmulArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("packed", c_void_p), ("scales", c_void_p),
        ("packed2", c_void_p), ("scales2", c_void_p), ("addend", c_void_p),
        ("gate", c_void_p), ("norm_weight", c_void_p), ("out", c_void_p),
        ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("M", c_int32), ("N", c_int32), ("K", c_int32), ("group_size", c_int32),
        ("addend_kind", c_int32), ("epilogue", c_int32),
        ("alpha", c_float), ("beta", c_float), ("rms_norm_eps", c_float),
        ("flags", c_int32),
    ]


class DequantizeArgs(Structure):
    _fields_ = [
        ("packed", c_void_p), ("scales", c_void_p), ("out", c_void_p),
        ("N", c_int32), ("K", c_int32), ("group_size", c_int32),
    ]


class RmsNormArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("residual", c_void_p), ("weight", c_void_p),
        ("out", c_void_p), ("sum_out", c_void_p),
        ("rows", c_int32), ("H", c_int32), ("eps", c_float),
    ]


class RopeArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("cos_table", c_void_p), ("sin_table", c_void_p), ("out", c_void_p),
        ("B", c_int32), ("heads", c_int32), ("T", c_int32), ("D", c_int32),
        ("stride_b", c_int64), ("stride_h", c_int64), ("stride_t", c_int64),
    ]


class EmbeddingArgs(Structure):
    _fields_ = [
        ("table", c_void_p), ("ids", c_void_p), ("out", c_void_p), ("bad_index", c_void_p),
        ("rows", c_int32), ("width", c_int32), ("count", c_int32),
    ]


class MaskSelectArgs(Structure):
    _fields_ = [
        ("mask", c_void_p), ("out", c_void_p), ("count", c_int64),
        ("on_true", c_float), ("on_false", c_float),
    ]


class ArgmaxArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("out", c_void_p), ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("rows", c_int32), ("width", c_int32),
    ]


class KvAppendArgs(Structure):
    _fields_ = [
        ("cache", c_void_p), ("row", c_void_p), ("key", c_void_p),
        ("cos_row", c_void_p), ("sin_row", c_void_p), ("q_out", c_void_p), ("new_pair", c_void_p),
        ("layer", c_int32), ("layers", c_int32), ("kv_heads", c_int32), ("capacity", c_int32),
        ("head_dim", c_int32), ("query_heads", c_int32), ("query_start", c_int32),
        ("key_start", c_int32), ("value_start", c_int32), ("rotate", c_int32),
    ]


class AttentionArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("mask", c_void_p), ("out", c_void_p),
        ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("query_heads", c_int32), ("kv_heads", c_int32), ("q_len", c_int32), ("kv_len", c_int32),
        ("head_dim", c_int32), ("causal", c_int32), ("scale", c_float),
    ]


class StepInputsArgs(Structure):
    _fields_ = [("counters", c_void_p), ("position", c_void_p), ("mask", c_void_p), ("capacity", c_int32)]


class GreedyPickArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("token", c_void_p), ("generated", c_void_p), ("counters", c_void_p),
        ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("width", c_int32), ("generated_capacity", c_int32),
    ]


class StepStage(Structure):
    """Mirror of ``aoto_step_stage`` (field order and types must match the header)."""

    _fields_ = [
        ("x", c_void_p), ("x_index", c_void_p),
        ("packed", c_void_p), ("scales", c_void_p), ("packed2", c_void_p), ("scales2", c_void_p),
        ("addend", c_void_p), ("norm_weight", c_void_p), ("out", c_void_p),
        ("row", c_void_p), ("cos_table", c_void_p), ("sin_table", c_void_p), ("position", c_void_p),
        ("cache_in", c_void_p), ("cache_out", c_void_p), ("mask", c_void_p), ("attn_out", c_void_p),
        ("token", c_void_p), ("generated", c_void_p), ("counters", c_void_p),
        ("x_rows", c_int64),
        ("kind", c_int32), ("flags", c_int32),
        ("N", c_int32), ("K", c_int32), ("group_size", c_int32), ("addend_mode", c_int32), ("epilogue", c_int32),
        ("query_heads", c_int32), ("kv_heads", c_int32), ("capacity", c_int32), ("head_dim", c_int32),
        ("query_start", c_int32), ("key_start", c_int32), ("value_start", c_int32), ("table_rows", c_int32),
        ("generated_capacity", c_int32), ("reserved", c_int32),
        ("alpha", c_float), ("beta", c_float), ("rms_norm_eps", c_float), ("scale", c_float),
    ]


class DecodeStepArgs(Structure):
    _fields_ = [
        ("stages", c_void_p), ("stage_count", c_int32), ("ctas", c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", c_int32),
        ("status", c_void_p), ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("trace", c_void_p),
    ]


class StreamStage(Structure):
    """Mirror of ``aoto_stream_stage`` (64 bytes)."""

    _fields_ = [
        ("x", c_void_p), ("out", c_void_p), ("addend", c_void_p), ("norm_weight", c_void_p),
        ("N", c_int32), ("K", c_int32),
        ("alpha", c_float), ("beta", c_float), ("rms_norm_eps", c_float),
        ("kind", ctypes.c_uint8), ("epilogue", ctypes.c_uint8), ("addend_mode", ctypes.c_uint8), ("flags", ctypes.c_uint8),
        ("next_attention", c_int32), ("ordinal", c_int32),
    ]


class StreamStepArgs(Structure):
    """Mirror of ``aoto_stream_step_args``."""

    _fields_ = [
        ("stages", c_void_p), ("cta_table", c_void_p), ("duties", c_void_p), ("starts", c_void_p), ("stream", c_void_p),
        ("stream_bytes", c_int64),
        ("stage_count", c_int32), ("ctas", c_int32), ("ring_depth", c_int32), ("max_k", c_int32),
        ("query_heads", c_int32), ("kv_heads", c_int32), ("capacity", c_int32), ("head_dim", c_int32),
        ("query_start", c_int32), ("key_start", c_int32), ("value_start", c_int32), ("table_rows", c_int32),
        ("scale", c_float), ("first_attention", c_int32),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("position", c_void_p), ("mask", c_void_p),
        ("x_index", c_void_p), ("x_rows", c_int64),
        ("token", c_void_p), ("generated", c_void_p), ("counters", c_void_p),
        ("generated_capacity", c_int32), ("window", c_int32),
        ("epoch", ctypes.c_uint32), ("attention_stages", c_int32),
        ("status", c_void_p), ("scratch", c_void_p), ("scratch_bytes", c_int64),
        ("world", c_int32), ("rank", c_int32), ("peer_delta", c_int64 * 8), ("pick_exchange", c_void_p),
        ("vocab_offset", c_int32), ("reserved2", c_int32),
        ("trace", c_void_p),
    ]


STAGE_GEMV, STAGE_ATTENTION, STAGE_PICK = 1, 2, 3
STAGE_FLAG_ARGMAX, STAGE_FLAG_WINDOW, STAGE_FLAG_OUT_PLAIN, STAGE_FLAG_X_GATHER = 2, 4, 8, 16
STAGE_FLAG_TO_PEERS, STAGE_FLAG_X_SUM, STAGE_FLAG_ADDEND_SUM = 32, 64, 128
STAGE_ADDEND_NONE, STAGE_ADDEND_PLAIN, STAGE_ADDEND_STAMPED, STAGE_ADDEND_GATHER = 0, 1, 2, 3


#: symbol -> (restype, argtypes); one entry per declaration in include/aoto_sm100.h
class PeerSumArgs(Structure):
    _fields_ = [
        ("buffers", POINTER(c_void_p)), ("partial", c_void_p), ("out", c_void_p), ("epoch", c_void_p),
        ("status", c_void_p),
        ("world", c_int32), ("rank", c_int32), ("count", c_int32), ("capacity_words", c_int32),
    ]


EXPORTS: dict[str, tuple] = {
    "aoto_sm100_abi_version": (c_int, []),
    "aoto_sm100_compiled_arch": (c_int, []),
    "aoto_sm100_status_string": (c_char_p, [c_int]),
    "aoto_sm100_qmatmul": (c_int, [POINTER(QMatmulArgs), c_void_p]),
    "aoto_sm100_qmatmul_supported": (c_int, [POINTER(QMatmulArgs)]),
    "aoto_sm100_qmatmul_scratch_bytes": (c_int64, [POINTER(QMatmulArgs)]),
    "aoto_sm100_qmatmul_variant": (c_char_p, [POINTER(QMatmulArgs)]),
    "aoto_sm100_qmatmul_take_timeout_flag": (c_int, []),
    "aoto_sm100_dequantize_i4": (c_int, [POINTER(DequantizeArgs), c_void_p]),
    "aoto_sm100_dequantize_i8": (c_int, [POINTER(DequantizeArgs), c_void_p]),
    "aoto_sm100_rms_norm": (c_int, [POINTER(RmsNormArgs), c_void_p]),
    "aoto_sm100_rope": (c_int, [POINTER(RopeArgs), c_void_p]),
    "aoto_sm100_embedding": (c_int, [POINTER(EmbeddingArgs), c_void_p]),
    "aoto_sm100_mask_select": (c_int, [POINTER(MaskSelectArgs), c_void_p]),
    "aoto_sm100_argmax": (c_int, [POINTER(ArgmaxArgs), c_void_p]),
    "aoto_sm100_argmax_scratch_bytes": (c_int64, [c_int32, c_int32]),
    "aoto_sm100_step_inputs": (c_int, [POINTER(StepInputsArgs), c_void_p]),
    "aoto_sm100_greedy_pick": (c_int, [POINTER(GreedyPickArgs), c_void_p]),
    "aoto_sm100_decode_step": (c_int, [POINTER(DecodeStepArgs), c_void_p]),
    "aoto_sm100_decode_step_scratch_bytes": (c_int64, [POINTER(StepStage), c_int32]),
    "aoto_sm100_decode_step_supported": (c_int, [POINTER(StepStage), c_int32]),
    "aoto_sm100_decode_step_stage_size": (c_int, []),
    "aoto_sm100_stamped_bytes": (c_int64, [c_int64]),
    "aoto_sm100_stream_step": (c_int, [POINTER(StreamStepArgs), c_void_p]),
    "aoto_sm100_stream_step_smem_bytes": (c_int64, [POINTER(StreamStepArgs)]),
    "aoto_sm100_stream_args_size": (c_int, []),
    "aoto_sm100_stream_step_scratch_bytes_for": (c_int64, [POINTER(StreamStepArgs)]),
    "aoto_sm100_stream_step_scratch_bytes": (c_int64, [c_int32]),
    "aoto_sm100_stream_stage_size": (c_int, []),
    "aoto_sm100_kv_cache_append": (c_int, [POINTER(KvAppendArgs), c_void_p]),
    "aoto_sm100_attention": (c_int, [POINTER(AttentionArgs), c_void_p]),
    "aoto_sm100_attention_scratch_bytes": (c_int64, [POINTER(AttentionArgs)]),
    "aoto_sm100_attention_decode_static": (c_int, [POINTER(AttentionArgs), c_void_p]),
    "aoto_sm100_attention_static_scratch_limit": (c_int64, []),
    "aoto_sm100_peer_sum": (c_int, [POINTER(PeerSumArgs), c_void_p]),
    "aoto_sm100_peer_sum_buffer_bytes": (c_int64, [c_int32, c_int32]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the kernel library once; raise ``DeviceError`` if it is not built."""

    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise DeviceError(
                f"the sm_100a kernel library is missing: {LIB_PATH}",
                hint="build it with `python -m aotolith_b200.csrc.build` (needs nvcc, not a GPU)",
            )
        try:
            lib = ctypes.CDLL(str(LIB_PATH))
        except OSError as error:
            raise DeviceError(
                f"the sm_100a kernel library failed to load: {error}",
                hint="it links against the CUDA runtime; check that libcudart is reachable",
            ) from error
        for name, (restype, argtypes) in EXPORTS.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as error:
                raise DeviceError(f"kernel library does not export {name}") from error
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.aoto_sm100_decode_step_stage_size() != ctypes.sizeof(StepStage):
            raise DeviceError(
                "the stage descriptor of the kernel library and of this binding differ in size "
                f"({lib.aoto_sm100_decode_step_stage_size()} vs {ctypes.sizeof(StepStage)})",
                hint="rebuild with `python -m aotolith_b200.csrc.build --force`",
            )
        if lib.aoto_sm100_stream_stage_size() != ctypes.sizeof(StreamStage):
            raise DeviceError(
                "the streamed-step stage descriptor of the kernel library and of this binding differ in size "
                f"({lib.aoto_sm100_stream_stage_size()} vs {ctypes.sizeof(StreamStage)})",
                hint="rebuild with `python -m aotolith_b200.csrc.build --force`",
            )
        if lib.aoto_sm100_stream_args_size() != ctypes.sizeof(StreamStepArgs):
            raise DeviceError(
                "the streamed-step arguments of the kernel library and of this binding differ in size "
                f"({lib.aoto_sm100_stream_args_size()} vs {ctypes.sizeof(StreamStepArgs)})",
                hint="rebuild with `python -m aotolith_b200.csrc.build --force`",
            )
        if lib.aoto_sm100_abi_version() != ABI_VERSION:
            raise DeviceError(
                f"kernel library ABI {lib.aoto_sm100_abi_version()} != binding ABI {ABI_VERSION}",
                hint="rebuild with `python -m aotolith_b200.csrc.build --force`",
            )
        _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().aoto_sm100_status_string(status).decode()


def check(status: int, what: str) -> None:
    """Map a non-zero status of entry point ``what`` to ``DeviceError``."""

    if status != OK:
        raise DeviceError(
            f"{what} failed with status {status}: {status_string(status)}",
            hint="the request was refused before or at launch; no device state was changed",
        )
