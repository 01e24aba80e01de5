from .decoder import (
    FAMILIES,
    DecoderBucketedRuntime,
    DecoderFamily,
    DecoderMemoryFootprint,
    DecoderStaticCacheRuntime,
    compile_decoder_bucketed,
    compile_decoder_static_cache,
    decode_rows_mask,
    family_for,
    prefill_mask,
)
from .llama import compile_llama_bucketed, compile_llama_static_cache
from .quantized import dequantize_i4, dequantize_i8, pack_weight
from .qwen2 import compile_qwen2_bucketed, compile_qwen2_static_cache

__all__ = [
    "FAMILIES", "DecoderBucketedRuntime", "DecoderFamily", "DecoderMemoryFootprint",
    "DecoderStaticCacheRuntime", "compile_decoder_bucketed", "compile_decoder_static_cache",
    "compile_llama_bucketed", "compile_llama_static_cache", "compile_qwen2_bucketed",
    "compile_qwen2_static_cache", "decode_rows_mask", "dequantize_i4", "dequantize_i8", "family_for", "pack_weight", "prefill_mask",
]
