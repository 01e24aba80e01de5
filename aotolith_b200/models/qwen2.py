"""Qwen2 / Qwen2.5 frontend: the shared static-cache adapter pinned to one family.

Mirrors ``src/aotolith/models/qwen2.py`` of the reference.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any

from .decoder import (
    DecoderBucketedRuntime,
    DecoderStaticCacheRuntime,
    compile_decoder_bucketed,
    compile_decoder_static_cache,
    family_for,
)

FAMILY = "qwen2"


def check_qwen2_model(model) -> None:
    family_for(model, require=FAMILY)


def compile_qwen2_static_cache(model, *, prompt_length: int, max_new_tokens: int, **options: Any) -> DecoderStaticCacheRuntime:
    check_qwen2_model(model)
    return compile_decoder_static_cache(
        model, prompt_length=prompt_length, max_new_tokens=max_new_tokens, family=FAMILY, **options
    )


def compile_qwen2_bucketed(model, *, prompt_lengths: Sequence[int], max_new_tokens: int, **options: Any) -> DecoderBucketedRuntime:
    check_qwen2_model(model)
    return compile_decoder_bucketed(
        model, prompt_lengths=prompt_lengths, max_new_tokens=max_new_tokens, family=FAMILY, **options
    )
