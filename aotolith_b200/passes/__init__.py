"""The rewrite pipeline: captured IR -> lowered IR.

Sixteen ordered passes, the order and names of the reference's
``src/aotolith/passes/driver.py:37-100``. The pipeline is target independent
except for one flag: ``native_matmul`` tells ``fuse_rms_norm_epilogue`` whether
dense single-row projections may absorb a norm too (packed ones always do).
"""

from __future__ import annotations

from collections.abc import Callable

from ..ir import Graph
from .cache import fuse_kv_cache_update, fuse_rope_into_kv_cache_update
from .cse import eliminate_common_subexpressions
from .fusion import (
    fuse_activation_epilogue,
    fuse_attention,
    fuse_gate_up_projection,
    fuse_norm_scale,
    fuse_pointwise,
    fuse_residual_epilogue,
    fuse_rms_norm_epilogue,
    fuse_rope,
)
from .layout import (
    canonicalize_batched_matmul,
    collapse_trailing_layouts,
    fold_matmul_input_layouts,
    simplify_layouts,
)
from .quantize import fold_quantized_weights

PIPELINE: tuple[tuple[str, Callable[..., Graph]], ...] = (
    ("fuse_kv_cache_update", fuse_kv_cache_update),
    ("simplify_layouts", simplify_layouts),
    ("canonicalize_batched_matmul", canonicalize_batched_matmul),
    ("fuse_attention", fuse_attention),
    ("fold_matmul_input_layouts", fold_matmul_input_layouts),
    ("fold_quantized_weights", fold_quantized_weights),
    ("fuse_norm_scale", fuse_norm_scale),
    ("fuse_rope", fuse_rope),
    ("fuse_rope_into_kv_cache_update", fuse_rope_into_kv_cache_update),
    ("fuse_residual_epilogue", fuse_residual_epilogue),
    ("fuse_pointwise", fuse_pointwise),
    ("fuse_gate_up_projection", fuse_gate_up_projection),
    ("fuse_activation_epilogue", fuse_activation_epilogue),
    ("eliminate_common_subexpressions", eliminate_common_subexpressions),
    ("fuse_rms_norm_epilogue", fuse_rms_norm_epilogue),
    ("collapse_trailing_layouts", collapse_trailing_layouts),
)


def rewrite(graph: Graph, *, native_matmul: bool = False) -> Graph:
    """Run the whole pipeline over ``graph``."""

    for _, step in PIPELINE:
        if step is fuse_rms_norm_epilogue:
            graph = step(graph, native_matmul=native_matmul)
        else:
            graph = step(graph)
    return graph


__all__ = ["PIPELINE", "rewrite"]
