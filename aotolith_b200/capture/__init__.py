"""FX capture: trace a callable with fake tensors and lower the ATen graph to IR.

``capture_fx(fn, example_inputs, promoted_constants=None) -> Graph`` is the
front door of the compiler (reference: ``src/aotolith/capture/__init__.py:30-48``).
Tracing is shape-only (``make_fx(tracing_mode="fake")``), so capturing a
multi-gigabyte model costs no arithmetic.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from typing import Any

from ..errors import PlatformError
from ..ir import Graph
from .legalize import legalize


def trace(fn: Callable[..., Any], example_inputs: Sequence[Any]):
    """``make_fx`` under fake tensors; returns the ``fx.GraphModule``."""

    try:
        from torch.fx.experimental.proxy_tensor import make_fx
    except ImportError as error:  # pragma: no cover - torch is a hard dependency here
        raise PlatformError("PyTorch is required for the FX frontend") from error
    return make_fx(fn, tracing_mode="fake")(*example_inputs)


def capture_fx(
    fn: Callable[..., Any],
    example_inputs: Sequence[Any],
    promoted_constants: list[Any] | None = None,
) -> Graph:
    """Trace ``fn`` on ``example_inputs`` and return the captured IR graph.

    Graph inputs are ``arg0..argN`` in placeholder order. A tensor the trace
    captured as a constant is refused unless ``promoted_constants`` is a list,
    in which case it becomes one more graph input and its value is appended to
    that list.
    """

    graph = legalize(trace(fn, example_inputs), promoted_constants)
    graph.validate()
    return graph


__all__ = ["capture_fx", "legalize", "trace"]
