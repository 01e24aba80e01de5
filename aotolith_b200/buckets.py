"""Sharing one copy of the weights across plans compiled from the same module.

Every bucket (and the prefill/decode pair of one bucket) traces the same module,
so a naive set of plans holds one copy of the weights each. ``share_plan_state``
rebinds state entries with the same name, shape, dtype and contents to one
device tensor; entries that genuinely differ (the rotary tables of buckets with
different capacities) are kept. Reference: ``src/aotolith/buckets.py:183-216``.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import replace

import torch

from .compiler import CompiledModulePlan


def _same(left: torch.Tensor, right: torch.Tensor) -> bool:
    if left is right:
        return True
    if left.shape != right.shape or left.dtype != right.dtype or left.device != right.device:
        return False
    return bool(torch.equal(left, right))


def share_plan_state(plans: Sequence[CompiledModulePlan]) -> list[CompiledModulePlan]:
    if len(plans) < 2:
        return list(plans)
    canonical: dict[str, list[torch.Tensor]] = {}
    for name, value in zip(plans[0].state_names, plans[0]._state_values):
        canonical.setdefault(name, []).append(value)
    shared = [plans[0]]
    for plan in plans[1:]:
        values = list(plan._state_values)
        changed = False
        for index, name in enumerate(plan.state_names):
            candidates = canonical.setdefault(name, [])
            for candidate in candidates:
                if _same(values[index], candidate):
                    if values[index] is not candidate:
                        values[index] = candidate
                        changed = True
                    break
            else:
                candidates.append(values[index])
        shared.append(replace(plan, _state_values=tuple(values)) if changed else plan)
    return shared
