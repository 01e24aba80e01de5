"""Loading the committed golden fixtures."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
PROMPT, NEW, GROUP = 8, 6, 16


def lowered_graphs() -> dict:
    return json.loads((GOLDEN / "lowered_graphs.json").read_text())


def eager_fixture(family: str):
    """``(model, arrays)``: the toy decoder rebuilt from the stored weights and the reference outputs."""

    from aotolith_b200.models.synthetic import tiny_decoder

    data = np.load(GOLDEN / f"adapter_eager_{family}.npz")
    model = tiny_decoder(family, seed=0)
    state = model.state_dict()
    for key in state:
        stored = torch.from_numpy(data[f"w::{key}"])
        state[key].copy_(stored.to(state[key].dtype))
    return model, data


def canonical_graph(graph) -> dict:
    """Same canonical form as ``tests/golden/make_fixtures.py`` writes."""

    live = set(graph.outputs)
    kept = []
    for op in reversed(graph.ops):
        if any(out in live for out in op.outputs):
            kept.append(op)
            live.update(op.inputs)
    kept.reverse()
    names: dict[str, str] = {v: f"in{i}" for i, v in enumerate(graph.inputs)}

    def name(value):
        if value not in names:
            names[value] = f"t{len(names)}"
        return names[value]

    def attr(value):
        if isinstance(value, tuple) and value and hasattr(value[0], "op"):
            return [
                {"op": item.op, "inputs": [name(v) for v in item.inputs],
                 "outputs": [name(v) for v in item.outputs],
                 "attrs": {k: attr(v) for k, v in sorted(item.attrs.items())}}
                for item in value
            ]
        if isinstance(value, tuple):
            return [attr(v) for v in value]
        if isinstance(value, float) and value in (float("inf"), float("-inf")):
            return "inf" if value > 0 else "-inf"
        return value

    ops = []
    for op in kept:
        inputs = [name(v) for v in op.inputs]
        ops.append({
            "op": op.op,
            "inputs": inputs,
            "input_types": [[list(graph.value(v).type.shape), graph.value(v).type.dtype.value] for v in op.inputs],
            "attrs": {k: attr(v) for k, v in sorted(op.attrs.items())},
            "outputs": [name(v) for v in op.outputs],
            "output_types": [[list(graph.value(v).type.shape), graph.value(v).type.dtype.value] for v in op.outputs],
        })
    return {"inputs": len(graph.inputs), "ops": ops, "outputs": [name(v) for v in graph.outputs]}


def real_shape_fixture():
    """``(model, arrays)`` of the two-layer cut of the Qwen2.5-0.5B shape (weights from the seed)."""

    from aotolith_b200.models.synthetic import qwen25_05b_shaped

    data = dict(np.load(GOLDEN / "adapter_eager_qwen05b_cut.npz"))
    prompt_length, new_tokens, group, seed = (int(v) for v in data["settings"])
    model = qwen25_05b_shaped(seed=seed, layers=2)
    data["logits"] = torch.from_numpy(data["logits_bf16_bits"]).view(torch.bfloat16).float()
    data["final_cache"] = torch.from_numpy(data["final_cache_bf16_bits"]).view(torch.bfloat16).float()
    data.update(prompt_length=prompt_length, new_tokens=new_tokens, group=group)
    return model, data
