"""Generate the golden fixtures from the reference tree (run where it is mounted).

    python tests/golden/make_fixtures.py [/path/to/reference]

Writes, next to this file:

* ``lowered_graphs.json`` - the reference's own ``capture_fx`` + ``rewrite`` output for
  its quantized prefill/decode adapters on two toy decoders (one Qwen2-like with
  q/k/v bias and tied embeddings, one Llama-like), in a canonical form (dead
  operations dropped, values renumbered in definition order);
* ``adapter_eager_<family>.npz`` - the toy weights, a seeded prompt and what the
  reference's adapter modules compute eagerly on PyTorch CPU: prefill logits,
  per-step decode logits, greedy tokens and the final cache, following the host
  loop of ``src/aotolith/models/decoder.py:811-1087``;
* ``quantize_kat.npz`` - packed words / scales / codes of the reference packer on
  seeded matrices (including an all-zero group and a row of extreme values);
* ``quantize_int8_kat.npz`` - the same for the eight-bit packer, plus what the
  reference's torch operator ``aotolith::dequantize_i8`` returns for bf16 scales
  (``python make_fixtures.py <reference> int8`` writes only the eight-bit files);
* ``lowered_graphs_int8.json``, ``adapter_eager_int8_<family>.npz`` - the lowered graphs and
  eager outputs of the same toy decoders packed with eight bits (the weights are the ones stored
  in ``adapter_eager_<family>.npz``);
* ``adapter_eager_qwen05b_cut.npz`` - a two-layer cut of the Qwen2.5-0.5B shape (hidden 896, MLP
  4864, 14/2 heads of 64, vocabulary 151 936, group 64; weights from
  ``qwen25_05b_shaped(seed=7, layers=2)``, not stored): prompt, the reference adapters' prefill
  logits of the last prompt position, per-step decode logits (bf16 bit patterns) and greedy tokens
  (``python make_fixtures.py <reference> real`` writes only this file).

The reference package refuses to import off Apple silicon and needs MLX, so it
is loaded by path with a permissive ``mlx`` stub; only its torch/NumPy code runs.
"""

from __future__ import annotations

import json
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def load_reference(path: str) -> None:
    import transformers  # noqa: F401 - must be imported before the mlx stub exists

    package = types.ModuleType("aotolith")
    package.__path__ = [str(Path(path) / "src" / "aotolith")]
    sys.modules["aotolith"] = package

    class _Any:
        def __init__(self, name="mx"):
            self._name = name

        def __getattr__(self, key):
            return _Any(self._name + "." + key)

        def __call__(self, *args, **kwargs):
            return _Any(self._name + "()")

        def __hash__(self):
            return hash(self._name)

        def __eq__(self, other):
            return isinstance(other, _Any) and other._name == self._name

    class _Module(types.ModuleType):
        def __getattr__(self, key):
            if key.startswith("__"):
                raise AttributeError(key)
            return _Any("mx." + key)

    mlx, core = _Module("mlx"), _Module("mlx.core")
    mlx.core = core
    sys.modules["mlx"], sys.modules["mlx.core"] = mlx, core


def canonical_graph(graph) -> dict:
    """Dead-code-free, renumbered description of a lowered graph."""

    live = set(graph.outputs)
    kept = []
    for op in reversed(graph.ops):
        if any(out in live for out in op.outputs):
            kept.append(op)
            live.update(op.inputs)
    kept.reverse()
    names: dict[str, str] = {}
    for position, value in enumerate(graph.inputs):
        names[value] = f"in{position}"

    def name(value):
        if value not in names:
            names[value] = f"t{len(names)}"
        return names[value]

    def attr(value):
        if isinstance(value, tuple) and value and hasattr(value[0], "op"):
            body = []
            for item in value:
                body.append({"op": item.op, "inputs": [name(v) for v in item.inputs],
                             "outputs": [name(v) for v in item.outputs],
                             "attrs": {k: attr(v) for k, v in sorted(item.attrs.items())}})
            return body
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


FAMILIES = {
    "qwen2": dict(model_type="qwen2", seed=11),
    "llama": dict(model_type="llama", seed=12),
}
PROMPT, NEW, GROUP = 8, 6, 16


def toy(family: str):
    from aotolith_b200.models.synthetic import tiny_decoder

    return tiny_decoder(FAMILIES[family]["model_type"], seed=FAMILIES[family]["seed"])


def run_family(family: str, bits: int, dense: bool = False):
    """Lowered graphs and eager outputs of the reference's adapters for one toy decoder.

    ``dense``: the unquantised adapters (``quantize=None``) instead of the packed ones.
    """

    from torch.func import functional_call

    import aotolith.models.decoder as D
    from aotolith.capture import capture_fx
    from aotolith.passes import rewrite

    model = toy(family)
    capacity = PROMPT + NEW
    settings = dict(cache_capacity=capacity, group_size=GROUP, weight_bits=bits, require=family)
    if dense:
        prefill = D.DecoderPrefillModule(model, cache_capacity=capacity, require=family).eval()
        decode = D.DecoderDecodeModule(model, cache_capacity=capacity, require=family).eval()
    else:
        prefill = D.QuantizedDecoderPrefillModule(model, **settings).eval()
        decode = D.QuantizedDecoderDecodeModule(model, **settings).eval()

    def lowered(module, examples):
        state = {**dict(module.named_parameters(remove_duplicate=False)),
                 **dict(module.named_buffers(remove_duplicate=False))}
        names = list(state)

        def fn(*flat):
            return functional_call(module, dict(zip(names, flat[len(examples):])), flat[: len(examples)])

        return rewrite(capture_fx(fn, (*examples, *state.values()), promoted_constants=[])), names

    cfg = model.config
    cache_shape = (cfg.num_hidden_layers, 2, 1, cfg.num_key_value_heads, capacity, cfg.head_dim)
    pre_graph, pre_names = lowered(prefill, (
        torch.zeros((1, PROMPT), dtype=torch.int64), torch.arange(PROMPT)[None, :],
        torch.from_numpy(D.prefill_mask(PROMPT, PROMPT))))
    dec_graph, dec_names = lowered(decode, (
        torch.zeros((1, 1), dtype=torch.int64), torch.zeros((1, 1), dtype=torch.int64),
        torch.ones((1, 1, 1, capacity), dtype=torch.bool), torch.zeros(cache_shape, dtype=torch.bfloat16)))
    entry = {
        "prefill": canonical_graph(pre_graph), "decode": canonical_graph(dec_graph),
        "prefill_state": pre_names, "decode_state": dec_names,
    }

    # eager run of the reference adapters (the host loop of decoder.py:811-1087)
    generator = torch.Generator().manual_seed(100 + FAMILIES[family]["seed"])
    prompt = torch.randint(0, cfg.vocab_size, (1, PROMPT), generator=generator)
    with torch.no_grad():
        logits, compact = prefill(prompt, torch.arange(PROMPT)[None, :], torch.from_numpy(D.prefill_mask(PROMPT, PROMPT)))
        cache = torch.cat((torch.zeros(compact.shape[:4] + (NEW,) + compact.shape[5:], dtype=compact.dtype), compact), dim=4)
        prefill_logits = logits.float().numpy()
        token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        tokens, step_logits = [int(token)], []
        valid = PROMPT
        for _ in range(NEW - 1):
            valid += 1
            mask = (torch.arange(capacity) >= capacity - valid).reshape(1, 1, 1, capacity)
            logits, cache = decode(token, torch.tensor([[valid - 1]]), mask, cache)
            step_logits.append(logits.float().numpy())
            token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
            tokens.append(int(token))
        # a short, left-padded prompt through the same prefill module (bucket semantics)
        short = prompt[:, : PROMPT - 3]
        pad = PROMPT - short.shape[1]
        padded_logits, _ = prefill(
            torch.cat((torch.zeros((1, pad), dtype=torch.int64), short), dim=1),
            torch.cat((torch.zeros((1, pad), dtype=torch.int64), torch.arange(short.shape[1])[None, :]), dim=1),
            torch.from_numpy(D.prefill_mask(short.shape[1], PROMPT)))
    arrays = dict(prompt=prompt.numpy(), prefill_logits=prefill_logits, step_logits=np.stack(step_logits),
                  tokens=np.array(tokens), final_cache=cache.float().numpy(),
                  padded_prefill_logits=padded_logits.float().numpy())
    if bits == 4 and not dense:  # the other files reuse the weights stored beside the four-bit outputs
        arrays.update({f"w::{k}": v.detach().float().numpy() for k, v in model.state_dict().items()})
    print(family, "dense" if dense else f"{bits} bits", ": tokens", tokens)
    return entry, arrays


REAL_PROMPT, REAL_NEW, REAL_GROUP, REAL_SEED = 16, 6, 64, 7


def write_real_shape_cut() -> None:
    """Two layers of the Qwen2.5-0.5B shape through the reference's quantized adapters, eagerly."""

    import aotolith.models.decoder as D
    from aotolith_b200.models.synthetic import qwen25_05b_shaped

    model = qwen25_05b_shaped(seed=REAL_SEED, layers=2)
    capacity = REAL_PROMPT + REAL_NEW
    settings = dict(cache_capacity=capacity, group_size=REAL_GROUP, weight_bits=4, require="qwen2")
    prefill = D.QuantizedDecoderPrefillModule(model, **settings).eval()
    decode = D.QuantizedDecoderDecodeModule(model, **settings).eval()
    prompt = torch.randint(0, model.config.vocab_size, (1, REAL_PROMPT), generator=torch.Generator().manual_seed(107))
    with torch.no_grad():
        logits, compact = prefill(prompt, torch.arange(REAL_PROMPT)[None, :],
                                  torch.from_numpy(D.prefill_mask(REAL_PROMPT, REAL_PROMPT)))
        cache = torch.cat((torch.zeros(compact.shape[:4] + (REAL_NEW,) + compact.shape[5:], dtype=compact.dtype),
                           compact), dim=4)
        rows = [logits[0, -1, :]]
        token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        tokens = [int(token)]
        valid = REAL_PROMPT
        for _ in range(REAL_NEW - 1):
            valid += 1
            mask = (torch.arange(capacity) >= capacity - valid).reshape(1, 1, 1, capacity)
            logits, cache = decode(token, torch.tensor([[valid - 1]]), mask, cache)
            rows.append(logits[0, -1, :])
            token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
            tokens.append(int(token))
    stacked = torch.stack(rows)
    assert stacked.dtype == torch.bfloat16
    np.savez_compressed(
        HERE / "adapter_eager_qwen05b_cut.npz", prompt=prompt.numpy(), tokens=np.array(tokens),
        logits_bf16_bits=stacked.view(torch.int16).numpy(),
        final_cache_bf16_bits=cache.contiguous().view(torch.int16).numpy(),
        settings=np.array([REAL_PROMPT, REAL_NEW, REAL_GROUP, REAL_SEED]))
    print("qwen05b cut: tokens", tokens)


def write_int8_decoders() -> None:
    """The toy decoders packed with eight bits: the reference's lowered graphs and eager outputs."""

    graphs = {}
    for family in FAMILIES:
        graphs[family], arrays = run_family(family, 8)
        np.savez_compressed(HERE / f"adapter_eager_int8_{family}.npz", **arrays)
    (HERE / "lowered_graphs_int8.json").write_text(json.dumps(graphs, indent=1, sort_keys=True))


def write_int8_kat() -> None:
    """Known answers of the reference's eight-bit packer and of its torch unpack operator."""

    import aotolith.quantize as Q
    from aotolith.models.quantized import dequantize_i8

    rng = np.random.default_rng(8)
    mats = {}
    for tag, (rows, inner, group) in {"a": (6, 128, 64), "b": (5, 64, 16), "c": (3, 96, 32)}.items():
        weight = (rng.standard_normal((rows, inner)) * 0.05).astype(np.float32)
        weight[0, :group] = 0.0
        weight[1, :] = np.where(np.arange(inner) % 2 == 0, 1.0, -1.0) * 0.75
        packed, scales = Q.quantize_int8(weight, group)
        mats[f"{tag}_weight"], mats[f"{tag}_packed"], mats[f"{tag}_scales"] = weight, packed, scales
        mats[f"{tag}_codes"] = Q.unpack_codes_int8(packed)
        mats[f"{tag}_dequant"] = Q.dequantize_int8(packed, scales, group)
        low = dequantize_i8(torch.from_numpy(packed), torch.from_numpy(scales).bfloat16(), group)
        mats[f"{tag}_dequant_bf16"] = low.float().numpy()
        mats[f"{tag}_group"] = np.array(group)
    # every byte value once (byte k of word j is 4j + k), unpacked by the reference
    words = np.arange(256, dtype=np.uint8).view("<i4").reshape(1, 64)
    mats["all_words"] = words
    mats["all_codes"] = Q.unpack_codes_int8(words)
    np.savez_compressed(HERE / "quantize_int8_kat.npz", **mats)


def plain_llama():
    """The tiny Llama of the reference's quick start (``README.md:67-84``): fp32, seeded, and its input."""

    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    model = LlamaForCausalLM(LlamaConfig(
        vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=16)).eval()
    ids = torch.randint(0, 128, (1, 4), generator=torch.Generator().manual_seed(1))
    return model, ids


def module_state(model):
    names = [n for n, _ in model.named_parameters(remove_duplicate=False)] + [n for n, _ in model.named_buffers(remove_duplicate=False)]
    values = [v.detach() for _, v in model.named_parameters(remove_duplicate=False)]
    values += [v.detach() for _, v in model.named_buffers(remove_duplicate=False)]
    return names, values


def write_plain_llama() -> None:
    """A plain Hugging Face model through the REFERENCE's capture and rewrite (no adapter, no packing):
    the lowered graph, the input ids and the model's own logits."""

    from torch.func import functional_call

    from aotolith.capture import capture_fx
    from aotolith.compiler import _select_module_output
    from aotolith.passes import rewrite

    model, ids = plain_llama()
    names, values = module_state(model)

    def traced(tokens, *state):
        return _select_module_output(functional_call(model, dict(zip(names, state)), (tokens,), {}), None)

    constants: list = []
    graph = capture_fx(traced, [ids, *values], promoted_constants=constants)
    lowered = rewrite(graph)
    with torch.no_grad():
        logits = model(ids).logits
    description = {"graph": canonical_graph(lowered), "captured_ops": len(graph.ops), "constants": len(constants),
                   "state_names": names}
    (HERE / "lowered_graph_plain_llama.json").write_text(json.dumps(description, indent=1, sort_keys=True))
    np.savez_compressed(HERE / "plain_llama_eager.npz", ids=ids.numpy(), logits=logits.numpy())
    print("plain Llama:", len(graph.ops), "captured,", len(lowered.ops), "lowered operations")


def write_dense_decoders() -> None:
    """The unquantised adapters of the reference on the same toy decoders (weights: the four-bit files)."""

    graphs = {}
    for family in FAMILIES:
        graphs[family], arrays = run_family(family, 4, dense=True)
        np.savez_compressed(HERE / f"adapter_eager_dense_{family}.npz", **arrays)
    (HERE / "lowered_graphs_dense.json").write_text(json.dumps(graphs, indent=1, sort_keys=True))


def main(reference: str, only: str | None = None) -> None:
    load_reference(reference)
    if only == "dense":
        write_dense_decoders()
        return
    if only == "plain":
        write_plain_llama()
        return
    if only == "real":
        write_real_shape_cut()
        return
    if only == "int8":
        write_int8_kat()
        write_int8_decoders()
        print("int8 fixtures written to", HERE)
        return
    import aotolith.quantize as Q

    graphs = {}
    for family in FAMILIES:
        graphs[family], arrays = run_family(family, 4)
        np.savez_compressed(HERE / f"adapter_eager_{family}.npz", **arrays)
    (HERE / "lowered_graphs.json").write_text(json.dumps(graphs, indent=1, sort_keys=True))

    rng = np.random.default_rng(5)
    mats = {}
    for tag, (rows, inner, group) in {"a": (6, 128, 64), "b": (5, 64, 16), "c": (3, 96, 32)}.items():
        weight = (rng.standard_normal((rows, inner)) * 0.05).astype(np.float32)
        weight[0, :group] = 0.0
        weight[1, :] = np.where(np.arange(inner) % 2 == 0, 1.0, -1.0) * 0.75
        packed, scales = Q.quantize_int4(weight, group)
        mats[f"{tag}_weight"], mats[f"{tag}_packed"], mats[f"{tag}_scales"] = weight, packed, scales
        mats[f"{tag}_codes"] = Q.unpack_codes(packed)
        mats[f"{tag}_dequant"] = Q.dequantize_int4(packed, scales, group)
        mats[f"{tag}_group"] = np.array(group)
    np.savez_compressed(HERE / "quantize_kat.npz", **mats)
    write_int8_kat()
    write_int8_decoders()
    write_real_shape_cut()
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: python make_fixtures.py <path of a checkout of the reference project> [int8|real|plain|dense]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
