"""The torch modules that are traced into the prefill and decode graphs.

A HuggingFace-style decoder (``model.model.layers[i].self_attn.{q,k,v,o}_proj``,
``.mlp.{gate,up,down}_proj``, ``.input_layernorm``,
``.post_attention_layernorm``, ``model.model.norm``,
``model.model.embed_tokens``, ``model.lm_head``) is re-expressed with an
explicit static KV cache:

* prefill: ``input_ids[1,P], positions[1,P], mask[1,1,P,P] bool`` ->
  ``logits[1,1,V], cache[L,2,1,KVH,P,D]``
* decode: ``token[1,1], position[1,1], mask[1,1,1,C] bool,
  cache[L,2,1,KVH,C,D]`` -> ``logits[1,1,V], cache[L,2,1,KVH,C,D]``

The decode cache is a rolling window: every step drops slot 0 and appends the
new (rotated key, value) at slot ``C-1``. Query, key and value share one packed
projection per layer. These are the semantics of the reference adapters
(``src/aotolith/models/decoder.py:282-737``); the state the modules register -
and therefore the compiled plans' state names - follows the reference's
quantized adapter (``embed_tokens_weight``, ``final_norm``,
``lm_head_0_packed/_scales``, ``qkv_{i}_packed/_scales``, ``qkv_bias_{i}``,
``input_norm_{i}``, ``post_attention_norm_{i}``,
``{o,gate,up,down}_proj_{i}_packed/_scales``, ``cosine_table``,
``sine_table``; ``decoder.py:640-698``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..errors import UnsupportedModelError
from .quantized import dequantize_i4, dequantize_i8, pack_weight


@dataclass(frozen=True, slots=True)
class DecoderFamily:
    """A decoder family whose module tree and causal masking were checked."""

    name: str
    model_types: tuple[str, ...]
    label: str


FAMILIES: tuple[DecoderFamily, ...] = (
    DecoderFamily("qwen2", ("qwen2",), "Qwen2/Qwen2.5"),
    DecoderFamily("llama", ("llama",), "Llama"),
)

_BY_MODEL_TYPE = {kind: family for family in FAMILIES for kind in family.model_types}


def family_for(model: torch.nn.Module, *, require: str | None = None) -> DecoderFamily:
    """The family of ``model``; refuses unknown families and a mismatch with ``require``."""

    model_type = getattr(model.config, "model_type", None)
    family = _BY_MODEL_TYPE.get(str(model_type))
    if family is None:
        covered = ", ".join(f"{item.label} ({'/'.join(item.model_types)})" for item in FAMILIES)
        raise UnsupportedModelError(
            f"the static-cache adapter does not cover model_type {model_type!r}; it covers {covered}",
            hint="compile a plain forward pass with compile_module instead",
        )
    if require is not None and family.name != require:
        raise UnsupportedModelError(
            f"this entry point compiles {require} and the model is {family.label} ({model_type!r})",
            hint=f"call compile_{family.name}_static_cache instead",
        )
    return family


def _rope_settings(config) -> tuple[float, bool]:
    """``(theta, scaled)`` from either config generation.

    Older configs carry ``rope_theta`` and ``rope_scaling`` (``None`` when the
    table is the plain one); newer ones carry a ``rope_parameters`` mapping with
    ``rope_theta`` and ``rope_type`` (``"default"`` when plain).
    """

    parameters = getattr(config, "rope_parameters", None)
    if isinstance(parameters, dict):
        theta = float(parameters.get("rope_theta", getattr(config, "rope_theta", None) or 10000.0))
        kind = parameters.get("rope_type", parameters.get("type", "default"))
        return theta, kind not in (None, "default")
    scaling = getattr(config, "rope_scaling", None)
    scaled = scaling is not None
    if isinstance(scaling, dict):
        scaled = scaling.get("rope_type", scaling.get("type", "default")) not in (None, "default")
    return float(getattr(config, "rope_theta", None) or 10000.0), scaled


def _check_attention_is_causal_only(model: torch.nn.Module) -> None:
    message = (
        "sliding-window attention is not supported: the static-cache adapter builds a "
        "plain causal mask for every layer"
    )
    kinds = getattr(model.config, "layer_types", None)
    if getattr(model.model, "has_sliding_layers", False) or (
        isinstance(kinds, (list, tuple)) and any(kind == "sliding_attention" for kind in kinds)
    ):
        raise UnsupportedModelError(message, hint="compile the model as a plain module")


def _check_activation(model: torch.nn.Module) -> None:
    """The gated MLP's activation must be SiLU, the one the epilogue kernels implement."""

    probe = torch.tensor((0.25, -0.75, 1.5, -2.5, 3.0, -6.0), dtype=torch.float32)
    for index, layer in enumerate(model.model.layers):
        activation = getattr(layer.mlp, "act_fn", None)
        if activation is None:
            raise UnsupportedModelError(
                f"layer {index} has no mlp.act_fn; the static-cache adapter requires a gated MLP",
                hint="compile the model as a plain module with compile_module",
            )
        try:
            matches = torch.allclose(activation(probe), F.silu(probe), atol=1e-6, rtol=1e-6)
        except Exception as error:  # noqa: BLE001
            raise UnsupportedModelError(
                f"the MLP activation {type(activation).__name__} of layer {index} cannot be "
                f"evaluated on a probe: {error}"
            ) from error
        if not matches:
            name = getattr(model.config, "hidden_act", "<unknown>")
            raise UnsupportedModelError(
                f"the cuda-sm100 target lowers the SiLU gated MLP only; layer {index} uses "
                f"{type(activation).__name__} (config hidden_act {name!r})",
                hint="pick a checkpoint whose hidden_act is 'silu'",
            )


def _packed_qkv_bias(attention: torch.nn.Module, family: DecoderFamily) -> torch.Tensor | None:
    parts = (attention.q_proj.bias, attention.k_proj.bias, attention.v_proj.bias)
    if all(part is None for part in parts):
        return None
    if any(part is None for part in parts):
        raise UnsupportedModelError(
            f"the {family.label} attention has a bias on some of q/k/v and not others, which "
            "cannot be packed into one projection",
            hint="a checkpoint needs all three biases or none of them",
        )
    return torch.cat(parts, dim=0).detach()


def rotary_tables(capacity: int, head_dim: int, theta: float, dtype: torch.dtype):
    """``(cos, sin)`` tables ``[capacity, head_dim]``.

    Angles are computed in fp32, duplicated over the two halves and cast to the
    model dtype BEFORE the cosine and sine are taken
    (``src/aotolith/models/decoder.py:323-334``).
    """

    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32)[None, :] / head_dim
    angles = torch.arange(capacity, dtype=torch.float32)[:, None] / torch.pow(
        torch.tensor(theta, dtype=torch.float32), exponent
    )
    angles = torch.cat((angles, angles), dim=-1).to(dtype)
    return angles.cos(), angles.sin()


def _rotate_half(value: torch.Tensor) -> torch.Tensor:
    half = value.shape[-1] // 2
    return torch.cat((-value[..., half:], value[..., :half]), dim=-1)


def _rotary(value: torch.Tensor, cosine: torch.Tensor, sine: torch.Tensor) -> torch.Tensor:
    return value * cosine + _rotate_half(value) * sine


_PER_LAYER = (("o_proj", "self_attn"), ("gate_proj", "mlp"), ("up_proj", "mlp"), ("down_proj", "mlp"))


class _QuantizedDecoder(torch.nn.Module):
    """Weights of a decoder, packed to 4 or 8 bits, plus the shared forward pieces."""

    def __init__(
        self,
        model: torch.nn.Module,
        *,
        cache_capacity: int,
        group_size: int,
        weight_bits: int = 4,
        require: str | None = None,
        packed_from: "_QuantizedDecoder | None" = None,
    ) -> None:
        super().__init__()
        config = model.config
        self.family = family_for(model, require=require)
        theta, scaled = _rope_settings(config)
        if scaled:
            raise UnsupportedModelError(
                f"{self.family.label} RoPE scaling is not supported yet",
                hint="the adapter builds one rotary table from rope_theta",
            )
        if weight_bits not in (4, 8):
            raise UnsupportedModelError(
                f"the cuda-sm100 target packs 4- or 8-bit weights, got weight_bits={weight_bits}"
            )
        _check_activation(model)
        _check_attention_is_causal_only(model)
        self.cache_capacity = int(cache_capacity)
        self.group_size = int(group_size)
        self.weight_bits = int(weight_bits)
        self.hidden_size = int(config.hidden_size)
        self.num_layers = int(config.num_hidden_layers)
        self.num_heads = int(config.num_attention_heads)
        self.num_key_value_heads = int(config.num_key_value_heads)
        self.head_dim = int(getattr(config, "head_dim", None) or self.hidden_size // self.num_heads)
        self.rms_norm_eps = float(config.rms_norm_eps)
        self.rope_theta = theta
        dtype = next(model.parameters()).dtype
        cosine, sine = rotary_tables(self.cache_capacity, self.head_dim, theta, dtype)
        self.register_buffer("cosine_table", cosine, persistent=False)
        self.register_buffer("sine_table", sine, persistent=False)
        if (isinstance(packed_from, _QuantizedDecoder) and packed_from.group_size == self.group_size
                and packed_from.weight_bits == self.weight_bits):
            # Packing is the expensive part of construction and does not depend on the
            # capacity: adopt the buffers another adapter of the same model already packed.
            for name, tensor in packed_from.named_buffers():
                if name not in ("cosine_table", "sine_table"):
                    self.register_buffer(name, tensor, persistent=False)
        else:
            self._pack(model, dtype)

    def _pack(self, model: torch.nn.Module, dtype: torch.dtype) -> None:
        def keep(name: str, tensor: torch.Tensor) -> None:
            self.register_buffer(name, tensor.detach(), persistent=False)

        def pack(name: str, weight: torch.Tensor) -> None:
            words, scales = pack_weight(weight, self.group_size, self.weight_bits)
            keep(f"{name}_packed", words)
            keep(f"{name}_scales", scales.to(dtype).contiguous())

        keep("embed_tokens_weight", model.model.embed_tokens.weight)
        keep("final_norm", model.model.norm.weight)
        if getattr(model.lm_head, "bias", None) is not None:
            raise UnsupportedModelError("packed compilation cannot pack an lm_head bias")
        pack("lm_head_0", model.lm_head.weight)
        for index, layer in enumerate(model.model.layers):
            attention = layer.self_attn
            pack(
                f"qkv_{index}",
                torch.cat((attention.q_proj.weight, attention.k_proj.weight, attention.v_proj.weight), dim=0),
            )
            bias = _packed_qkv_bias(attention, self.family)
            if bias is not None:
                keep(f"qkv_bias_{index}", bias)
            keep(f"input_norm_{index}", layer.input_layernorm.weight)
            keep(f"post_attention_norm_{index}", layer.post_attention_layernorm.weight)
            for name, owner in _PER_LAYER:
                projection = getattr(getattr(layer, owner), name)
                if projection.bias is not None:
                    raise UnsupportedModelError(
                        f"packed compilation cannot pack the {name} bias of the {self.family.label} adapter",
                        hint="the quantized plan holds only the packed q/k/v bias",
                    )
                pack(f"{name}_{index}", projection.weight)

    # -- shared forward pieces -------------------------------------------------

    def _weight(self, name: str, index: int) -> torch.Tensor:
        unpack = dequantize_i8 if self.weight_bits == 8 else dequantize_i4
        return unpack(
            self.get_buffer(f"{name}_{index}_packed"),
            self.get_buffer(f"{name}_{index}_scales"),
            self.group_size,
        )

    def _norm(self, hidden: torch.Tensor, name: str) -> torch.Tensor:
        return F.rms_norm(hidden, (hidden.shape[-1],), self.get_buffer(name), self.rms_norm_eps)

    def _qkv(self, hidden: torch.Tensor, positions: torch.Tensor, index: int):
        projected = F.linear(
            self._norm(hidden, f"input_norm_{index}"),
            self._weight("qkv", index),
            self._buffers.get(f"qkv_bias_{index}"),
        )
        heads, kv_heads, dim = self.num_heads, self.num_key_value_heads, self.head_dim
        query, key, value = projected.split((heads * dim, kv_heads * dim, kv_heads * dim), dim=-1)
        batch, steps = hidden.shape[:2]
        query = query.reshape(batch, steps, heads, dim).transpose(1, 2)
        key = key.reshape(batch, steps, kv_heads, dim).transpose(1, 2)
        value = value.reshape(batch, steps, kv_heads, dim).transpose(1, 2)
        cosine = F.embedding(positions, self.cosine_table)[:, None, :, :]
        sine = F.embedding(positions, self.sine_table)[:, None, :, :]
        return _rotary(query, cosine, sine), _rotary(key, cosine, sine), value

    def _mlp_and_residuals(self, hidden: torch.Tensor, attended: torch.Tensor, index: int) -> torch.Tensor:
        batch, steps = hidden.shape[:2]
        attended = attended.transpose(1, 2).reshape(batch, steps, self.num_heads * self.head_dim)
        hidden = hidden + F.linear(attended, self._weight("o_proj", index))
        normalized = self._norm(hidden, f"post_attention_norm_{index}")
        gate = F.linear(normalized, self._weight("gate_proj", index))
        up = F.linear(normalized, self._weight("up_proj", index))
        return hidden + F.linear(F.silu(gate) * up, self._weight("down_proj", index))

    def _logits(self, hidden: torch.Tensor) -> torch.Tensor:
        hidden = self._norm(hidden, "final_norm")[:, -1:, :]
        return F.linear(hidden, self._weight("lm_head", 0))


class QuantizedDecoderPrefillModule(_QuantizedDecoder):
    """A fixed-length prompt pass that also emits the compact per-layer KV cache."""

    def forward(self, input_ids, positions, attention_mask):
        hidden = F.embedding(input_ids, self.embed_tokens_weight)
        kept: list[torch.Tensor] = []
        for index in range(self.num_layers):
            query, key, value = self._qkv(hidden, positions, index)
            attended = F.scaled_dot_product_attention(
                query, key, value, attn_mask=attention_mask, enable_gqa=True
            )
            hidden = self._mlp_and_residuals(hidden, attended, index)
            kept.extend((key, value))
        cache = torch.stack(kept, dim=0).reshape(
            self.num_layers, 2, input_ids.shape[0], self.num_key_value_heads,
            input_ids.shape[1], self.head_dim,
        )
        return self._logits(hidden), cache


class QuantizedDecoderDecodeModule(_QuantizedDecoder):
    """One token against a fixed-capacity rolling KV cache."""

    def forward(self, input_ids, positions, attention_mask, cache):
        hidden = F.embedding(input_ids, self.embed_tokens_weight)
        pairs: list[torch.Tensor] = []
        for index in range(self.num_layers):
            query, key, value = self._qkv(hidden, positions, index)
            pair = torch.cat(
                (cache[index, :, :, :, 1:, :], torch.stack((key, value), dim=0)), dim=3
            )
            attended = F.scaled_dot_product_attention(
                query, pair[0], pair[1], attn_mask=attention_mask, enable_gqa=True
            )
            hidden = self._mlp_and_residuals(hidden, attended, index)
            pairs.append(pair)
        next_cache = torch.stack(pairs, dim=0).reshape(
            self.num_layers, 2, input_ids.shape[0], self.num_key_value_heads,
            self.cache_capacity, self.head_dim,
        )
        return self._logits(hidden), next_cache


class QuantizedDecoderRowsModule(_QuantizedDecoder):
    """``m`` tokens in one step against the rolling cache, with the logits of every row.

    The plan shape the reference names as its next step and does not ship
    (``docs/host-runtime.md:186-208``: token and position inputs ``[m]`` wide, a mask of ``m``
    rows, ``m`` rows of logits for a host that verifies proposed tokens). The window moves by
    ``m`` slots; everything else is the one-token step (``models/decoder.py:586-633``).
    """

    def forward(self, input_ids, positions, attention_mask, cache):
        rows = input_ids.shape[1]
        hidden = F.embedding(input_ids, self.embed_tokens_weight)
        pairs: list[torch.Tensor] = []
        for index in range(self.num_layers):
            query, key, value = self._qkv(hidden, positions, index)
            pair = torch.cat(
                (cache[index, :, :, :, rows:, :], torch.stack((key, value), dim=0)), dim=3
            )
            attended = F.scaled_dot_product_attention(
                query, pair[0], pair[1], attn_mask=attention_mask, enable_gqa=True
            )
            hidden = self._mlp_and_residuals(hidden, attended, index)
            pairs.append(pair)
        next_cache = torch.stack(pairs, dim=0).reshape(
            self.num_layers, 2, input_ids.shape[0], self.num_key_value_heads,
            self.cache_capacity, self.head_dim,
        )
        return F.linear(self._norm(hidden, "final_norm"), self._weight("lm_head", 0)), next_cache


# ---------------------------------------------------------------------------
# dense (unquantised) adapters
# ---------------------------------------------------------------------------

class _DenseDecoder(_QuantizedDecoder):
    """The same forward pieces over the model's own bf16 weights.

    Follows the dense adapter of the reference (``src/aotolith/models/decoder.py:282-420``): the
    adapter keeps the model as a submodule, so the plan's state carries the model's own tensor
    names; only the per-layer q/k/v weights (and biases) are concatenated once into
    ``qkv_weight_{i}`` / ``qkv_bias_{i}`` buffers, registered after the rotary tables.
    """

    def __init__(self, model: torch.nn.Module, *, cache_capacity: int, require: str | None = None) -> None:
        super().__init__(model, cache_capacity=cache_capacity, group_size=0, weight_bits=4, require=require)

    def _pack(self, model: torch.nn.Module, dtype: torch.dtype) -> None:
        self.model = model
        for index, layer in enumerate(model.model.layers):
            attention = layer.self_attn
            self.register_buffer(
                f"qkv_weight_{index}",
                torch.cat((attention.q_proj.weight, attention.k_proj.weight, attention.v_proj.weight), dim=0).detach(),
                persistent=False,
            )
            bias = _packed_qkv_bias(attention, self.family)
            if bias is not None:
                self.register_buffer(f"qkv_bias_{index}", bias, persistent=False)
            for name, owner in _PER_LAYER:
                if getattr(getattr(layer, owner), name).bias is not None:
                    raise UnsupportedModelError(
                        f"the {name} bias of the {self.family.label} adapter has no place in the decoder graphs")

    @property
    def embed_tokens_weight(self) -> torch.Tensor:
        return self.model.model.embed_tokens.weight

    def _weight(self, name: str, index: int) -> torch.Tensor:
        if name == "qkv":
            return self.get_buffer(f"qkv_weight_{index}")
        if name == "lm_head":
            return self.model.lm_head.weight
        owner = dict(_PER_LAYER)[name]
        return getattr(getattr(self.model.model.layers[index], owner), name).weight

    def _norm(self, hidden: torch.Tensor, name: str) -> torch.Tensor:
        if name == "final_norm":
            weight = self.model.model.norm.weight
        else:
            kind, _, index = name.rpartition("_")
            layer = self.model.model.layers[int(index)]
            weight = layer.input_layernorm.weight if kind == "input_norm" else layer.post_attention_layernorm.weight
        return F.rms_norm(hidden, (hidden.shape[-1],), weight, self.rms_norm_eps)


class DecoderPrefillModule(_DenseDecoder, QuantizedDecoderPrefillModule):
    """Dense prompt pass (``quantize=None``)."""


class DecoderDecodeModule(_DenseDecoder, QuantizedDecoderDecodeModule):
    """Dense decode step (``quantize=None``)."""


class DecoderRowsModule(_DenseDecoder, QuantizedDecoderRowsModule):
    """Dense step over ``m`` tokens (``quantize=None``)."""
