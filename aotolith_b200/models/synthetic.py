"""Random-init decoders with the HuggingFace module tree, for shapes without a checkpoint.

``SyntheticDecoder`` has exactly the attributes the static-cache adapter reads
(``config``, ``model.embed_tokens``, ``model.layers[i].self_attn.{q,k,v,o}_proj``,
``.mlp.{gate,up,down}_proj``, ``.mlp.act_fn``, ``.input_layernorm``,
``.post_attention_layernorm``, ``model.norm``, ``lm_head``) and nothing else: it
is a weight container, not a forward pass. Benchmarks and tests use it for the
Qwen2.5-0.5B and Llama-3-8B shapes, seeded, with N(0, 0.02) weights.
"""

from __future__ import annotations

from types import SimpleNamespace

import torch
from torch import nn


class _Norm(nn.Module):
    def __init__(self, width: int, dtype: torch.dtype) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=dtype), requires_grad=False)


def _linear(out_features: int, in_features: int, bias: bool, dtype, generator, std: float) -> nn.Linear:
    device = generator.device
    layer = nn.Linear(in_features, out_features, bias=bias, dtype=dtype, device="meta")
    layer = layer.to_empty(device=device)
    with torch.no_grad():
        layer.weight.copy_(torch.randn(out_features, in_features, generator=generator, dtype=torch.float32, device=device) * std)
        if bias:
            layer.bias.copy_(torch.randn(out_features, generator=generator, dtype=torch.float32, device=device) * 0.5)
    layer.weight.requires_grad_(False)
    if bias:
        layer.bias.requires_grad_(False)
    return layer


class SyntheticDecoder(nn.Module):
    def __init__(
        self,
        *,
        model_type: str,
        vocab_size: int,
        hidden_size: int,
        intermediate_size: int,
        num_hidden_layers: int,
        num_attention_heads: int,
        num_key_value_heads: int,
        head_dim: int | None = None,
        max_position_embeddings: int = 4096,
        rope_theta: float = 10000.0,
        rms_norm_eps: float = 1e-6,
        attention_bias: bool = False,
        tie_word_embeddings: bool = False,
        dtype: torch.dtype = torch.bfloat16,
        seed: int = 0,
        std: float = 0.02,
        device: str | torch.device = "cpu",
    ) -> None:
        """``device``: where the weights are drawn and kept. A model of billions of parameters is
        built in seconds on a GPU (and minutes on the host); the values depend on the device kind
        (each has its own generator) and are the same on every GPU of one kind for one seed."""

        super().__init__()
        device = torch.device(device)
        head_dim = head_dim or hidden_size // num_attention_heads
        self.config = SimpleNamespace(
            model_type=model_type, vocab_size=vocab_size, hidden_size=hidden_size,
            intermediate_size=intermediate_size, num_hidden_layers=num_hidden_layers,
            num_attention_heads=num_attention_heads, num_key_value_heads=num_key_value_heads,
            head_dim=head_dim, max_position_embeddings=max_position_embeddings,
            rope_theta=rope_theta, rope_scaling=None, rms_norm_eps=rms_norm_eps,
            hidden_act="silu", layer_types=None, tie_word_embeddings=tie_word_embeddings,
        )
        generator = torch.Generator(device=device).manual_seed(seed)
        make = lambda o, i, b=False: _linear(o, i, b, dtype, generator, std)
        self.model = nn.Module()
        self.model.embed_tokens = nn.Embedding(vocab_size, hidden_size, dtype=dtype, device=device)
        with torch.no_grad():
            self.model.embed_tokens.weight.copy_(
                torch.randn(vocab_size, hidden_size, generator=generator, dtype=torch.float32, device=device) * std
            )
        self.model.embed_tokens.weight.requires_grad_(False)
        layers = []
        for _ in range(num_hidden_layers):
            layer = nn.Module()
            layer.self_attn = nn.Module()
            layer.self_attn.q_proj = make(num_attention_heads * head_dim, hidden_size, attention_bias)
            layer.self_attn.k_proj = make(num_key_value_heads * head_dim, hidden_size, attention_bias)
            layer.self_attn.v_proj = make(num_key_value_heads * head_dim, hidden_size, attention_bias)
            layer.self_attn.o_proj = make(hidden_size, num_attention_heads * head_dim)
            layer.mlp = nn.Module()
            layer.mlp.gate_proj = make(intermediate_size, hidden_size)
            layer.mlp.up_proj = make(intermediate_size, hidden_size)
            layer.mlp.down_proj = make(hidden_size, intermediate_size)
            layer.mlp.act_fn = nn.SiLU()
            layer.input_layernorm = _Norm(hidden_size, dtype).to(device)
            layer.post_attention_layernorm = _Norm(hidden_size, dtype).to(device)
            with torch.no_grad():
                for norm in (layer.input_layernorm, layer.post_attention_layernorm):
                    norm.weight.add_(torch.randn(hidden_size, generator=generator, device=device) * 0.05)
            layers.append(layer)
        self.model.layers = nn.ModuleList(layers)
        self.model.norm = _Norm(hidden_size, dtype).to(device)
        self.lm_head = nn.Linear(hidden_size, vocab_size, bias=False, dtype=dtype, device="meta").to_empty(device=device)
        self.lm_head.weight.requires_grad_(False)
        if tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        else:
            with torch.no_grad():
                self.lm_head.weight.copy_(
                    torch.randn(vocab_size, hidden_size, generator=generator, dtype=torch.float32, device=device) * std
                )
        self.eval()


def qwen25_05b_shaped(seed: int = 0, *, layers: int = 24, max_position_embeddings: int = 32768,
                      device: str | torch.device = "cpu") -> SyntheticDecoder:
    """Qwen2.5-0.5B shapes: hidden 896, MLP 4864, 24 layers, 14/2 heads, dim 64, vocab 151936."""

    return SyntheticDecoder(
        model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
        num_hidden_layers=layers, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
        max_position_embeddings=max_position_embeddings, rope_theta=1e6, rms_norm_eps=1e-6,
        attention_bias=True, tie_word_embeddings=True, seed=seed, device=device,
    )


def llama3_8b_shaped(seed: int = 0, *, layers: int = 32, max_position_embeddings: int = 8192,
                     device: str | torch.device = "cpu") -> SyntheticDecoder:
    """Llama-3-8B shapes: hidden 4096, MLP 14336, 32 layers, 32/8 heads, dim 128, vocab 128256."""

    return SyntheticDecoder(
        model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
        num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        max_position_embeddings=max_position_embeddings, rope_theta=5e5, rms_norm_eps=1e-5,
        attention_bias=False, tie_word_embeddings=False, seed=seed, device=device,
    )


def tiny_decoder(model_type: str = "qwen2", seed: int = 0, **overrides) -> SyntheticDecoder:
    """A two-layer toy (hidden 64) for fast tests."""

    settings = dict(
        model_type=model_type, vocab_size=128, hidden_size=64, intermediate_size=128,
        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        max_position_embeddings=64, rope_theta=1e6 if model_type == "qwen2" else 5e5,
        attention_bias=model_type == "qwen2", tie_word_embeddings=model_type == "qwen2",
        seed=seed, std=0.08,
    )
    settings.update(overrides)
    return SyntheticDecoder(**settings)
