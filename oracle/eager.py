"""The adapter modules run eagerly on the CPU: the timed CPU arm of the benchmark.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The reference's own CPU execution of this path is its torch adapter modules
evaluated eagerly by PyTorch (``src/aotolith/models/decoder.py:524-737`` with
the eager ``dequantize_i4`` of ``models/quantized.py:61-76``). The reference
tree cannot travel to the benchmark machine, so the same computation is run
from this repository's adapter modules (same operations in the same order) with
a CPU implementation of the unpack operator registered here - the shipped
package registers none.
"""

from __future__ import annotations

import time

import torch

from . import ops_ref

_registered = False


def register_cpu_dequantize() -> None:
    global _registered
    if _registered:
        return
    from aotolith_b200.models import quantized

    quantized._register()

    @torch.library.impl(quantized.DEQUANTIZE_I4, "CPU")
    def _dequantize_cpu(packed, scales, group_size):
        return ops_ref.dequantize_i4(packed, scales, group_size)

    _registered = True


class EagerCpuDecoder:
    """Prefill + greedy decode of a decoder on the host cores, bf16, batch 1."""

    def __init__(self, model, prompt_length: int, max_new_tokens: int, group_size: int) -> None:
        from aotolith_b200.models.adapters import QuantizedDecoderDecodeModule, QuantizedDecoderPrefillModule
        from aotolith_b200.models.decoder import prefill_mask

        register_cpu_dequantize()
        self.prompt_length, self.capacity = prompt_length, prompt_length + max_new_tokens
        settings = dict(cache_capacity=self.capacity, group_size=group_size)
        self.prefill = QuantizedDecoderPrefillModule(model, **settings).eval()
        self.decode = QuantizedDecoderDecodeModule(model, packed_from=self.prefill, **settings).eval()
        self.mask = torch.from_numpy(prefill_mask(prompt_length, prompt_length))

    @torch.no_grad()
    def start(self, prompt) -> float:
        """Prefill ``prompt`` and keep the padded cache; returns the prefill seconds."""

        prompt = torch.as_tensor(prompt, dtype=torch.int64).reshape(1, -1)
        begin = time.perf_counter()
        logits, compact = self.prefill(prompt, torch.arange(self.prompt_length)[None, :], self.mask)
        pad = torch.zeros(compact.shape[:4] + (self.capacity - self.prompt_length,) + compact.shape[5:], dtype=compact.dtype)
        self._first_cache = torch.cat((pad, compact), dim=4)
        self._first_token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        self.rewind()
        return time.perf_counter() - begin

    def rewind(self) -> None:
        """Back to the state right after the prefill."""

        self.cache, self.token, self.valid = self._first_cache, self._first_token, self.prompt_length
        self.tokens = [int(self.token)]

    @torch.no_grad()
    def step(self) -> float:
        """One greedy decode step on the host; returns its seconds."""

        if self.valid + 1 >= self.capacity:
            self.rewind()
        begin = time.perf_counter()
        self.valid += 1
        mask = (torch.arange(self.capacity) >= self.capacity - self.valid).reshape(1, 1, 1, -1)
        logits, self.cache = self.decode(self.token, torch.tensor([[self.valid - 1]]), mask, self.cache)
        self.token = logits[:, -1, :].float().argmax(dim=-1, keepdim=True)
        self.tokens.append(int(self.token))
        return time.perf_counter() - begin

    def run(self, prompt, decode_steps: int):
        """Returns ``(tokens, prefill_seconds, decode_seconds)`` for ``decode_steps`` decode steps."""

        prefill_seconds = self.start(prompt)
        decode_seconds = sum(self.step() for _ in range(decode_steps))
        return self.tokens, prefill_seconds, decode_seconds
