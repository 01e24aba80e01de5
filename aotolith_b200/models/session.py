"""Device-resident greedy decoding: one recorded CUDA graph per decode step.

The reference's greedy loop hands every step to MLX's asynchronous executor and
synchronises once at the end (``src/aotolith/models/decoder.py:1054-1087``).
The CUDA counterpart records a whole step - the inputs of the step, the decode
plan's kernels, the greedy pick - into a graph, so the host's share of a step is
one graph launch:

    step_inputs   position = valid_length - 1, mask = window of valid_length slots
    decode plan   embedding ... projections ... logits, next cache
    greedy_pick   token = argmax(logits); generated[n] = token; counters += 1

Two graphs are recorded over two cache buffers (A -> B, B -> A): the decode
plan writes each layer's shifted window straight into the other buffer, so a
step moves every window once and nothing is copied between steps. Tokens stay
on the device until the caller reads the result.
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import PlanInputError


class DecodeSession:
    def __init__(self, runtime) -> None:
        self.runtime = runtime
        module_plan = runtime.decode
        self.plan = module_plan.plan
        self.device = torch.device(self.plan.device)
        graph = self.plan.graph
        if len(graph.outputs) != 2 or module_plan.input_count != 4:
            raise PlanInputError("the decode plan does not have the (token, position, mask, cache) signature")
        self.cache_output = graph.outputs[1]
        cache_type = runtime._cache_tensor_type()
        capacity = runtime.cache_capacity
        device = self.device
        self.token = torch.zeros((1, 1), dtype=torch.int64, device=device)
        self.position = torch.zeros((1, 1), dtype=torch.int64, device=device)
        self.mask = torch.zeros((1, 1, 1, capacity), dtype=torch.bool, device=device)
        self.caches = [
            torch.zeros(cache_type.shape, dtype=torch.bfloat16, device=device) for _ in range(2)
        ]
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.generated = torch.zeros(max(runtime.max_new_tokens, 1), dtype=torch.int64, device=device)
        self.state = list(module_plan._state_values)
        self.graphs: list[torch.cuda.CUDAGraph] = []
        self._record()

    def _step(self, source: int) -> None:
        ops.step_inputs(self.counters, self.position, self.mask)
        target = self.caches[1 - source]
        logits, cache = self.plan.run_eager(
            [self.token, self.position, self.mask, self.caches[source], *self.state],
            buffers={self.cache_output: target},
        )
        if cache.data_ptr() != target.data_ptr():
            target.copy_(cache)  # the plan could not place its result: one copy instead
        ops.greedy_pick(logits.reshape(-1), self.token, self.generated, self.counters)

    def _record(self) -> None:
        device = self.device
        self.counters.copy_(torch.tensor([1, 0], dtype=torch.int32))
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            self._step(0)
            self._step(1)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        pool = None
        for source in (0, 1):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=pool):
                self._step(source)
            pool = graph.pool()
            self.graphs.append(graph)

    def run(self, token: torch.Tensor, cache: torch.Tensor, valid_length: int, steps: int) -> torch.Tensor:
        """Decode ``steps`` tokens after ``token``; returns them as int64 ``[steps]``.

        ``cache`` holds ``valid_length`` tokens (the last ``valid_length`` slots)
        and is not modified.
        """

        if steps < 0 or steps > self.generated.numel():
            raise PlanInputError(f"steps must be in [0, {self.generated.numel()}], got {steps}")
        if valid_length + steps >= self.runtime.cache_capacity + 1:
            raise PlanInputError("the requested steps do not fit the cache capacity")
        self.token.copy_(token.reshape(1, 1))
        self.caches[0].copy_(cache)
        self.counters.copy_(
            torch.tensor([valid_length + 1, 0], dtype=torch.int32).pin_memory(), non_blocking=True
        )
        for step in range(steps):
            self.graphs[step & 1].replay()
        return self.generated[:steps].clone()

    def final_cache(self, steps: int) -> torch.Tensor:
        """The cache after the last ``run`` of ``steps`` steps (a copy)."""

        return self.caches[steps & 1].clone()


def decode_session(runtime) -> DecodeSession:
    """The session of ``runtime``, recorded on first use."""

    key = id(runtime.decode.plan)
    session = runtime._sessions.get(key)
    if session is None:
        session = DecodeSession(runtime)
        runtime._sessions[key] = session
    return session
