"""Device-resident greedy decoding: the host's share of a decode step is one launch.

The reference's greedy loop hands every step to MLX's asynchronous executor and
synchronises once at the end (``src/aotolith/models/decoder.py:1054-1087``).
Here a whole step - the step's inputs, the decode plan, the greedy pick - runs on
the device without a host round trip:

    step inputs   position = valid_length - 1, mask = window of valid_length slots
    decode plan   embedding ... projections ... logits, next cache
    greedy pick   token = argmax(logits); generated[n] = token; counters += 1

When the decode graph has the form of a stage program
(:mod:`aotolith_b200.runtime.step_program`) the step is ONE launch of the
persistent ``aoto_sm100_decode_step`` kernel; otherwise the per-operation plan is
recorded into a CUDA graph and replayed. Either way two variants exist over two
cache buffers (A -> B, B -> A): each layer's shifted window is written straight
into the other buffer, so a step moves every window once and nothing is copied
between steps. Tokens stay on the device until the caller reads the result.
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import DeviceError, PlanInputError


#: set to route every session to the kernel that reads the weights in place (tests compare the two)
STREAM_STEP_DISABLED = False


class DecodeSession:
    """Static buffers plus either the persistent step kernel or two recorded graphs."""

    def __init__(self, runtime, parallel=None) -> None:
        """``parallel`` (``tensor_parallel.ShardExchange``): the runtime is one rank's shard of a
        tensor-parallel decoder; only the streamed kernel has a form for that."""

        self.runtime = runtime
        self.parallel = parallel
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
        self.programs: list[torch.Tensor] = []
        self.mode = "graphs"
        self.kernel_name = None
        with torch.cuda.device(device):
            if self.plan.step_program is not None and self._bind_stream():
                self.mode, self.kernel_name = "kernel", "stream_step_kernel"
            elif parallel is not None:
                raise DeviceError("the sharded decode step needs the streamed step kernel, which declined this program",
                                  hint="group size 64, K a multiple of 128 and head_dim 64 or 128 are required")
            elif self.plan.step_program is not None and self._bind_program():
                self.mode, self.kernel_name = "kernel", "decode_step_kernel"
            else:
                self._record()

    # -- persistent kernel, weights streamed ahead -------------------------------------
    def _bind_stream(self) -> bool:
        """Lay the packed weights out as per-warp streams and bind the streamed step kernel.

        False if the kernel has no form for the program (the caller then tries the kernel
        that reads the weights in place).
        """

        from .. import _native as N
        from ..runtime import step_program
        from ..runtime import stream_plan as sp

        if STREAM_STEP_DISABLED:
            return False
        program = self.plan.step_program
        graph = self.plan.graph
        device = self.device
        properties = torch.cuda.get_device_properties(device)
        ctas = properties.multi_processor_count
        depth = sp.choose_ring_depth(program, ctas, properties.shared_memory_per_block_optin)
        if depth == 0:
            return False
        tensors = dict(zip(graph.inputs[4:], self.state))
        tensors[program.token_input] = self.token
        tensors[program.position_input] = self.position
        tensors[program.mask_input] = self.mask
        layout, stream, table, starts, duties = sp.device_stream(program, tensors, device, ctas, depth)
        self.arena = torch.zeros(program.arena_bytes, dtype=torch.uint8, device=device)
        self.logits = torch.zeros((1, 1, program.vocab), dtype=torch.bfloat16, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        lib = N.load()
        import ctypes

        need = int(lib.aoto_sm100_stream_step_scratch_bytes_for(ctypes.byref(sp.base_args(program, ctas, depth))))
        if need < 0:
            return False
        self.scratch = torch.zeros(max(need, 1 << 12), dtype=torch.uint8, device=device)
        self.stage_count = len(program.stages) + 1
        self._stream_keep = (stream, table, starts, duties)
        self._stream_args = []
        self.programs = []
        geo = sp.geometry(program)
        for source in (0, 1):
            def resolve(ref, _source=source):
                if ref.space == "arena":
                    return self.arena.data_ptr() + program.arena_offsets[ref.key] + ref.offset
                if ref.space == "output":
                    base = self.logits if ref.key == 0 else self.caches[1 - _source]
                    return base.data_ptr() + ref.offset
                if ref.key == program.cache_input:
                    return self.caches[_source].data_ptr() + ref.offset
                return tensors[ref.key].data_ptr() + ref.offset

            array = sp.stage_array(program, resolve)
            if self.parallel is not None:
                self.parallel.route(array, len(program.stages))
            stages = step_program.to_device(array, device)
            self.programs.append(stages)
            args = sp.base_args(program, ctas, depth)
            if self.parallel is not None:
                self.parallel.fill(args, program.vocab)
            args.stages = stages.data_ptr()
            args.cta_table, args.starts, args.duties = table.data_ptr(), starts.data_ptr(), duties.data_ptr()
            args.stream, args.stream_bytes = stream.data_ptr(), stream.numel()
            if geo is not None:
                args.cos_table, args.sin_table = resolve(geo["cos_table"]), resolve(geo["sin_table"])
                args.position, args.mask = resolve(geo["position"]), resolve(geo["mask"])
            args.x_index = self.token.data_ptr()
            args.x_rows = self._embedding_rows(program, graph)
            args.token, args.generated = self.token.data_ptr(), self.generated.data_ptr()
            args.counters, args.generated_capacity = self.counters.data_ptr(), self.generated.numel()
            args.window = 1
            args.status, args.scratch = self.status.data_ptr(), self.scratch.data_ptr()
            args.scratch_bytes = self.scratch.numel()
            self._stream_args.append(args)
        self.epoch = 0
        self._launch = None
        return True

    @staticmethod
    def _embedding_rows(program, graph) -> int:
        for spec in program.stages:
            if "x_rows" in spec.ints:
                return int(spec.ints["x_rows"])
        return 0

    # -- persistent kernel, weights read in place ----------------------------------------
    def _bind_program(self) -> bool:
        """Resolve the stage program against this session's buffers; False if it does not fit."""

        from ..runtime import step_program as sp

        program = self.plan.step_program
        graph = self.plan.graph
        device = self.device
        tensors = dict(zip(graph.inputs[4:], self.state))
        tensors[program.token_input] = self.token
        tensors[program.position_input] = self.position
        tensors[program.mask_input] = self.mask
        self.arena = torch.zeros(program.arena_bytes, dtype=torch.uint8, device=device)
        self.logits = torch.zeros((1, 1, program.vocab), dtype=torch.bfloat16, device=device)
        greedy = dict(
            token=self.token.data_ptr(), generated=self.generated.data_ptr(),
            counters=self.counters.data_ptr(), generated_capacity=self.generated.numel(),
        )
        arrays = []
        for source in (0, 1):
            def resolve(ref, _source=source):
                if ref.space == "arena":
                    return self.arena.data_ptr() + program.arena_offsets[ref.key] + ref.offset
                if ref.space == "output":
                    base = self.logits if ref.key == 0 else self.caches[1 - _source]
                    return base.data_ptr() + ref.offset
                if ref.key == program.cache_input:
                    return self.caches[_source].data_ptr() + ref.offset
                return tensors[ref.key].data_ptr() + ref.offset

            arrays.append(sp.stage_array(program, resolve, greedy=greedy))
        if not sp.supported(arrays[0]):
            return False
        self.stage_count = len(arrays[0])
        self.programs = [sp.to_device(array, device) for array in arrays]
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.scratch = torch.zeros(max(sp.scratch_bytes(arrays[0]), 1 << 16), dtype=torch.uint8, device=device)
        self._launch = sp.launch
        return True

    def _check_status(self) -> None:
        stage = int(self.status.item())
        if stage:
            self.status.zero_()
            self.scratch.zero_()
            self.arena.zero_()
            raise DeviceError(
                f"the decode-step kernel gave up polling for the inputs of stage {stage - 1}",
                hint="the device could not keep every CTA of the cooperative launch resident; the "
                "arena and scratch were cleared and the session can be used again",
            )

    # -- recorded graphs (the per-operation plan, two cache directions) ---------------
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
            with torch.cuda.graph(graph, pool=pool, stream=side):
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
        with torch.cuda.device(self.device):  # launches go to the current device's stream
            return self._run(token, cache, valid_length, steps)

    def _run(self, token: torch.Tensor, cache: torch.Tensor, valid_length: int, steps: int) -> torch.Tensor:
        self.token.copy_(token.reshape(1, 1))
        self.caches[0].copy_(cache)
        self.counters.copy_(
            torch.tensor([valid_length + 1, 0], dtype=torch.int32).pin_memory(), non_blocking=True
        )
        if self.mode == "kernel":
            for step in range(steps):
                self.launch_step(step & 1)
            tokens = self.generated[:steps].clone()
            self._check_status()
            return tokens
        for step in range(steps):
            self.graphs[step & 1].replay()
        return self.generated[:steps].clone()

    def launch_step(self, source: int, trace: torch.Tensor | None = None) -> None:
        """One launch of the persistent kernel reading cache ``source`` and writing the other."""

        self.epoch = self.epoch % 0xFFFFFFFE + 1
        if self.kernel_name == "stream_step_kernel":
            from ..runtime import stream_plan as sp

            sp.launch(self._stream_args[source], self.epoch, trace)
        else:
            self._launch(self.programs[source], self.stage_count, self.epoch, self.status, self.scratch, trace=trace)

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
