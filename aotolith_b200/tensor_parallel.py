"""Tensor-parallel greedy decoding of a packed decoder over the GPUs of one node.

Models whose weights do not leave room for speed on one GPU (the Llama-3-8B
shape) shard the Megatron way, one process per GPU:

* q/k/v, gate and up are split by output rows (q/k/v by head: every rank owns
  ``QH/tp`` query heads and ``KVH/tp`` key/value heads, so attention and the KV
  cache need no exchange);
* o and down are split along K at multiples of the quantisation group, so a
  rank's slice of the packed words and of the scales is exactly what packing
  the whole matrix would have put there; every rank produces a partial sum and
  ONE all-reduce per attention block and ONE per MLP block combines them. The
  residual is folded into rank 0's partial (the GEMV/GEMM addend), so the
  reduced tensor already is the new hidden state on every rank;
* in decode that all-reduce is one launch of ``aoto_sm100_peer_sum`` per rank: stamped 8-byte
  stores into every peer's receive buffer over NVLink and a poll of the own buffer, no library
  collective (``aotolith_b200.peer``); prefill rows (megabytes) go through NCCL;
* the LM head is split over the vocabulary; ranks all-gather their logits
  slices and take the argmax of the whole row;
* embeddings, norms and rotary tables are replicated.

Every step's kernels are the single-GPU ones (``aotolith_b200.ops``) on the
local shard; the collectives are NCCL calls on the same stream. A decode step
(kernels and all-reduces) is recorded once into a CUDA graph per cache
direction and replayed per token; tokens stay on the device until the caller
reads them. The reference has no multi-device path: this follows the packed
decoder adapter (``src/aotolith/models/decoder.py:524-737``) shard by shard.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist

from .errors import CompilationError, PlanInputError
from .models.adapters import _rope_settings, rotary_tables
from .models.quantized import pack_weight


# ---------------------------------------------------------------------------
# sharding of weights (host side, testable without a GPU)
# ---------------------------------------------------------------------------

def check_divisible(name: str, value: int, world: int, multiple: int = 1) -> int:
    if value % (world * multiple) != 0:
        raise CompilationError(
            f"{name} = {value} cannot be split over {world} ranks in multiples of {multiple}",
            hint="choose a tensor-parallel degree that divides the heads, the MLP width and the vocabulary",
        )
    return value // world


def rows_of(weight: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rank ``rank``'s block of output rows (column parallelism)."""

    share = check_divisible("rows", weight.shape[0], world)
    return weight[rank * share:(rank + 1) * share]


def columns_of(weight: torch.Tensor, world: int, rank: int, group_size: int) -> torch.Tensor:
    """Rank ``rank``'s block of input columns (row parallelism), whole quantisation groups only."""

    share = check_divisible("columns", weight.shape[1], world, group_size)
    return weight[:, rank * share:(rank + 1) * share]


def qkv_rows_of(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *, heads: int, kv_heads: int,
                head_dim: int, world: int, rank: int) -> torch.Tensor:
    """The packed q/k/v matrix of one rank: its query heads, then its key heads, then its value heads."""

    q_share = check_divisible("query heads", heads, world) * head_dim
    kv_share = check_divisible("key/value heads", kv_heads, world) * head_dim
    return torch.cat((
        query[rank * q_share:(rank + 1) * q_share],
        key[rank * kv_share:(rank + 1) * kv_share],
        value[rank * kv_share:(rank + 1) * kv_share],
    ), dim=0)


def shard_packed_rows(packed: torch.Tensor, scales: torch.Tensor, world: int, rank: int):
    """Row block of an already packed matrix (equals packing the row block)."""

    return rows_of(packed, world, rank).contiguous(), rows_of(scales, world, rank).contiguous()


def shard_packed_columns(packed: torch.Tensor, scales: torch.Tensor, world: int, rank: int, group_size: int):
    """Column block of an already packed matrix: eight codes per word, one scale per group."""

    k = packed.shape[1] * 8
    share = check_divisible("columns", k, world, max(group_size, 8))
    words, groups = share // 8, share // group_size
    return (packed[:, rank * words:(rank + 1) * words].contiguous(),
            scales[:, rank * groups:(rank + 1) * groups].contiguous())


# ---------------------------------------------------------------------------
# the sharded decoder
# ---------------------------------------------------------------------------

class TensorParallelDecoder:
    """One rank's shard of a packed decoder plus the greedy loop over it."""

    def __init__(self, model: torch.nn.Module, *, prompt_length: int, max_new_tokens: int, group_size: int = 64,
                 world: int | None = None, rank: int | None = None, device: Any = None, group: Any = None,
                 peer_exchange: bool = True) -> None:
        from . import ops  # the CUDA path: fails loudly without the kernel library

        self.ops = ops
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        config = model.config
        self.hidden = int(config.hidden_size)
        self.layers = int(config.num_hidden_layers)
        self.heads = int(config.num_attention_heads)
        self.kv_heads = int(config.num_key_value_heads)
        self.head_dim = int(getattr(config, "head_dim", None) or self.hidden // self.heads)
        self.vocab = int(config.vocab_size)
        self.eps = float(config.rms_norm_eps)
        self.group_size = int(group_size)
        self.prompt_length, self.max_new_tokens = int(prompt_length), int(max_new_tokens)
        self.capacity = self.prompt_length + self.max_new_tokens
        tp = self.world
        self.local_heads = check_divisible("query heads", self.heads, tp)
        self.local_kv_heads = check_divisible("key/value heads", self.kv_heads, tp)
        check_divisible("MLP width", int(config.intermediate_size), tp, self.group_size)
        check_divisible("attention width", self.heads * self.head_dim, tp, self.group_size)
        self.local_vocab = check_divisible("vocabulary", self.vocab, tp)
        dtype = next(model.parameters()).dtype
        if dtype != torch.bfloat16:
            raise CompilationError("the cuda-sm100 kernels compute in bfloat16", hint="convert the model with .bfloat16()")

        def put(tensor: torch.Tensor) -> torch.Tensor:
            return tensor.detach().contiguous().to(self.device)

        def pack(weight: torch.Tensor):
            words, scales = pack_weight(weight, self.group_size)
            return put(words), put(scales.to(dtype))

        r, g = self.rank, self.group_size
        self.embed = put(model.model.embed_tokens.weight)
        self.final_norm = put(model.model.norm.weight)
        self.lm_head = pack(rows_of(model.lm_head.weight, tp, r))
        cosine, sine = rotary_tables(self.capacity, self.head_dim, _rope_settings(config)[0], dtype)
        self.cosine, self.sine = put(cosine), put(sine)
        self.blocks = []
        for layer in model.model.layers:
            attention, mlp = layer.self_attn, layer.mlp
            qkv = qkv_rows_of(attention.q_proj.weight, attention.k_proj.weight, attention.v_proj.weight,
                              heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, world=tp, rank=r)
            bias = None
            if attention.q_proj.bias is not None:
                bias = put(qkv_rows_of(attention.q_proj.bias, attention.k_proj.bias, attention.v_proj.bias,
                                       heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, world=tp, rank=r))
            self.blocks.append(dict(
                input_norm=put(layer.input_layernorm.weight), post_norm=put(layer.post_attention_layernorm.weight),
                qkv=pack(qkv), qkv_bias=bias,
                o=pack(columns_of(attention.o_proj.weight, tp, r, g)),
                gate=pack(rows_of(mlp.gate_proj.weight, tp, r)), up=pack(rows_of(mlp.up_proj.weight, tp, r)),
                down=pack(columns_of(mlp.down_proj.weight, tp, r, g)),
            ))
        cache_shape = (self.layers, 2, 1, self.local_kv_heads, self.capacity, self.head_dim)
        self.caches = [torch.zeros(cache_shape, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self.token = torch.zeros((1, 1), dtype=torch.int64, device=self.device)
        self.position = torch.zeros((1, 1), dtype=torch.int64, device=self.device)
        self.mask = torch.zeros((1, 1, 1, self.capacity), dtype=torch.bool, device=self.device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.generated = torch.zeros(max(self.max_new_tokens, 1), dtype=torch.int64, device=self.device)
        self.logits = torch.zeros((1, self.vocab), dtype=torch.bfloat16, device=self.device)
        self.graphs: list[torch.cuda.CUDAGraph] = []
        # Decode all-reduces move one hidden-state row (a few KB): a kernel of this library over
        # peer memory replaces the NCCL call there; prefill rows (MBs) stay with NCCL.
        self.peer = None
        if peer_exchange and self.world > 1:
            from .peer import PeerSum

            self.peer = PeerSum(self.hidden, group=group, device=self.device)

    # -- collectives -------------------------------------------------------------
    def _all_reduce(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            if self.peer is not None and tensor.numel() <= self.hidden and tensor.is_contiguous():
                self.peer.sum_(tensor)
            else:
                dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor

    def _gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            self.logits.copy_(local.reshape(1, -1))
        else:
            dist.all_gather_into_tensor(self.logits.reshape(-1), local.reshape(-1).contiguous(), group=self.group)
        return self.logits

    def _residual(self, hidden: torch.Tensor) -> torch.Tensor | None:
        return hidden if self.rank == 0 else None  # the residual enters the sum exactly once

    # -- prefill -----------------------------------------------------------------
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Fill cache buffer 0 with the prompt's keys and values; returns the last position's logits."""

        ops, P, D = self.ops, self.prompt_length, self.head_dim
        ids = ids.to(self.device).reshape(1, -1)
        if ids.shape[1] != P:
            raise PlanInputError(f"expected a prompt of {P} tokens, got {ids.shape[1]}")
        hidden = ops.embedding(self.embed, ids).reshape(P, self.hidden)
        cosine, sine = self.cosine[:P][None, None], self.sine[:P][None, None]
        causal = torch.ones((P, P), dtype=torch.bool, device=self.device).tril()[None, None]
        mask = ops.mask_select(causal, 0.0, -math.inf)
        cache = self.caches[0]
        cache.zero_()
        q_width, kv_width = self.local_heads * D, self.local_kv_heads * D
        for index, block in enumerate(self.blocks):
            normed = ops.rms_norm(hidden, block["input_norm"], self.eps)
            row = ops.qmatmul(normed, *block["qkv"], group_size=self.group_size, addend=block["qkv_bias"])
            query = row[:, :q_width].reshape(1, P, self.local_heads, D).transpose(1, 2)
            key = row[:, q_width:q_width + kv_width].reshape(1, P, self.local_kv_heads, D).transpose(1, 2)
            value = row[:, q_width + kv_width:].reshape(1, P, self.local_kv_heads, D).transpose(1, 2)
            query, key = ops.rope(query.contiguous(), cosine, sine), ops.rope(key.contiguous(), cosine, sine)
            cache[index, 0, 0, :, self.capacity - P:, :] = key[0]
            cache[index, 1, 0, :, self.capacity - P:, :] = value[0]
            attended = ops.attention(query, key, value.contiguous(), mask)
            attended = attended.transpose(1, 2).reshape(P, q_width)
            hidden = self._all_reduce(ops.qmatmul(attended, *block["o"], group_size=self.group_size,
                                                  addend=self._residual(hidden)))
            normed = ops.rms_norm(hidden, block["post_norm"], self.eps)
            gate = ops.qmatmul(normed, *block["gate"], group_size=self.group_size)
            act = ops.qmatmul(normed, *block["up"], group_size=self.group_size, gate=gate)
            hidden = self._all_reduce(ops.qmatmul(act, *block["down"], group_size=self.group_size,
                                                  addend=self._residual(hidden)))
        local = ops.qmatmul(hidden[-1:], *self.lm_head, group_size=self.group_size,
                            norm_weight=self.final_norm, rms_norm_eps=self.eps)
        return self._gather_logits(local)

    # -- decode ------------------------------------------------------------------
    def _step(self, source: int) -> None:
        """One decode step from cache buffer ``source`` into the other one (device-resident inputs)."""

        ops, D = self.ops, self.head_dim
        ops.step_inputs(self.counters, self.position, self.mask)
        mask = ops.mask_select(self.mask, 0.0, -math.inf)
        cosine = ops.embedding(self.cosine, self.position)
        sine = ops.embedding(self.sine, self.position)
        hidden = ops.embedding(self.embed, self.token).reshape(1, self.hidden)
        q_width, kv_width = self.local_heads * D, self.local_kv_heads * D
        old, new = self.caches[source], self.caches[1 - source]
        for index, block in enumerate(self.blocks):
            row = ops.qmatmul(hidden, *block["qkv"], group_size=self.group_size, addend=block["qkv_bias"],
                              norm_weight=block["input_norm"], rms_norm_eps=self.eps)
            query, _, keys, values = ops.rope_kv_cache_append(
                old, row, cosine, sine, layer=index, query_start=0, key_start=q_width,
                value_start=q_width + kv_width, query_heads=self.local_heads, new_pair=new[index])
            attended = ops.attention(query, keys, values, mask).reshape(1, q_width)
            hidden = self._all_reduce(ops.qmatmul(attended, *block["o"], group_size=self.group_size,
                                                  addend=self._residual(hidden)))
            act = ops.qmatmul(hidden, *block["gate"], group_size=self.group_size, packed2=block["up"][0],
                              scales2=block["up"][1], norm_weight=block["post_norm"], rms_norm_eps=self.eps)
            hidden = self._all_reduce(ops.qmatmul(act, *block["down"], group_size=self.group_size,
                                                  addend=self._residual(hidden)))
        local = ops.qmatmul(hidden, *self.lm_head, group_size=self.group_size,
                            norm_weight=self.final_norm, rms_norm_eps=self.eps)
        ops.greedy_pick(self._gather_logits(local).reshape(-1), self.token, self.generated, self.counters)

    def _record(self) -> None:
        """Two CUDA graphs (cache 0 -> 1, 1 -> 0); the collectives are part of the recording."""

        saved = [cache.clone() for cache in self.caches]
        state = (self.token.clone(), self.counters.clone(), self.generated.clone())
        self.counters.copy_(torch.tensor([1, 0], dtype=torch.int32))
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._step(0)
            self._step(1)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        pool = None
        for source in (0, 1):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=pool, stream=side):
                self._step(source)
            pool = graph.pool()
            self.graphs.append(graph)
        for cache, kept in zip(self.caches, saved):
            cache.copy_(kept)
        self.token.copy_(state[0]); self.counters.copy_(state[1]); self.generated.copy_(state[2])

    def close(self) -> None:
        """Drop the recorded graphs. Call before ``destroy_process_group``: a communicator cannot be
        torn down while recorded graphs still hold its kernels (the teardown then never returns)."""

        torch.cuda.synchronize(self.device)
        self.graphs.clear()
        torch.cuda.synchronize(self.device)
        if self.peer is not None:
            self.peer.check()

    def greedy_generate(self, ids: torch.Tensor, *, max_new_tokens: int | None = None, use_graphs: bool = True) -> torch.Tensor:
        """Prefill ``ids`` and decode greedily; every rank returns the same ``[1, steps]`` tokens."""

        steps = self.max_new_tokens if max_new_tokens is None else int(max_new_tokens)
        if not 0 < steps <= self.max_new_tokens:
            raise PlanInputError(f"max_new_tokens must be in [1, {self.max_new_tokens}], got {steps}")
        if use_graphs and not self.graphs:
            self._record()
        logits = self.prefill(ids)
        first = self.ops.argmax(logits).reshape(1, 1)
        return torch.cat((first, self.decode_after_prefill(first, steps - 1, use_graphs).reshape(1, -1)), dim=1)

    def decode_after_prefill(self, first: torch.Tensor, steps: int, use_graphs: bool = True) -> torch.Tensor:
        """``steps`` greedy tokens after ``first`` (the prompt's caches are in buffer 0); int64 ``[steps]``."""

        if use_graphs and not self.graphs:
            self._record()
        self.token.copy_(first.reshape(1, 1))
        self.counters.copy_(torch.tensor([self.prompt_length + 1, 0], dtype=torch.int32).pin_memory(), non_blocking=True)
        for step in range(steps):
            if use_graphs:
                self.graphs[step & 1].replay()
            else:
                self._step(step & 1)
        return self.generated[:steps]



# ---------------------------------------------------------------------------
# the sharded decode step as ONE kernel per rank: compute and exchange in the same launch
# ---------------------------------------------------------------------------

class _ShardConfig:
    """Config of one rank's shard: the model's, with the local head counts and MLP width."""

    def __init__(self, config, **changes) -> None:
        for name in dir(config):
            if not name.startswith("_") and not callable(getattr(config, name, None)):
                try:
                    setattr(self, name, getattr(config, name))
                except AttributeError:
                    pass
        for name, value in changes.items():
            setattr(self, name, value)


def shard_module(model: torch.nn.Module, world: int, rank: int, group_size: int) -> torch.nn.Module:
    """One rank's shard of ``model`` as a decoder of its own (the module tree the adapters read).

    ``QH/world`` query heads and ``KVH/world`` key/value heads (rows of q/k/v, columns of o),
    ``I/world`` rows of gate and up (columns of down), ``V/world`` rows of the LM head; embeddings and
    norms whole. Compiled like any decoder, it computes this rank's PARTIAL o and down products
    (their K is split), which is why its decode step only makes sense with the exchange of
    :class:`ShardExchange`. Weights are views of ``model``'s where the slice is contiguous.
    """

    from torch import nn

    config = model.config
    heads, kv_heads = int(config.num_attention_heads), int(config.num_key_value_heads)
    head_dim = int(getattr(config, "head_dim", None) or config.hidden_size // heads)
    check_divisible("query heads", heads, world)
    check_divisible("key/value heads", kv_heads, world)
    check_divisible("MLP width", int(config.intermediate_size), world, group_size)
    check_divisible("attention width", heads * head_dim, world, group_size)
    check_divisible("vocabulary", int(config.vocab_size), world)

    def linear(weight: torch.Tensor, bias: torch.Tensor | None = None) -> nn.Module:
        layer = nn.Module()
        layer.weight = nn.Parameter(weight.detach().contiguous(), requires_grad=False)
        layer.bias = None if bias is None else nn.Parameter(bias.detach().contiguous(), requires_grad=False)
        return layer

    def norm(source: nn.Module) -> nn.Module:
        layer = nn.Module()
        layer.weight = nn.Parameter(source.weight.detach(), requires_grad=False)
        return layer

    shard = nn.Module()
    shard.config = _ShardConfig(
        config, num_attention_heads=heads // world, num_key_value_heads=kv_heads // world, head_dim=head_dim,
        intermediate_size=int(config.intermediate_size) // world, tie_word_embeddings=False)
    shard.model = nn.Module()
    shard.model.embed_tokens = nn.Module()
    shard.model.embed_tokens.weight = nn.Parameter(model.model.embed_tokens.weight.detach(), requires_grad=False)
    shard.model.norm = norm(model.model.norm)
    shard.lm_head = linear(rows_of(model.lm_head.weight, world, rank))
    layers = []
    q_share, kv_share = heads // world * head_dim, kv_heads // world * head_dim
    for layer in model.model.layers:
        attention, mlp = layer.self_attn, layer.mlp
        block, attn, feed = nn.Module(), nn.Module(), nn.Module()

        def rows(projection, share):
            bias = None if projection.bias is None else projection.bias[rank * share:(rank + 1) * share]
            return linear(projection.weight[rank * share:(rank + 1) * share], bias)

        attn.q_proj, attn.k_proj, attn.v_proj = rows(attention.q_proj, q_share), rows(attention.k_proj, kv_share), rows(attention.v_proj, kv_share)
        attn.o_proj = linear(columns_of(attention.o_proj.weight, world, rank, group_size))
        feed.gate_proj = linear(rows_of(mlp.gate_proj.weight, world, rank))
        feed.up_proj = linear(rows_of(mlp.up_proj.weight, world, rank))
        feed.down_proj = linear(columns_of(mlp.down_proj.weight, world, rank, group_size))
        feed.act_fn = getattr(mlp, "act_fn", None)
        block.self_attn, block.mlp = attn, feed
        block.input_layernorm, block.post_attention_layernorm = norm(layer.input_layernorm), norm(layer.post_attention_layernorm)
        layers.append(block)
    shard.model.layers = nn.ModuleList(layers)
    return shard.eval()


def route_exchange(array, stages: int, base: int, vector_bytes: int, row_bytes: int, rank: int) -> int:
    """Turn the residual stages of a shard's stage array into exchanged ones; returns how many.

    A GEMV stage that adds a residual (stamped or gathered addend) is an o or down projection: its
    result moves to the next free exchanged vector at ``base`` and is flagged ``TO_PEERS``; every
    later stage that read the old place as its input gets ``X_SUM``, as its stamped addend
    ``ADDEND_SUM``. Ranks other than 0 drop the residual: it enters the sum once.
    """

    from . import _native as N

    moved: dict[int, int] = {}
    used = 0
    for index in range(stages):
        stage = array[index]
        if stage.kind != N.STAGE_GEMV:
            continue
        if stage.x is not None and int(stage.x) in moved and not stage.flags & N.STAGE_FLAG_X_GATHER:
            stage.x = moved[int(stage.x)]
            stage.flags |= N.STAGE_FLAG_X_SUM
        if stage.addend_mode in (N.STAGE_ADDEND_STAMPED, N.STAGE_ADDEND_GATHER):
            if stage.N * 4 != row_bytes or stage.flags & N.STAGE_FLAG_OUT_PLAIN:
                raise CompilationError("a residual stage of the shard does not produce a hidden-state row")
            if stage.addend_mode == N.STAGE_ADDEND_STAMPED and int(stage.addend) in moved:
                stage.addend = moved[int(stage.addend)]
                stage.flags |= N.STAGE_FLAG_ADDEND_SUM
            if rank != 0:
                stage.addend_mode = N.STAGE_ADDEND_NONE
                stage.flags &= ~N.STAGE_FLAG_ADDEND_SUM
            moved[int(stage.out)] = base + used * vector_bytes
            stage.out = base + used * vector_bytes
            stage.flags |= N.STAGE_FLAG_TO_PEERS
            used += 1
    return used


class ShardExchange:
    """Buffers and rewiring that turn a shard's stage program into this rank's part of a sharded step.

    The o and down projections of a shard are partial products (their K is split over the ranks).
    In the stage program they are the GEMV stages that add a residual. Their results become
    *exchanged vectors*: ``world`` rows of stamped words in a buffer every peer can store into
    (torch symmetric memory); a stage writes its row on EVERY rank, the stages that read the
    vector add its rows while they stage it. The residual enters the sum once (rank 0). The ranks'
    best logits meet the same way in the pick stage. No library collective runs in the step.
    """

    def __init__(self, hidden: int, stages: int, *, group: Any = None, device: Any = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.row_bytes = hidden * 4                      # a row of an exchanged vector: hidden / 2 words
        self.vector_bytes = (self.world * self.row_bytes + 255) // 256 * 256
        self.vectors = stages                            # upper bound: one per stage
        self.pick_offset = self.vectors * self.vector_bytes
        nbytes = self.pick_offset + 256
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        pointers = [int(p) for p in self.handle.buffer_ptrs]
        if len(pointers) != self.world or any(p == 0 for p in pointers):
            raise CompilationError("symmetric memory did not return one mapped buffer per rank")
        self.deltas = [p - pointers[self.rank] for p in pointers]
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every buffer is zero before any rank stores into it

    def route(self, array, stages: int) -> None:
        """Rewire one stage array (one cache direction) in place."""

        used = route_exchange(array, stages, self.buffer.data_ptr(), self.vector_bytes, self.row_bytes, self.rank)
        if used > self.vectors:
            raise CompilationError("more exchanged vectors than the exchange buffer holds")

    def fill(self, args, local_vocab: int) -> None:
        args.world, args.rank = self.world, self.rank
        for q, delta in enumerate(self.deltas):
            args.peer_delta[q] = delta
        args.pick_exchange = self.buffer.data_ptr() + self.pick_offset
        args.vocab_offset = self.rank * local_vocab


class StreamedTensorParallelDecoder(TensorParallelDecoder):
    """Tensor-parallel greedy decoding whose decode step is ONE kernel per rank.

    Prefill is the per-operation path of :class:`TensorParallelDecoder` (NCCL all-reduces of the
    prompt rows). A decode step is one cooperative launch of the streamed step kernel over this
    rank's shard: the o and down stages store their partial rows straight into every peer's
    exchange buffer over NVLink, the stages that consume them add the rows while staging, the
    ranks' best logits meet in the pick stage - compute and exchange overlap tile by tile, and no
    collective kernel is launched.
    """

    def __init__(self, model: torch.nn.Module, *, prompt_length: int, max_new_tokens: int, group_size: int = 64,
                 world: int | None = None, rank: int | None = None, device: Any = None, group: Any = None) -> None:
        super().__init__(model, prompt_length=prompt_length, max_new_tokens=max_new_tokens, group_size=group_size,
                         world=world, rank=rank, device=device, group=group, peer_exchange=False)
        from .models.adapters import family_for
        from .models.decoder import compile_decoder_static_cache
        from .models.session import DecodeSession

        with torch.cuda.device(self.device):
            shard = shard_module(model, self.world, self.rank, self.group_size)
            self.shard_runtime = compile_decoder_static_cache(
                shard, prompt_length=prompt_length, max_new_tokens=max_new_tokens, quantize=self.group_size,
                family=family_for(model).name)
            del shard
            program = self.shard_runtime.decode.plan.step_program
            if program is None:
                raise CompilationError("the shard's decode graph has no stage program")
            self.exchange = None
            if self.world > 1:
                self.exchange = ShardExchange(self.hidden, len(program.stages), group=group, device=self.device)
            self.session = DecodeSession(self.shard_runtime, parallel=self.exchange)
        # the per-operation copies of the shards are only needed by prefill; the step has its streams
        self.graphs = []

    def greedy_generate(self, ids: torch.Tensor, *, max_new_tokens: int | None = None, use_graphs: bool = True) -> torch.Tensor:
        steps = self.max_new_tokens if max_new_tokens is None else int(max_new_tokens)
        if not 0 < steps <= self.max_new_tokens:
            raise PlanInputError(f"max_new_tokens must be in [1, {self.max_new_tokens}], got {steps}")
        logits = self.prefill(ids)
        first = self.ops.argmax(logits).reshape(1, 1)
        return torch.cat((first, self.decode_after_prefill(first, steps - 1).reshape(1, -1)), dim=1)

    def decode_after_prefill(self, first: torch.Tensor, steps: int, use_graphs: bool = True) -> torch.Tensor:
        return self.session.run(first.reshape(1, 1), self.caches[0], self.prompt_length, steps)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)  # no rank frees its exchange buffer while a peer may still store into it
        self.session = None
        self.exchange = None


class TensorParallelRuntime:
    """What ``compile_*_static_cache(..., tensor_parallel=group)`` returns on every rank of the group.

    The generation calls of ``DecoderStaticCacheRuntime`` over a sharded decoder: every rank makes
    the same calls with the same prompt and gets the same tokens. There is no per-rank artifact
    to ``save`` and no host-visible cache: keys and values stay sharded by head on the ranks'
    devices.
    """

    def __init__(self, decoder: TensorParallelDecoder, family: str) -> None:
        self.decoder = decoder
        self.family = family
        self.prompt_length = decoder.prompt_length
        self.max_new_tokens = decoder.max_new_tokens
        self.cache_capacity = decoder.capacity
        self.num_layers = decoder.layers
        self.world, self.rank = decoder.world, decoder.rank

    @property
    def device(self) -> torch.device:
        return self.decoder.device

    def prefill_logits(self, input_ids: Any) -> torch.Tensor:
        """``[1, vocab]`` logits of the prompt's last position (the caches now hold the prompt)."""

        return self.decoder.prefill(torch.as_tensor(input_ids))

    def greedy_generate(self, input_ids: Any, *, max_new_tokens: int | None = None) -> torch.Tensor:
        """Greedy tokens ``[1, steps]`` (int64, on this rank's device), the same on every rank."""

        return self.decoder.greedy_generate(torch.as_tensor(input_ids), max_new_tokens=max_new_tokens)

    def close(self) -> None:
        """Drop the recorded steps; call on every rank before the process group is destroyed."""

        self.decoder.close()


def compile_tensor_parallel(model: torch.nn.Module, *, prompt_length: int, max_new_tokens: int, quantize: int | None,
                            quantize_bits: int = 4, family: str | None = None, tensor_parallel: Any = True,
                            device: Any = None) -> TensorParallelRuntime:
    """The sharded counterpart of ``compile_decoder_static_cache``: same model checks, same refusals.

    ``tensor_parallel`` is a process group whose ranks each own one GPU, or ``True`` for the
    default group. Every rank calls this with the same model (same weights).
    """

    from .errors import DynamicShapeError, UnsupportedModelError
    from .models.adapters import _check_activation, _check_attention_is_causal_only, _rope_settings, family_for

    found = family_for(model, require=family)
    if _rope_settings(model.config)[1]:
        raise UnsupportedModelError(f"{found.label} RoPE scaling is not supported yet",
                                    hint="the adapter builds one rotary table from rope_theta")
    _check_activation(model)
    _check_attention_is_causal_only(model)
    if getattr(model, "training", False):
        raise CompilationError("compile_decoder_static_cache requires model.eval()", hint="call model.eval() first")
    if prompt_length <= 0 or max_new_tokens < 0:
        raise CompilationError("prompt_length must be positive and max_new_tokens non-negative",
                               hint="both are compile-time constants of the plan pair")
    if prompt_length + max_new_tokens > int(model.config.max_position_embeddings):
        raise DynamicShapeError(
            "prompt_length + max_new_tokens exceeds the model's maximum position embeddings "
            f"({model.config.max_position_embeddings})", hint="shorten the prompt or the generation")
    if quantize is None or quantize_bits != 4:
        raise UnsupportedModelError("tensor parallelism shards 4-bit packed decoders", hint="pass quantize=64")
    if not dist.is_initialized():
        raise CompilationError("tensor_parallel needs an initialised torch.distributed process group",
                               hint="launch one process per GPU and call init_process_group('nccl') first")
    group = None if tensor_parallel is True else tensor_parallel
    settings = dict(prompt_length=prompt_length, max_new_tokens=max_new_tokens, group_size=quantize, group=group,
                    device=device)
    if streamed_step_applies(model, dist.get_world_size(group), quantize):
        decoder = StreamedTensorParallelDecoder(model, **settings)   # the decode step is one kernel per rank
    else:
        decoder = TensorParallelDecoder(model, **settings)           # recorded per-operation step
    return TensorParallelRuntime(decoder, found.name)


def streamed_step_applies(model: torch.nn.Module, world: int, group_size: int) -> bool:
    """Whether a rank's shard has the shapes the streamed step kernel takes (decided the same way on every
    rank, from the model alone): group size 64, every shard's row length a multiple of 128, head
    dimension 64 or 128."""

    config = model.config
    heads, kv_heads = int(config.num_attention_heads), int(config.num_key_value_heads)
    hidden, inner = int(config.hidden_size), int(config.intermediate_size)
    head_dim = int(getattr(config, "head_dim", None) or hidden // heads)
    if group_size != 64 or head_dim not in (64, 128) or heads % world or kv_heads % world or inner % world:
        return False
    rows = (hidden, heads // world * head_dim, inner // world)   # K of q/k/v, gate, up and the LM head; of o; of down
    return all(k % 128 == 0 for k in rows) and int(config.vocab_size) % (2 * world) == 0
