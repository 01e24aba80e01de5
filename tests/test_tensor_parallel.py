"""Tensor parallelism: sharding rules on CPU (two gloo ranks), the sharded decoder on GPUs.

CPU: the column/row shards of a packed matrix are exactly what packing the shard
gives (codes and scales bit for bit), the row-parallel partial products of two
ranks all-reduce to the full product, the column-parallel blocks concatenate to
it. GPU (one device): a world-of-one ``TensorParallelDecoder`` generates what the
compiled static-cache runtime generates. GPU (two devices, skipped otherwise):
two NCCL ranks generate the same tokens as one.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aotolith_b200 import tensor_parallel as tp
from aotolith_b200.models.quantized import pack_weight
from aotolith_b200.models.synthetic import tiny_decoder
from tests.helpers import exact_packed_matmul

GROUP = 16


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _weight(seed, rows, cols):
    return (torch.randn(rows, cols, generator=torch.Generator().manual_seed(seed)) * 0.05).bfloat16()


def test_shards_of_a_packed_matrix_equal_packing_the_shard():
    weight = _weight(1, 48, 128)
    packed, scales = pack_weight(weight, GROUP)
    for world in (1, 2, 4):
        for rank in range(world):
            p_rows, s_rows = tp.shard_packed_rows(packed, scales, world, rank)
            want_p, want_s = pack_weight(tp.rows_of(weight, world, rank), GROUP)
            assert torch.equal(p_rows, want_p) and torch.equal(s_rows.view(torch.int16), want_s.view(torch.int16))
            p_cols, s_cols = tp.shard_packed_columns(packed, scales, world, rank, GROUP)
            want_p, want_s = pack_weight(tp.columns_of(weight, world, rank, GROUP).contiguous(), GROUP)
            assert torch.equal(p_cols, want_p) and torch.equal(s_cols.view(torch.int16), want_s.view(torch.int16))
    from aotolith_b200.errors import CompilationError
    with pytest.raises(CompilationError):
        tp.columns_of(weight, 16, 0, GROUP)      # 128 columns do not split into 16 blocks of whole groups
    with pytest.raises(CompilationError):
        tp.rows_of(weight, 5, 0)


def test_qkv_rows_keep_heads_together():
    heads, kv_heads, dim = 4, 2, 8
    q = torch.arange(heads * dim)[:, None].float().expand(-1, 3)
    k = 100 + torch.arange(kv_heads * dim)[:, None].float().expand(-1, 3)
    v = 200 + torch.arange(kv_heads * dim)[:, None].float().expand(-1, 3)
    shard = tp.qkv_rows_of(q, k, v, heads=heads, kv_heads=kv_heads, head_dim=dim, world=2, rank=1)
    assert shard[:, 0].tolist() == list(range(16, 32)) + list(range(108, 116)) + list(range(208, 216))


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = (torch.randn(3, 128, generator=torch.Generator().manual_seed(5))).bfloat16()
        down = _weight(2, 32, 128)          # row parallel: K split
        up = _weight(3, 64, 128)            # column parallel: rows split
        packed, scales = pack_weight(tp.columns_of(down, world, rank, GROUP).contiguous(), GROUP)
        share = 128 // world
        partial = exact_packed_matmul(x[:, rank * share:(rank + 1) * share], packed, scales, GROUP)
        dist.all_reduce(partial)
        packed, scales = pack_weight(tp.rows_of(up, world, rank), GROUP)
        block = exact_packed_matmul(x, packed, scales, GROUP)
        blocks = [torch.empty_like(block) for _ in range(world)]
        dist.all_gather(blocks, block)
        torch.save({"reduced": partial, "gathered": torch.cat(blocks, dim=1)}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reduce_to_the_full_product(tmp_path):
    world = 2
    mp.start_processes(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    x = (torch.randn(3, 128, generator=torch.Generator().manual_seed(5))).bfloat16()
    full_down = exact_packed_matmul(x, *pack_weight(_weight(2, 32, 128), GROUP), GROUP)
    full_up = exact_packed_matmul(x, *pack_weight(_weight(3, 64, 128), GROUP), GROUP)
    for rank in range(world):
        result = torch.load(tmp_path / f"rank{rank}.pt", weights_only=False)
        assert torch.allclose(result["reduced"], full_down, rtol=1e-12, atol=1e-12)
        assert torch.equal(result["gathered"], full_up)


# ---------------------------------------------------------------------------
# GPU
# ---------------------------------------------------------------------------

PROMPT, NEW = 8, 6


def _tiny():
    return tiny_decoder("llama", seed=11)


def _prompt():
    return torch.randint(0, 128, (1, PROMPT), generator=torch.Generator().manual_seed(3))


@pytest.mark.gpu
def test_world_of_one_matches_the_compiled_runtime(cuda):
    import aotolith_b200 as aoto

    model = _tiny()
    runtime = aoto.compile_llama_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP)
    want = runtime.greedy_generate(_prompt()).cpu()
    decoder = tp.TensorParallelDecoder(model, prompt_length=PROMPT, max_new_tokens=NEW, group_size=GROUP,
                                       world=1, rank=0, device=cuda)
    eager = decoder.greedy_generate(_prompt(), use_graphs=False).cpu()
    replayed = decoder.greedy_generate(_prompt(), use_graphs=True).cpu()
    assert torch.equal(eager, want) and torch.equal(replayed, want)


def _gpu_rank(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        decoder = tp.TensorParallelDecoder(_tiny(), prompt_length=PROMPT, max_new_tokens=NEW, group_size=GROUP)
        assert decoder.peer is not None
        tokens = decoder.greedy_generate(_prompt()).cpu()
        logits = decoder.prefill(_prompt()).float().cpu()
        # the same steps with the library collective instead of the peer-memory kernel
        plain = tp.TensorParallelDecoder(_tiny(), prompt_length=PROMPT, max_new_tokens=NEW, group_size=GROUP,
                                         peer_exchange=False)
        plain_tokens = plain.greedy_generate(_prompt()).cpu()
        # the exchange alone: every rank contributes rank + 1 in every element
        row = torch.full((1, 64), float(rank + 1), dtype=torch.bfloat16, device=f"cuda:{rank}")
        for _ in range(5):
            row.fill_(float(rank + 1))
            decoder.peer.sum_(row)
        # the public route to the same thing: the compile call with a process group
        import aotolith_b200 as aoto

        runtime = aoto.compile_llama_static_cache(_tiny(), prompt_length=PROMPT, max_new_tokens=NEW, quantize=GROUP,
                                                  tensor_parallel=dist.group.WORLD)
        assert (runtime.world, runtime.rank, runtime.cache_capacity) == (world, rank, PROMPT + NEW)
        compiled_tokens = runtime.greedy_generate(_prompt()).cpu()
        torch.save({"tokens": tokens, "logits": logits, "plain_tokens": plain_tokens, "row": row.float().cpu(),
                    "compiled_tokens": compiled_tokens}, os.path.join(out_dir, f"gpu{rank}.pt"))
        dist.barrier()
        decoder.close()
        plain.close()
        runtime.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_two_nccl_ranks_generate_what_one_rank_does(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    single = tp.TensorParallelDecoder(_tiny(), prompt_length=PROMPT, max_new_tokens=NEW, group_size=GROUP,
                                      world=1, rank=0, device=cuda)
    want_tokens = single.greedy_generate(_prompt()).cpu()
    want_logits = single.prefill(_prompt()).float().cpu()
    mp.start_processes(_gpu_rank, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    results = [torch.load(tmp_path / f"gpu{r}.pt", weights_only=False) for r in range(2)]
    assert torch.equal(results[0]["tokens"], results[1]["tokens"])
    for result in results:
        assert torch.equal(result["tokens"], result["plain_tokens"])     # same sum, different transport
        assert torch.equal(result["tokens"], result["compiled_tokens"])  # the compile option builds the same decoder
        assert torch.equal(result["row"], torch.full((1, 64), 3.0))       # 1 + 2 on every rank
    # partial sums are rounded to bf16 before the all-reduce: logits agree within the toy-model tolerance
    scale = float(want_logits.abs().max())
    assert float((results[0]["logits"] - want_logits).abs().max()) <= 3e-2 * scale
    assert torch.equal(results[0]["logits"], results[1]["logits"])
    agree = int((results[0]["tokens"] == want_tokens).sum())
    assert agree >= NEW - 1, (results[0]["tokens"], want_tokens)


def test_tensor_parallel_compile_option_refuses_what_the_compiler_refuses():
    """``compile_llama_static_cache(..., tensor_parallel=...)``: the model checks come before any device work."""

    import aotolith_b200 as aoto
    from aotolith_b200.errors import CompilationError, DynamicShapeError, UnsupportedModelError

    model = _tiny()
    with pytest.raises(UnsupportedModelError):
        aoto.compile_qwen2_static_cache(model, prompt_length=8, max_new_tokens=4, quantize=GROUP, tensor_parallel=True)
    with pytest.raises(UnsupportedModelError):
        aoto.compile_llama_static_cache(model, prompt_length=8, max_new_tokens=4, tensor_parallel=True)  # dense
    with pytest.raises(DynamicShapeError):
        aoto.compile_llama_static_cache(model, prompt_length=10**6, max_new_tokens=4, quantize=GROUP, tensor_parallel=True)
    with pytest.raises(CompilationError):
        aoto.compile_llama_static_cache(model, prompt_length=8, max_new_tokens=4, quantize=GROUP, tensor_parallel=True,
                                        autotune=True)
    with pytest.raises(CompilationError, match="process group"):
        aoto.compile_llama_static_cache(model, prompt_length=8, max_new_tokens=4, quantize=GROUP, tensor_parallel=True)
