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


def _wide():
    """Small, but with the group size and row lengths the step kernels take (group 64, K multiples of 128)."""

    from aotolith_b200.models.synthetic import SyntheticDecoder

    return SyntheticDecoder(model_type="llama", vocab_size=1024, hidden_size=512, intermediate_size=1024,
                            num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=4, head_dim=64,
                            max_position_embeddings=64, rope_theta=5e5, rms_norm_eps=1e-5, seed=5)


def _wide_prompt():
    return torch.randint(0, 1024, (1, PROMPT), generator=torch.Generator().manual_seed(4))


@pytest.mark.gpu
def test_streamed_decoder_of_one_rank_matches_the_compiled_runtime(cuda):
    """The shard of a world of one is the whole model: the streamed decoder is the compiled runtime."""

    import aotolith_b200 as aoto

    model = _wide()
    runtime = aoto.compile_llama_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW, quantize=64)
    want = runtime.greedy_generate(_wide_prompt()).cpu()
    decoder = tp.StreamedTensorParallelDecoder(model, prompt_length=PROMPT, max_new_tokens=NEW, group_size=64,
                                               world=1, rank=0, device=cuda)
    assert decoder.session.kernel_name == "stream_step_kernel"
    assert torch.equal(decoder.greedy_generate(_wide_prompt()).cpu(), want)
    decoder.close()


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
        # the decode step as ONE kernel per rank that stores its partial rows into the peers
        wide = _wide()
        per_operation = tp.TensorParallelDecoder(wide, prompt_length=PROMPT, max_new_tokens=NEW, group_size=64)
        wide_tokens = per_operation.greedy_generate(_wide_prompt()).cpu()
        streamed = tp.StreamedTensorParallelDecoder(wide, prompt_length=PROMPT, max_new_tokens=NEW, group_size=64)
        assert streamed.session.kernel_name == "stream_step_kernel"
        streamed_tokens = streamed.greedy_generate(_wide_prompt()).cpu()
        streamed_again = streamed.greedy_generate(_wide_prompt()).cpu()
        local_logits = streamed.session.logits.float().cpu().reshape(-1)            # this rank's slice, last step
        share = per_operation.local_vocab
        want_logits = per_operation.logits.float().cpu().reshape(-1)[rank * share:(rank + 1) * share]
        torch.save({"tokens": tokens, "logits": logits, "plain_tokens": plain_tokens, "row": row.float().cpu(),
                    "compiled_tokens": compiled_tokens, "wide_tokens": wide_tokens, "streamed_tokens": streamed_tokens,
                    "streamed_again": streamed_again, "streamed_logits": local_logits, "wide_logits": want_logits,
                    "status": int(streamed.session.status.item())}, os.path.join(out_dir, f"gpu{rank}.pt"))
        dist.barrier()
        decoder.close()
        plain.close()
        runtime.close()
        per_operation.close()
        streamed.close()
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
    # the streamed step kernel with peer stores against the recorded per-operation step with peer sums
    for result in results:
        assert result["status"] == 0
        assert torch.equal(result["streamed_tokens"], results[0]["streamed_tokens"])   # every rank picks the same token
        assert torch.equal(result["streamed_tokens"], result["streamed_again"])        # and again on the next request
        scale = float(result["wide_logits"].abs().max())
        assert float((result["streamed_logits"] - result["wide_logits"]).abs().max()) <= 2e-2 * scale
    same = int((results[0]["streamed_tokens"] == results[0]["wide_tokens"]).sum())
    assert same >= NEW - 1, (results[0]["streamed_tokens"], results[0]["wide_tokens"])


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


def test_a_shard_compiles_and_its_residual_stages_become_exchanged():
    """``shard_module`` + ``route_exchange``: the stage program of one rank's shard, rewired on the CPU."""

    import aotolith_b200 as aoto
    from aotolith_b200 import _native as N
    from aotolith_b200.models.synthetic import SyntheticDecoder
    from aotolith_b200.runtime import stream_plan as sp

    model = SyntheticDecoder(model_type="llama", vocab_size=512, hidden_size=256, intermediate_size=512,
                             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                             max_position_embeddings=64, seed=3)
    shard = tp.shard_module(model, 2, 1, 64)
    assert (shard.config.num_attention_heads, shard.config.num_key_value_heads, shard.config.intermediate_size) == (2, 1, 256)
    assert torch.equal(shard.lm_head.weight, model.lm_head.weight[256:])
    assert torch.equal(shard.model.layers[1].self_attn.o_proj.weight, model.model.layers[1].self_attn.o_proj.weight[:, 128:])
    assert torch.equal(shard.model.layers[0].mlp.down_proj.weight, model.model.layers[0].mlp.down_proj.weight[:, 256:])
    runtime = aoto.compile_llama_static_cache(shard, prompt_length=8, max_new_tokens=6, quantize=64)
    program = runtime.decode.plan.step_program
    assert program is not None and program.vocab == 256

    places: dict = {}

    def resolve(ref):  # distinct fake addresses, 64 KB apart
        return 0x10000 * (1 + places.setdefault((ref.space, str(ref.key)), len(places))) + ref.offset

    base, vector_bytes, row_bytes = 0x7000_0000, 2048, 256 * 4
    for rank in (0, 1):
        array = sp.stage_array(program, resolve)
        count = len(program.stages)
        before = [(int(array[i].x or 0), int(array[i].out or 0), int(array[i].addend or 0), array[i].addend_mode)
                  for i in range(count)]
        used = tp.route_exchange(array, count, base, vector_bytes, row_bytes, rank)
        assert used == 4  # o and down of two layers
        exchanged = [i for i in range(count) if array[i].flags & N.STAGE_FLAG_TO_PEERS]
        assert [array[i].K for i in exchanged] == [128, 256, 128, 256]
        assert [int(array[i].out) for i in exchanged] == [base + n * vector_bytes for n in range(4)]
        for n, i in enumerate(exchanged):
            # the stage after an exchanged one reads it as a sum; the next residual stage adds it as a sum (rank 0)
            assert array[i + 1].flags & N.STAGE_FLAG_X_SUM and int(array[i + 1].x) == base + n * vector_bytes
            if rank == 0:
                assert array[i].addend_mode == before[i][3]
                if n > 0:
                    assert array[i].flags & N.STAGE_FLAG_ADDEND_SUM and int(array[i].addend) == base + (n - 1) * vector_bytes
            else:
                assert array[i].addend_mode == N.STAGE_ADDEND_NONE and not array[i].flags & N.STAGE_FLAG_ADDEND_SUM
        untouched = [i for i in range(count) if i not in exchanged and not array[i].flags & N.STAGE_FLAG_X_SUM]
        for i in untouched:
            assert (int(array[i].x or 0), int(array[i].out or 0)) == before[i][:2]
    with pytest.raises(Exception):
        tp.route_exchange(sp.stage_array(program, resolve), len(program.stages), base, vector_bytes, row_bytes + 4, 0)


def test_which_models_get_the_streamed_sharded_step():
    from aotolith_b200.models.synthetic import llama3_8b_shaped  # noqa: F401 - shapes only, nothing is built

    assert not tp.streamed_step_applies(_tiny(), 2, GROUP)           # group size 16
    assert tp.streamed_step_applies(_wide(), 2, 64) and tp.streamed_step_applies(_wide(), 4, 64)
    assert not tp.streamed_step_applies(_wide(), 8, 64)              # 8 x 64 / 8 = 64 columns of o a rank: not a block
    assert not tp.streamed_step_applies(_wide(), 3, 64)
    from types import SimpleNamespace

    big = SimpleNamespace(config=SimpleNamespace(num_attention_heads=32, num_key_value_heads=8, hidden_size=4096,
                                                 intermediate_size=14336, head_dim=128, vocab_size=128256))
    assert all(tp.streamed_step_applies(big, world, 64) for world in (1, 2, 4, 8))
