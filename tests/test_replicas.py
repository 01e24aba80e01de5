"""The N > 1 path on CPU: two gloo ranks serve a sharded request stream.

The decode path has no exchange step, so several GPUs means independent replicas
(``aotolith_b200.replicas``). What the ranks share is host logic only - who serves
which request, and how the job's throughput is formed (sum of units over the
slowest rank's time). The served computation here is the CPU oracle of a toy
decoder, so the test also shows that sharding leaves every request's tokens
unchanged.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aotolith_b200 import replicas

PROMPT, NEW, GROUP, REQUESTS = 8, 4, 16, 5


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _prompts():
    generator = torch.Generator().manual_seed(123)
    return [torch.randint(0, 64, (PROMPT,), generator=generator).tolist() for _ in range(REQUESTS)]


def _serve(prompt):
    from aotolith_b200.models.synthetic import tiny_decoder
    from oracle.eager import EagerCpuDecoder

    model = tiny_decoder("qwen2", seed=3)
    decoder = EagerCpuDecoder(model, PROMPT, NEW, GROUP)
    tokens, _, _ = decoder.run(torch.tensor(prompt), NEW - 1)
    return [int(t) for t in tokens]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        prompts = _prompts()
        mine = list(replicas.shard_indices(len(prompts), world, rank))
        dist.barrier()
        served = [(i, _serve(prompts[i])) for i in mine]
        dist.barrier()
        # made-up device times: rank r took 10 * (r + 1) ms for its share
        job = replicas.job_throughput(len(served) * NEW, 10.0 * (rank + 1))
        merged = replicas.gather_results(served)
        torch.save({"mine": mine, "job": (job.units, job.milliseconds, job.world, job.per_second), "merged": merged},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_shard_indices_partition_the_stream():
    for count in (0, 1, 5, 8, 17):
        for world in (1, 2, 3, 8):
            seen = [i for r in range(world) for i in replicas.shard_indices(count, world, r)]
            assert sorted(seen) == list(range(count))
            sizes = [len(replicas.shard_indices(count, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    assert replicas.shard(list("abcde"), 2, 1) == ["b", "d"]
    with pytest.raises(ValueError):
        replicas.shard_indices(4, 2, 2)
    with pytest.raises(ValueError):
        replicas.shard_indices(-1, 2, 0)


def test_job_throughput_without_a_group_is_local():
    job = replicas.job_throughput(640, 500.0)
    assert (job.units, job.milliseconds, job.world) == (640.0, 500.0, 1)
    assert job.per_second == pytest.approx(1280.0)
    assert replicas.gather_results([(0, [1, 2])]) == {0: [1, 2]}


@pytest.mark.timeout(300)
def test_two_gloo_ranks_serve_disjoint_shares(tmp_path):
    world = 2
    port = _free_port()
    mp.start_processes(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    results = [torch.load(tmp_path / f"rank{r}.pt", weights_only=False) for r in range(world)]
    assert results[0]["mine"] == [0, 2, 4] and results[1]["mine"] == [1, 3]
    # both ranks agree on the job figures: all units, the slowest rank's time
    for result in results:
        units, ms, seen_world, per_second = result["job"]
        assert units == REQUESTS * NEW and ms == 20.0 and seen_world == world
        assert per_second == pytest.approx(REQUESTS * NEW / 0.020)
    assert results[0]["merged"] == results[1]["merged"]
    # sharding does not change what a request generates
    prompts = _prompts()
    expected = {i: _serve(p) for i, p in enumerate(prompts)}
    assert results[0]["merged"] == expected
