"""Host-side sharding logic, including a world_size-2 gloo run on the CPU."""
import os
import random

import pytest
import torch

from flash_attention_factory_b200.sharding import (choose_variant, shard_kv_heads,
                                                   shard_sequences_by_kv_length, split_by_variant)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_sequence_shards_cover_and_balance(world):
    rng = random.Random(world)
    ctx = [min(32768, max(16, int(rng.lognormvariate(7.5, 1.0)))) for _ in range(1024)]
    shards = shard_sequences_by_kv_length(ctx, world)
    assert len(shards) == world
    assert shards[0][0] == 0 and shards[-1][1] == len(ctx)
    for (a, b), (c, d) in zip(shards, shards[1:]):
        assert b == c and a <= b
    total = sum(ctx)
    for lo, hi in shards:
        # balanced to within one maximum-length sequence
        assert abs(sum(ctx[lo:hi]) - total / world) <= max(ctx)


def test_sequence_shards_edge_cases():
    assert shard_sequences_by_kv_length([], 4) == [(0, 0)] * 4
    assert shard_sequences_by_kv_length([5], 2) in ([(0, 1), (1, 1)], [(0, 0), (0, 1)])
    assert shard_sequences_by_kv_length([0, 0, 0], 2)[-1][1] == 3
    with pytest.raises(ValueError):
        shard_sequences_by_kv_length([1], 0)


@pytest.mark.parametrize("heads,world", [(8, 1), (8, 2), (8, 4), (8, 8), (8, 3), (2, 4)])
def test_kv_head_shards(heads, world):
    shards = shard_kv_heads(heads, world)
    assert shards[0][0] == 0 and shards[-1][1] == heads
    sizes = [b - a for a, b in shards]
    assert max(sizes) - min(sizes) <= 1


def test_variant_choice_depends_on_the_sequence_only():
    assert choose_variant(100) == "loop" and choose_variant(32768) == "reduce"
    ctx = [10, 5000, 600, 2048, 1]
    loop_idx, reduce_idx = split_by_variant(ctx)
    assert sorted(loop_idx + reduce_idx) == list(range(5))
    assert all(choose_variant(ctx[i]) == "reduce" for i in reduce_idx)


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    ctx = torch.randint(16, 4096, (64,), generator=g).tolist()  # same on every rank
    lo, hi = shard_sequences_by_kv_length(ctx, world)[rank]
    # every rank works on its own shard only; the only exchange is the final gather of results
    mine = torch.tensor([float(sum(ctx[lo:hi])), float(hi - lo)])
    gathered = [torch.zeros(2) for _ in range(world)]
    dist.all_gather(gathered, mine)
    if rank == 0:
        q.put((sum(ctx), len(ctx), [t.tolist() for t in gathered]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_shards_partition_the_batch():
    import torch.multiprocessing as mp

    ctx_mp = mp.get_context("spawn")
    q = ctx_mp.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx_mp.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    total, n, parts = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sum(p[0] for p in parts) == total and sum(p[1] for p in parts) == n
    assert abs(parts[0][0] - parts[1][0]) <= 2 * 4096


def test_lpt_sharding_is_a_balanced_partition():
    import random

    from flash_attention_factory_b200.sharding import shard_sequences_lpt

    rng = random.Random(7)
    lens = [max(16, min(32768, int(rng.lognormvariate(7.5, 1.0)))) for _ in range(1024)]
    for world in (1, 2, 4, 8):
        shards = shard_sequences_lpt(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(len(lens)))  # a partition
        assert all(s == sorted(s) for s in shards)
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.001 * sum(lens) / world
    assert shard_sequences_lpt([], 3) == [[], [], []]
    assert shard_sequences_lpt([5, 5, 5], 2) == [[0, 2], [1]]  # ties: lower id first, lower rank first


def test_library_split_agrees_with_the_python_sharding_helper():
    """pa_split_by_kv_length (the sub-batches of the pipelined host step, the sequence shards of the
    multi-GPU driver) and sharding.shard_sequences_by_kv_length are the same function."""
    import random

    from flash_attention_factory_b200 import _cabi, build
    from flash_attention_factory_b200.sharding import shard_sequences_by_kv_length

    build.build()
    rng = random.Random(4)
    cases = [[], [0, 0, 0], [5], [1] * 7, [100, 1, 1, 1, 100], [0, 7, 0, 0, 9, 0]]
    cases += [[rng.randint(0, 40000) for _ in range(rng.randint(1, 300))] for _ in range(30)]
    for lens in cases:
        for parts in (1, 2, 3, 4, 8):
            got = _cabi.split_by_kv_length(lens, parts)
            assert got == shard_sequences_by_kv_length(lens, parts), (lens[:10], parts)
            assert got[0][0] == 0 and got[-1][1] == len(lens)
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
