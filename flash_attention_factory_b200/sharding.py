"""Host-side work partitioning for multi-GPU decode (no counterpart in the reference, which is
single-device: each call builds its own queue, launch_kernels_loop.h:32-34).

Every (sequence, KV head) is an independent unit of the path, so a batch shards across GPUs
with no exchange step: by sequence, balanced on cumulative KV length, and additionally by KV
head when there are fewer long sequences than GPUs.  Each GPU owns the KV pool, block tables,
queries and outputs of its shard; the only cross-GPU step is an optional gather of the (small)
outputs after the operator has finished.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_sequences_by_kv_length(context_lens: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [lo, hi) sequence ranges, one per rank, balanced on cumulative KV length.

    Rank r gets the sequences whose cumulative length (inclusive) falls in
    (r*T/W, (r+1)*T/W], T being the total; ranges are disjoint, ordered and cover the batch.
    Depends only on the lengths, so every rank computes the same answer without talking.
    """
    if world_size < 1:
        raise ValueError("world_size must be positive")
    n = len(context_lens)
    total = sum(int(c) for c in context_lens)
    bounds, cum, rank = [0], 0, 0
    for i, c in enumerate(context_lens):
        cum += int(c)
        # close every shard whose upper limit this sequence reaches
        while rank < world_size - 1 and cum * world_size >= (rank + 1) * total and total > 0:
            bounds.append(i + 1)
            rank += 1
    while len(bounds) < world_size:
        bounds.append(n)
    bounds.append(n)
    return [(bounds[r], bounds[r + 1]) for r in range(world_size)]


def shard_sequences_lpt(context_lens: Sequence[int], world_size: int) -> List[List[int]]:
    """Sequence ids per rank, balanced by "longest first to the lightest rank".

    Not contiguous, but balanced to within a fraction of one sequence where the contiguous
    split can be off by a whole long sequence (1024 log-normal contexts on 8 ranks: heaviest
    rank 0.01 % over the mean instead of 2.7 %).  Deterministic: ties go to the lower id /
    lower rank, so every rank computes the same answer.  Ids are returned in ascending order.
    """
    if world_size < 1:
        raise ValueError("world_size must be positive")
    loads = [0] * world_size
    shards: List[List[int]] = [[] for _ in range(world_size)]
    for i in sorted(range(len(context_lens)), key=lambda j: (-int(context_lens[j]), j)):
        r = min(range(world_size), key=lambda k: (loads[k], k))
        loads[r] += int(context_lens[i])
        shards[r].append(i)
    return [sorted(s) for s in shards]


def shard_kv_heads(num_kv_heads: int, world_size: int) -> List[Tuple[int, int]]:
    """[lo, hi) KV-head ranges per rank for head sharding (very long contexts, few sequences).

    Rank r reads key_cache[:, :, lo:hi, :] and writes the disjoint slice
    out[:, lo*G:hi*G, :]; concatenation of the slices is the full output, no reduction.
    """
    if world_size < 1 or num_kv_heads < 1:
        raise ValueError("world_size and num_kv_heads must be positive")
    base, extra = divmod(num_kv_heads, world_size)
    out, lo = [], 0
    for r in range(world_size):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def choose_variant(context_len: int, partition_size: int = 512, split_threshold_partitions: int = 2) -> str:
    """Loop or reduce for one sequence, from its own length only.

    Depending on nothing but the sequence itself keeps the choice, and therefore the result
    bits, identical however the batch is sharded.  Contexts that fit one partition take the
    single-pass loop kernel (one launch, no scratch traffic); from `split_threshold_partitions`
    partitions on, the persistent split-context kernel balances ragged lengths better than one
    cluster per (sequence, KV-head group) can (measured on B200: 6.2 vs 4.7 TB/s on log-normal
    contexts).
    """
    partitions = (int(context_len) + partition_size - 1) // partition_size
    return "reduce" if partitions >= split_threshold_partitions else "loop"


def split_by_variant(context_lens: Sequence[int], partition_size: int = 512,
                     split_threshold_partitions: int = 2) -> Tuple[List[int], List[int]]:
    """Indices of the sequences that go to the loop launch and to the reduce launch."""
    loop_idx, reduce_idx = [], []
    for i, c in enumerate(context_lens):
        (reduce_idx if choose_variant(c, partition_size, split_threshold_partitions) == "reduce"
         else loop_idx).append(i)
    return loop_idx, reduce_idx
