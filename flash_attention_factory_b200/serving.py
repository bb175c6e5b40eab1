"""Per-sequence choice between the loop and the reduce variant for one decode batch.

No counterpart in the reference (its tests call one module for the whole batch,
test_paged.py:465-483).  A serving loop knows the context lengths on the host; short
sequences go to the single-pass loop kernel, long ones to the split-context pair, each as one
launch on its own stream.  The choice depends on the sequence alone
(`sharding.choose_variant`).  No tensor is gathered or scattered: each launch gets the list of
sequence ids it covers (`pa_params.seq_indices`) and works on the caller's tensors in place;
torch only provides the streams and events.

Two launches on two streams cost a fork and a join (about 17 us per call measured on B200, and
the programmatic-launch chain between consecutive calls is lost), which a handful of short
sequences cannot pay back: when the short sequences hold less than `fold_short_fraction` of the
batch's KV tokens they are folded into the split-context launch, which treats them as
one-partition items, and the batch is a single launch pair on the current stream.  With
`fold_short_fraction=0` the choice is strictly per sequence, and a sequence then gets the same
bits however the batch is composed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _cabi
from .lib import _shim
from .sharding import split_by_variant


@dataclass
class _SubBatch:
    index: torch.Tensor  # int32 [n] sequence ids of the sub-batch (device), passed as seq_indices
    count: int
    max_ctx: int


class AutoDecodePlan:
    """Index lists and scratch for one batch composition; reusable while the split of the
    batch into loop / reduce sequences stays the same (rebuild it when sequences join, leave
    or cross the length threshold)."""

    def __init__(self, context_lens_host: Sequence[int], num_heads: int, head_size: int, block_size: int,
                 max_blocks_per_seq: int, device, split_threshold_partitions: int = 2,
                 fold_short_fraction: float = 0.25):
        self.device = torch.device(device)
        self.psize = _cabi.partition_size(head_size)
        lens = [int(c) for c in context_lens_host]
        loop_idx, reduce_idx = split_by_variant(lens, self.psize, split_threshold_partitions)
        short_tokens = sum(lens[i] for i in loop_idx)
        if loop_idx and reduce_idx and short_tokens < fold_short_fraction * sum(lens):
            loop_idx, reduce_idx = [], list(range(len(lens)))  # one launch pair for the whole batch
        self.loop = self._make(loop_idx, lens)
        self.reduce = self._make(reduce_idx, lens)
        s = len(lens)
        # scratch of the split variant, indexed by the sequence id like every other tensor
        npart = max(1, (self.reduce.max_ctx + self.psize - 1) // self.psize) if self.reduce else 1
        self.max_logits = torch.empty(s, num_heads, npart, dtype=torch.float32, device=self.device)
        self.exp_sums = torch.empty_like(self.max_logits)
        self.tmp_out = torch.empty(s, num_heads, npart, head_size, dtype=torch.float16, device=self.device)
        self.alibi = torch.ones(num_heads, dtype=torch.float32, device=self.device)
        self.streams = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))

    def _make(self, idx, lens) -> Optional[_SubBatch]:
        if not idx:
            return None
        return _SubBatch(index=torch.tensor(idx, dtype=torch.int32, device=self.device), count=len(idx),
                         max_ctx=max(lens[i] for i in idx))


def paged_attention_auto(plan: AutoDecodePlan, out, query, key_cache, value_cache, block_tables,
                         context_lens, num_queries_per_tokens: int, sm_scale: float,
                         fp8_scale: float = 1.0, sinks=None) -> None:
    """Asynchronous decode attention of a whole batch: loop kernel for the plan's short
    sequences, split-context pair for its long ones.  Both launches work on the caller's
    tensors in place (each is given the list of sequence ids it covers), on two streams that
    fork from and join the current stream.  `out` [S, H, D] is written for every sequence."""
    fp8 = key_cache.dtype != torch.float16
    dev = plan.device

    def launch(sub: _SubBatch, variant: str) -> None:
        p = _shim.build_params(plan.max_logits, plan.exp_sums, plan.tmp_out, out, None, query, key_cache,
                               value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                               fp8_scale, key_cache.size(1), sub.max_ctx, plan.alibi, sinks, -1.0, fp8=fp8)
        if variant == "reduce":
            _shim.check_scratch(p, plan.max_logits, plan.exp_sums, plan.tmp_out)
        if sub.count != query.size(0):
            p.num_seqs = sub.count
            p.seq_indices = sub.index.data_ptr()
        _shim.enqueue_entry(f"launch_kernels_{'fp8_' if fp8 else ''}{variant}", p, dev)

    subs = [(sub, variant) for sub, variant in ((plan.loop, "loop"), (plan.reduce, "reduce")) if sub is not None]
    if len(subs) == 1:
        launch(*subs[0])  # one variant for the whole batch: the current stream, no fork and join
        return
    current = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(current)
    for (sub, variant), stream in zip(subs, plan.streams):
        with torch.cuda.stream(stream):
            stream.wait_event(fork)
            launch(sub, variant)
            done = torch.cuda.Event()
            done.record(stream)
        current.wait_event(done)
