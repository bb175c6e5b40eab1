"""Per-sequence choice between the loop and the reduce variant for one decode batch.

No counterpart in the reference (its tests call one module for the whole batch,
test_paged.py:465-483).  A serving loop knows the context lengths on the host; short
sequences go to the single-pass loop kernel, long ones to the split-context pair, each as one
launch on its own stream.  The choice depends on the sequence alone
(`sharding.choose_variant`), so a sequence gets the same bits however the batch is sharded.
torch is used for the gathers / scatters of the small per-sequence tensors and for streams.
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
    index: torch.Tensor        # int64 [n] positions in the full batch (device)
    query: torch.Tensor        # fp16 [n, H, D]
    out: torch.Tensor          # fp16 [n, H, D]
    block_tables: torch.Tensor # int32 [n, MB']
    context_lens: torch.Tensor # int32 [n]
    max_ctx: int
    max_logits: Optional[torch.Tensor] = None
    exp_sums: Optional[torch.Tensor] = None
    tmp_out: Optional[torch.Tensor] = None


class AutoDecodePlan:
    """Buffers and index sets for one batch composition; reusable while the lengths' split
    into loop / reduce sequences stays the same (rebuild it when sequences join or leave)."""

    def __init__(self, context_lens_host: Sequence[int], num_heads: int, head_size: int, block_size: int,
                 max_blocks_per_seq: int, device, split_threshold_partitions: int = 2):
        self.device = torch.device(device)
        self.psize = _cabi.partition_size(head_size)
        self.block_size = block_size
        lens = [int(c) for c in context_lens_host]
        loop_idx, reduce_idx = split_by_variant(lens, self.psize, split_threshold_partitions)
        self.loop = self._make(loop_idx, lens, num_heads, head_size, max_blocks_per_seq, scratch=False)
        self.reduce = self._make(reduce_idx, lens, num_heads, head_size, max_blocks_per_seq, scratch=True)
        self.streams = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))

    def _make(self, idx, lens, h, d, mb, scratch) -> Optional[_SubBatch]:
        if not idx:
            return None
        n, dev = len(idx), self.device
        max_ctx = max(lens[i] for i in idx)
        mb_sub = min(mb, max(1, (max_ctx + self.block_size - 1) // self.block_size))
        sb = _SubBatch(
            index=torch.tensor(idx, dtype=torch.int64, device=dev),
            query=torch.empty(n, h, d, dtype=torch.float16, device=dev),
            out=torch.empty(n, h, d, dtype=torch.float16, device=dev),
            block_tables=torch.empty(n, mb_sub, dtype=torch.int32, device=dev),
            context_lens=torch.empty(n, dtype=torch.int32, device=dev),
            max_ctx=max_ctx)
        if scratch:
            npart = max(1, (max_ctx + self.psize - 1) // self.psize)
            sb.max_logits = torch.empty(n, h, npart, dtype=torch.float32, device=dev)
            sb.exp_sums = torch.empty_like(sb.max_logits)
            sb.tmp_out = torch.empty(n, h, npart, d, dtype=torch.float16, device=dev)
        return sb


def paged_attention_auto(plan: AutoDecodePlan, out, query, key_cache, value_cache, block_tables,
                         context_lens, num_queries_per_tokens: int, sm_scale: float,
                         fp8_scale: float = 1.0, sinks=None) -> None:
    """Asynchronous decode attention of a whole batch: loop kernel for the plan's short
    sequences, split-context pair for its long ones, on two streams that fork from and join
    the current stream.  `out` [S, H, D] is written for every sequence."""
    fp8 = key_cache.dtype != torch.float16
    dev = plan.device
    current = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(current)
    dummy_f32 = torch.empty(1, 1, 1, dtype=torch.float32, device=dev)
    alibi = torch.empty(query.size(1), dtype=torch.float32, device=dev)
    for sub, variant, stream in ((plan.loop, "loop", plan.streams[0]), (plan.reduce, "reduce", plan.streams[1])):
        if sub is None:
            continue
        with torch.cuda.stream(stream):
            stream.wait_event(fork)
            torch.index_select(query, 0, sub.index, out=sub.query)
            torch.index_select(context_lens, 0, sub.index, out=sub.context_lens)
            sub.block_tables.copy_(block_tables.index_select(0, sub.index)[:, : sub.block_tables.size(1)])
            ml = sub.max_logits if sub.max_logits is not None else dummy_f32
            es = sub.exp_sums if sub.exp_sums is not None else dummy_f32
            tmp = sub.tmp_out if sub.tmp_out is not None else sub.out
            p = _shim.build_params(ml, es, tmp, sub.out, None, sub.query, key_cache, value_cache,
                                   sub.block_tables, sub.context_lens, num_queries_per_tokens, sm_scale,
                                   fp8_scale, key_cache.size(1), sub.max_ctx, alibi, sinks, -1.0, fp8=fp8)
            if variant == "reduce":
                _shim.check_scratch(p, ml, es, tmp)
            _shim.enqueue_entry(f"launch_kernels_{'fp8_' if fp8 else ''}{variant}", p, dev)
            out.index_copy_(0, sub.index, sub.out)
            done = torch.cuda.Event()
            done.record(stream)
        current.wait_event(done)
