"""torch custom-op registration of the four operators (asynchronous form).

`import flash_attention_factory_b200.torch_ops` registers
`torch.ops.paged_attention_b200.{loop, reduce, fp8_loop, fp8_reduce}`: in-place operators on
torch's current stream that a serving stack can call from traced / graph-captured code
without the blocking, time-returning `run(...)` of the reference surface.  The argument order
is the reference's (paged_attention_loop/paged_attention_loop.cpp:21-38); `debug_output` is
dropped because nothing ever reads it.
"""
from __future__ import annotations

from typing import Optional

import torch

from .lib import paged_attention_fp8_loop, paged_attention_fp8_reduce, paged_attention_loop, paged_attention_reduce

_MUTATED = ("max_logits", "exp_sums", "tem_output", "output")


@torch.library.custom_op("paged_attention_b200::loop", mutates_args=_MUTATED)
def loop(max_logits: torch.Tensor, exp_sums: torch.Tensor, tem_output: torch.Tensor, output: torch.Tensor,
         query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
         context_lens: torch.Tensor, num_queries_per_tokens: int, sm_scale: float, block_size: int,
         max_context_len: int, alibi_slopes: torch.Tensor, sinks: Optional[torch.Tensor], softcap: float) -> None:
    paged_attention_loop.enqueue(max_logits, exp_sums, tem_output, output, None, query, key_cache, value_cache,
                                 block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size,
                                 max_context_len, alibi_slopes, sinks, softcap)


@torch.library.custom_op("paged_attention_b200::reduce", mutates_args=_MUTATED)
def reduce(max_logits: torch.Tensor, exp_sums: torch.Tensor, tem_output: torch.Tensor, output: torch.Tensor,
           query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
           context_lens: torch.Tensor, num_queries_per_tokens: int, sm_scale: float, block_size: int,
           max_context_len: int, alibi_slopes: torch.Tensor, sinks: Optional[torch.Tensor], softcap: float) -> None:
    paged_attention_reduce.enqueue(max_logits, exp_sums, tem_output, output, None, query, key_cache, value_cache,
                                   block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size,
                                   max_context_len, alibi_slopes, sinks, softcap)


@torch.library.custom_op("paged_attention_b200::fp8_loop", mutates_args=_MUTATED)
def fp8_loop(max_logits: torch.Tensor, exp_sums: torch.Tensor, tem_output: torch.Tensor, output: torch.Tensor,
             query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
             context_lens: torch.Tensor, num_queries_per_tokens: int, sm_scale: float, fp8_scale: float,
             block_size: int, max_context_len: int, alibi_slopes: torch.Tensor, sinks: Optional[torch.Tensor],
             softcap: float) -> None:
    paged_attention_fp8_loop.enqueue(max_logits, exp_sums, tem_output, output, None, query, key_cache,
                                     value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                                     fp8_scale, block_size, max_context_len, alibi_slopes, sinks, softcap)


@torch.library.custom_op("paged_attention_b200::fp8_reduce", mutates_args=_MUTATED)
def fp8_reduce(max_logits: torch.Tensor, exp_sums: torch.Tensor, tem_output: torch.Tensor, output: torch.Tensor,
               query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
               context_lens: torch.Tensor, num_queries_per_tokens: int, sm_scale: float, fp8_scale: float,
               block_size: int, max_context_len: int, alibi_slopes: torch.Tensor, sinks: Optional[torch.Tensor],
               softcap: float) -> None:
    paged_attention_fp8_reduce.enqueue(max_logits, exp_sums, tem_output, output, None, query, key_cache,
                                       value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                                       fp8_scale, block_size, max_context_len, alibi_slopes, sinks, softcap)
