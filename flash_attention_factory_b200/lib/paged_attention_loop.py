"""``paged_attention_loop.run``: fp16 KV cache, single pass.

Drop-in for the reference extension module of the same name
(paged_attention_loop/paged_attention_loop.cpp:21-38,82-84); same 17 positional arguments, same
return value (device microseconds: [kernel]).
"""
from __future__ import annotations

from . import _shim

ENTRY = _ENTRY = "launch_kernels_loop"


def run(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
        block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size, max_context_len,
        alibi_slopes, sinks, softcap):
    p = _shim.build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                           value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                           1.0, block_size, max_context_len, alibi_slopes, sinks, softcap, fp8=False)
    return _shim.run_entry(_ENTRY, p, query.device)


def params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
           block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size,
           max_context_len, alibi_slopes, sinks, softcap, *, use_alibi=False, use_softcap=False):
    """The checked argument block (`pa_params`) of an ``enqueue`` call with these arguments,
    for callers that launch many steps on the same tensors (`host_io.DecodeStepIO.bind`)."""
    p = _shim.build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                           value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                           1.0, block_size, max_context_len, alibi_slopes, sinks, softcap, fp8=False,
                           use_alibi=use_alibi, use_softcap=use_softcap)
    return p


def enqueue(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
            block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size,
            max_context_len, alibi_slopes, sinks, softcap, *, use_alibi=False, use_softcap=False):
    """Same arguments as ``run`` but asynchronous on the current stream (returns nothing).

    ``use_alibi`` / ``use_softcap`` (no reference counterpart) make ``alibi_slopes`` / ``softcap``
    live; by default both are ignored, as the reference ignores them."""
    p = params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
               block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size, max_context_len,
               alibi_slopes, sinks, softcap, use_alibi=use_alibi, use_softcap=use_softcap)
    _shim.enqueue_entry(_ENTRY, p, query.device)
