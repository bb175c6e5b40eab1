"""``paged_attention_reduce.run``: fp16 KV cache, split-context (attention + merge kernel).

Drop-in for the reference extension module of the same name
(paged_attention_reduce/paged_attention_reduce.cpp:21-38,82-84); same 17 positional arguments, same
return value (device microseconds: [attention, merge]).
"""
from __future__ import annotations

from . import _shim

ENTRY = _ENTRY = "launch_kernels_reduce"


def run(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
        block_tables, context_lens, num_queries_per_tokens, sm_scale, block_size, max_context_len,
        alibi_slopes, sinks, softcap):
    p = _shim.build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                           value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                           1.0, block_size, max_context_len, alibi_slopes, sinks, softcap, fp8=False)
    _shim.check_scratch(p, max_logits, exp_sums, tem_output)
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
    _shim.check_scratch(p, max_logits, exp_sums, tem_output)
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
