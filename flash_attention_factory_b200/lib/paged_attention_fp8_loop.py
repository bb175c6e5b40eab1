"""``paged_attention_fp8_loop.run``: FP8 KV cache, single pass.

Drop-in for the reference extension module of the same name
(paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:21-39,84-86); same 18 positional
arguments (``fp8_scale`` after ``sm_scale``).  The cache format follows the tensor
dtype: ``float8_e5m2`` or plain ``uint8`` mean e5m2 (what the reference binding fixes),
``float8_e4m3fn`` means e4m3.
"""
from __future__ import annotations

from . import _shim

ENTRY = _ENTRY = "launch_kernels_fp8_loop"


def run(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
        block_tables, context_lens, num_queries_per_tokens, sm_scale, fp8_scale, block_size,
        max_context_len, alibi_slopes, sinks, softcap):
    p = _shim.build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                           value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                           fp8_scale, block_size, max_context_len, alibi_slopes, sinks, softcap,
                           fp8=True)
    return _shim.run_entry(_ENTRY, p, query.device)


def params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
           block_tables, context_lens, num_queries_per_tokens, sm_scale, fp8_scale, block_size,
           max_context_len, alibi_slopes, sinks, softcap, *, k_scale_per_head=None, v_scale_per_head=None,
           use_alibi=False, use_softcap=False, k_scale_per_block=None, v_scale_per_block=None):
    """The checked argument block (`pa_params`) of an ``enqueue`` call with these arguments,
    for callers that launch many steps on the same tensors (`host_io.DecodeStepIO.bind`)."""
    p = _shim.build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                           value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                           fp8_scale, block_size, max_context_len, alibi_slopes, sinks, softcap,
                           fp8=True, k_scale_per_head=k_scale_per_head, v_scale_per_head=v_scale_per_head,
                           use_alibi=use_alibi, use_softcap=use_softcap, k_scale_per_block=k_scale_per_block,
                           v_scale_per_block=v_scale_per_block)
    return p


def enqueue(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
            block_tables, context_lens, num_queries_per_tokens, sm_scale, fp8_scale, block_size,
            max_context_len, alibi_slopes, sinks, softcap, *, k_scale_per_head=None, v_scale_per_head=None,
            use_alibi=False, use_softcap=False, k_scale_per_block=None, v_scale_per_block=None):
    """Same arguments as ``run`` but asynchronous on the current stream (returns nothing).

    ``k_scale_per_head`` / ``v_scale_per_head`` (float32 [num_kv_heads], optional, no reference
    counterpart) replace the scalar ``fp8_scale`` for K / V with one scale per KV head;
    ``k_scale_per_block`` / ``v_scale_per_block`` (float32 [num_blocks, num_kv_heads]) with one per
    block and head."""
    p = params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache, value_cache,
               block_tables, context_lens, num_queries_per_tokens, sm_scale, fp8_scale, block_size,
               max_context_len, alibi_slopes, sinks, softcap, k_scale_per_head=k_scale_per_head,
               v_scale_per_head=v_scale_per_head, use_alibi=use_alibi, use_softcap=use_softcap,
               k_scale_per_block=k_scale_per_block, v_scale_per_block=v_scale_per_block)
    _shim.enqueue_entry(_ENTRY, p, query.device)
