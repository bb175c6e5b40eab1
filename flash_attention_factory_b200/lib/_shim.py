"""Shared body of the four ``run`` functions.

Unpacks torch tensors exactly as the reference's pybind shims do
(paged_attention_loop/paged_attention_loop.cpp:44-79,
paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:44-81): sizes come from
the tensor shapes, pointers from ``data_ptr()``, int32 tables are read as
uint32.  torch is used for device memory and the current stream only.
"""
from __future__ import annotations

import torch

from .. import _cabi


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _kv_dtype_of(cache: torch.Tensor, fp8: bool) -> int:
    if not fp8:
        _require(cache.dtype == torch.float16, f"key/value cache must be float16, got {cache.dtype}")
        return _cabi.KV_F16
    if cache.dtype == torch.float8_e4m3fn:
        return _cabi.KV_FP8_E4M3
    # uint8 storage means e5m2, the format the reference binding hard-wires
    # (paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:43)
    _require(cache.dtype in (torch.float8_e5m2, torch.uint8),
             f"FP8 cache must be float8_e5m2, float8_e4m3fn or uint8, got {cache.dtype}")
    return _cabi.KV_FP8_E5M2


def build_params(max_logits, exp_sums, tem_output, output, debug_output, query, key_cache,
                 value_cache, block_tables, context_lens, num_queries_per_tokens, sm_scale,
                 fp8_scale, block_size, max_context_len, alibi_slopes, sinks, softcap,
                 fp8: bool, k_scale_per_head=None, v_scale_per_head=None,
                 use_alibi: bool = False, use_softcap: bool = False,
                 k_scale_per_block=None, v_scale_per_block=None) -> _cabi.PaParams:
    """Validates what the reference's ``data_ptr<float>()`` calls would and fills pa_params.

    ``debug_output``, ``alibi_slopes``, ``softcap`` are accepted and ignored like in the
    reference (paged_attention_kernel_loop.hpp:175-178,329-342).
    """
    _require(query.is_cuda, "paged attention needs CUDA tensors (no CPU fallback exists)")
    # the reference's data_ptr<float>() calls reject other dtypes (paged_attention_loop.cpp:47-52)
    for name, t in (("max_logits", max_logits), ("exp_sums", exp_sums), ("alibi_slopes", alibi_slopes),
                    ("debug_output", debug_output)):
        if name == "debug_output" and t is None:
            continue  # callers of this package that have no debug tensor pass None
        _require(t.dtype == torch.float32, f"expected scalar type Float but found {t.dtype} ({name})")
    _require(query.dtype == torch.float16 and output.dtype == torch.float16,
             "query and output must be float16")
    _require(block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32,
             "block_tables and context_lens must be int32")
    _require(query.dim() == 3 and key_cache.dim() == 4 and block_tables.dim() == 2
             and max_logits.dim() == 3, "unexpected tensor rank")
    _require(key_cache.shape == value_cache.shape and key_cache.dtype == value_cache.dtype,
             "key_cache and value_cache must have the same shape and dtype")
    tensors = [max_logits, exp_sums, tem_output, output, query, key_cache, value_cache,
               block_tables, context_lens]
    if sinks is not None:
        _require(sinks.dtype == torch.float16, "sinks must be float16")
        tensors.append(sinks)
    for t in tensors:
        _require(t.is_contiguous(), "all tensors must be contiguous")
        _require(t.device == query.device, "all tensors must be on the same device")
    _require(key_cache.size(1) == block_size, "block_size does not match key_cache.size(1)")
    _require(key_cache.size(3) == query.size(2), "head_size of cache and query differ")
    _require(context_lens.numel() == query.size(0) and block_tables.size(0) == query.size(0),
             "context_lens / block_tables do not match the number of sequences")

    p = _cabi.PaParams()
    p.out = output.data_ptr()
    p.max_logits = max_logits.data_ptr()
    p.exp_sums = exp_sums.data_ptr()
    p.tmp_out = tem_output.data_ptr()
    p.query = query.data_ptr()
    p.key_cache = key_cache.data_ptr()
    p.value_cache = value_cache.data_ptr()
    p.sinks = sinks.data_ptr() if sinks is not None else None
    p.block_tables = block_tables.data_ptr()
    p.context_lens = context_lens.data_ptr()
    p.num_seqs = query.size(0)
    p.num_heads = query.size(1)
    p.head_size = query.size(2)
    p.num_kv_heads = key_cache.size(2)
    p.max_num_partitions = max_logits.size(2)
    p.max_blocks_per_seq = block_tables.size(1)
    p.block_size = int(block_size)
    p.num_queries_per_tokens = int(num_queries_per_tokens)
    p.max_context_len = max(0, min(int(max_context_len), 0xFFFFFFFF))
    p.num_blocks = key_cache.size(0)
    p.sm_scale = float(sm_scale)
    p.fp8_scale = float(fp8_scale)
    p.kv_dtype = _kv_dtype_of(key_cache, fp8)
    for name, t in (("k_scale_per_head", k_scale_per_head), ("v_scale_per_head", v_scale_per_head)):
        if t is not None:
            _require(fp8, "per-head scales belong to the FP8 operators")
            _require(t.dtype == torch.float32 and t.is_contiguous() and t.device == query.device
                     and t.numel() == key_cache.size(2), f"{name} must be float32 [num_kv_heads] on the device")
            setattr(p, name, t.data_ptr())
    for name, t in (("k_scale_per_block", k_scale_per_block), ("v_scale_per_block", v_scale_per_block)):
        if t is not None:
            _require(fp8, "per-block scales belong to the FP8 operators")
            _require(t.dtype == torch.float32 and t.is_contiguous() and t.device == query.device
                     and tuple(t.shape) == (key_cache.size(0), key_cache.size(2)),
                     f"{name} must be float32 [num_blocks, num_kv_heads] on the device")
            setattr(p, name, t.data_ptr())
    # opt-in only: by default alibi_slopes and softcap are ignored, as in the reference
    if use_alibi:
        _require(alibi_slopes.is_cuda and alibi_slopes.is_contiguous()
                 and alibi_slopes.numel() == query.size(1), "alibi_slopes must be float32 [num_heads] on the device")
        p.alibi_slopes = alibi_slopes.data_ptr()
    if use_softcap and softcap > 0:
        p.softcap = float(softcap)
    return p


def check_scratch(p: _cabi.PaParams, max_logits, exp_sums, tem_output) -> None:
    """The split variant writes [S, H, NP] and [S, H, NP, D] scratch: check the extents."""
    s, h, npart, d = p.num_seqs, p.num_heads, p.max_num_partitions, p.head_size
    _require(tuple(max_logits.shape) == (s, h, npart) and tuple(exp_sums.shape) == (s, h, npart),
             "max_logits / exp_sums must be [num_seqs, num_heads, max_num_partitions]")
    _require(tem_output.dtype == torch.float16 and tem_output.numel() >= s * h * npart * d,
             "tem_output must be float16 [num_seqs, num_heads, max_num_partitions, head_size]")


def run_entry(entry: str, p: _cabi.PaParams, device: torch.device) -> list[float]:
    """Blocking launch on torch's current stream; returns device microseconds per kernel."""
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        return _cabi.launch(entry, p, stream, timed=True)


def enqueue_entry(entry: str, p: _cabi.PaParams, device: torch.device) -> None:
    """Asynchronous launch on torch's current stream (no timing, no host sync)."""
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _cabi.launch(entry, p, stream, timed=False)
