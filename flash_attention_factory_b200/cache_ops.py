"""Writing new tokens into the paged KV cache (the step before decode attention).

`reshape_and_cache` scatters this step's K/V rows into the cache the attention operators read
([num_blocks, block_size, num_kv_heads, head_size]) and casts them to the cache type on the
way.  The reference builds its caches on the host with torch casts
(test_paged_fp8cache.py:180-203); this is the device-side counterpart of that fixture code.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi


def _kv_dtype(cache: torch.Tensor) -> int:
    if cache.dtype == torch.float16:
        return _cabi.KV_F16
    if cache.dtype == torch.float8_e4m3fn:
        return _cabi.KV_FP8_E4M3
    if cache.dtype in (torch.float8_e5m2, torch.uint8):
        return _cabi.KV_FP8_E5M2
    raise RuntimeError(f"unsupported cache dtype {cache.dtype}")


def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, slot_mapping: torch.Tensor, fp8_scale: float = 1.0, *,
                      k_scale_per_head=None, v_scale_per_head=None,
                      k_scale_per_block=None, v_scale_per_block=None) -> None:
    """key/value fp16 [T, HK, D] -> caches at slot_mapping[t] = block_id * block_size + row.

    Negative slots are skipped.  FP8 caches store round-to-nearest-even(x / scale),
    saturating, where scale is `fp8_scale` or, when given, the entry of the token's KV head
    in `k_scale_per_head` / `v_scale_per_head` (float32 [HK]) or of its block and KV head in
    `k_scale_per_block` / `v_scale_per_block` (float32 [num_blocks, HK]); the attention
    operators take the same scale arguments.  Asynchronous on torch's current stream.
    """
    if not key.is_cuda:
        raise RuntimeError("reshape_and_cache needs CUDA tensors (no CPU fallback exists)")
    for t in (key, value, key_cache, value_cache, slot_mapping):
        if not t.is_contiguous() or t.device != key.device:
            raise RuntimeError("all tensors must be contiguous and on the same device")
    if key.dtype != torch.float16 or value.dtype != torch.float16 or key.shape != value.shape:
        raise RuntimeError("key and value must be float16 tensors of the same shape")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != key.size(0):
        raise RuntimeError("slot_mapping must be int64 with one entry per token")
    if key_cache.shape != value_cache.shape or key_cache.dtype != value_cache.dtype:
        raise RuntimeError("key_cache and value_cache must match")
    if key_cache.dim() != 4 or tuple(key_cache.shape[2:]) != tuple(key.shape[1:]):
        raise RuntimeError("cache must be [num_blocks, block_size, num_kv_heads, head_size]")
    p = _cabi.PaCacheWriteParams()
    p.key, p.value = key.data_ptr(), value.data_ptr()
    p.key_cache, p.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    p.slot_mapping = slot_mapping.data_ptr()
    p.num_tokens, p.num_kv_heads, p.head_size = key.size(0), key.size(1), key.size(2)
    p.block_size, p.num_blocks = key_cache.size(1), key_cache.size(0)
    p.fp8_scale = float(fp8_scale)
    p.kv_dtype = _kv_dtype(key_cache)
    per_head, per_block = (key.size(1),), (key_cache.size(0), key.size(1))
    for name, t, shape in (("k_scale_per_head", k_scale_per_head, per_head),
                           ("v_scale_per_head", v_scale_per_head, per_head),
                           ("k_scale_per_block", k_scale_per_block, per_block),
                           ("v_scale_per_block", v_scale_per_block, per_block)):
        if t is None:
            continue
        if (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()
                or t.device != key.device):
            raise RuntimeError(f"{name} must be a contiguous float32 tensor of shape {shape} on the cache's device")
        setattr(p, name, t.data_ptr())
    lib = _cabi.load_library()
    with torch.cuda.device(key.device):
        stream = torch.cuda.current_stream(key.device).cuda_stream
        _cabi.check(lib.pa_reshape_and_cache(ctypes.byref(p), ctypes.c_void_p(stream)))
