"""CPU oracle for the paged-attention decode path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch on the CPU, what the reference computes on the
path `block table -> gathered K/V -> softmax(q.k) . v`.  It is the checker used by
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``; nothing in the shipped package imports it and the product never
falls back to it.

Parity status: PINNED.  ``paged_attention_ref`` reproduces the reference's own CPU
implementation (``attention_ref`` in test_paged.py:40-168 and ``attention_ref_fp8kv`` in
test_paged_fp8cache.py:38-168) and is checked against golden vectors produced by running
those very functions (``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py``).
The per-partition quantities of the split variant (``partition_stats_ref``) have no
reference test that fixes their values; they restate the kernel math of
paged_attention_reduce/paged_attention_kernel_v2.hpp:373-392,425-442,521-546 and are pinned
only through the identity merge(partition_stats) == paged_attention_ref.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def dequantize_cache(cache: torch.Tensor, fp8_scale: float = 1.0) -> torch.Tensor:
    """KV cache -> the fp16 values the kernels multiply with, times the tensor scale in fp32.

    The reference oracle casts the FP8 cache to the query dtype first
    (test_paged_fp8cache.py:80-81); every finite e5m2 / e4m3 code is exact in fp16.  The
    per-tensor scale multiplies the dequantised value once
    (paged_attention_fp8_loop/paged_attention_kernel_fp8_loop.hpp:333,545).
    """
    if cache.dtype == torch.uint8:  # raw bytes mean e5m2, as in the reference binding
        cache = cache.view(torch.float8_e5m2)
    x = cache.to(torch.float16).to(torch.float32)
    if torch.is_tensor(fp8_scale):
        # one scale per KV head (an extension over the reference's scalar): [..., kv_heads, head_size]
        x = x * fp8_scale.to(torch.float32).view(-1, 1)
    elif fp8_scale != 1.0:
        x = x * fp8_scale
    return x


def gather_sequence(cache_paged: torch.Tensor, block_table_row: torch.Tensor, context_len: int) -> torch.Tensor:
    """Logical tokens [0, context_len) of one sequence: [context_len, kv_heads, head_size].

    Token t lives in physical block block_table[t // block_size], row t % block_size
    (test_paged.py:184-193; paged_attention_loop/paged_attention_kernel_loop.hpp:278-297).
    """
    block_size = cache_paged.shape[1]
    n_blocks = (context_len + block_size - 1) // block_size
    ids = block_table_row[:n_blocks].to(torch.long)
    pages = cache_paged[ids]  # [n_blocks, block_size, kv_heads, head_size]
    return pages.reshape(n_blocks * block_size, *cache_paged.shape[2:])[:context_len]


def attention_one_sequence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           sinks: Optional[torch.Tensor], sm_scale: Optional[float],
                           softcap: float = 0.0, alibi_slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 attention of one decode token: q [H, D], k/v [T, HK, D] (fp32) -> [H, D] fp32.

    Follows attention_ref with upcast=True (test_paged.py:82-123,165): GQA repeat of K/V,
    scores = (q / sqrt(d)) . k, optional sink that joins the row maximum and the
    denominator but not the numerator, P . v in fp32.
    """
    h, d = q.shape
    t, hk, _ = k.shape
    g = h // hk
    if t == 0:
        return torch.zeros(h, d, dtype=torch.float32)
    k = k.repeat_interleave(g, dim=1)  # "b s h d -> b s (h g) d" (test_paged.py:85)
    v = v.repeat_interleave(g, dim=1)
    qs = q / math.sqrt(d) if sm_scale is None else q * sm_scale  # test_paged.py:89
    scores = torch.einsum("hd,shd->hs", qs, k)
    if softcap > 0:
        scores = (scores / softcap).tanh() * softcap  # test_paged.py:92-95
    if alibi_slopes is not None:
        # attn_bias of a decode token at position t-1 (test_paged.py:109-110 adds attn_bias; the
        # helper that would build it from slopes is not defined in the reference, so the usual
        # ALiBi form is taken: -slope * distance to the query position)
        dist = torch.arange(t, dtype=torch.float32) - float(t - 1)
        scores = scores + alibi_slopes.to(torch.float32).reshape(h, 1) * dist.reshape(1, t)
    smax = scores.max(dim=-1, keepdim=True).values
    if sinks is not None:
        sk = sinks.to(torch.float32).reshape(h, 1)
        m = torch.maximum(sk, smax)  # test_paged.py:116
        e = torch.exp(scores - m)
        denom = e.sum(dim=-1, keepdim=True) + torch.exp(sk - m)  # test_paged.py:118
    else:
        e = torch.exp(scores - smax)  # test_paged.py:121
        denom = e.sum(dim=-1, keepdim=True)
    p = e / denom
    return torch.einsum("hs,shd->hd", p, v)  # test_paged.py:165


def paged_attention_ref(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                        block_tables: torch.Tensor, context_lens: Sequence[int],
                        sm_scale: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
                        fp8_scale: float = 1.0, k_scales: Optional[torch.Tensor] = None,
                        v_scales: Optional[torch.Tensor] = None, softcap: float = 0.0,
                        alibi_slopes: Optional[torch.Tensor] = None,
                        k_block_scales: Optional[torch.Tensor] = None,
                        v_block_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reference result of all four entry points: fp16 [num_seqs, num_heads, head_size].

    `k_scales` / `v_scales` ([kv_heads] each) replace `fp8_scale` for K / V when given;
    `k_block_scales` / `v_block_scales` ([num_blocks, kv_heads] each, an extension over the
    reference's scalar) give every (block, head) its own scale: the dequantised cache is
    fp16(code) * scale[block, head].

    query fp16 [S, H, D]; caches [num_blocks, block_size, HK, D] in fp16, float8_e5m2,
    float8_e4m3fn or uint8 (= e5m2).  One sequence at a time, which bounds memory the way
    BASELINE-sized inputs need.  A context length of 0 yields zeros.
    """
    s, h, d = query.shape
    out = torch.zeros(s, h, d, dtype=torch.float16)
    lens = [int(c) for c in context_lens]

    def tokens_of(cache, block_scales, head_scales, i):
        x = dequantize_cache(gather_sequence(cache, block_tables[i], lens[i]),
                             1.0 if block_scales is not None else (fp8_scale if head_scales is None else head_scales))
        if block_scales is not None:
            bs = cache.shape[1]
            ids = block_tables[i, :(lens[i] + bs - 1) // bs].to(torch.long)
            per_token = block_scales.to(torch.float32)[ids].repeat_interleave(bs, dim=0)[:lens[i]]  # [ctx, kv_heads]
            x = x * per_token.unsqueeze(-1)
        return x

    for i in range(s):
        k = tokens_of(key_cache, k_block_scales, k_scales, i)
        v = tokens_of(value_cache, v_block_scales, v_scales, i)
        o = attention_one_sequence(query[i].to(torch.float32), k, v, sinks, sm_scale, softcap, alibi_slopes)
        out[i] = o.to(torch.float16)  # test_paged.py:168
    return out


def partition_stats_ref(query, key_cache, value_cache, block_tables, context_lens, partition_size: int,
                        sm_scale: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
                        fp8_scale: float = 1.0, max_num_partitions: Optional[int] = None):
    """What the first kernel of the split variant leaves in its scratch buffers.

    Returns (max_logits [S,H,NP] fp32, exp_sums [S,H,NP] fp32, tmp_out [S,H,NP,D] fp32,
    written [S,NP] bool).  For partition p of sequence i (tokens [p*P, min(ctx,(p+1)*P))):
    m_p = max(scores, sink if p == 0); l_p = sum exp(s - m_p) (+ exp(sink - m_p) if p == 0);
    tmp_out = sum (exp(s - m_p) / l_p) . v
    (paged_attention_reduce/paged_attention_kernel_v2.hpp:373-392,425-442,521-546).
    Entries with written == False are left untouched by the kernel (:577-579).
    """
    s, h, d = query.shape
    lens = [int(c) for c in context_lens]
    np_needed = max([(c + partition_size - 1) // partition_size for c in lens] + [1])
    npart = max_num_partitions if max_num_partitions is not None else np_needed
    max_logits = torch.zeros(s, h, npart)
    exp_sums = torch.zeros(s, h, npart)
    tmp_out = torch.zeros(s, h, npart, d)
    written = torch.zeros(s, npart, dtype=torch.bool)
    for i in range(s):
        k = dequantize_cache(gather_sequence(key_cache, block_tables[i], lens[i]), fp8_scale)
        v = dequantize_cache(gather_sequence(value_cache, block_tables[i], lens[i]), fp8_scale)
        hk = k.shape[1]
        g = h // hk
        q = query[i].to(torch.float32)
        qs = q / math.sqrt(d) if sm_scale is None else q * sm_scale
        for p in range(min(npart, (lens[i] + partition_size - 1) // partition_size)):
            lo, hi = p * partition_size, min(lens[i], (p + 1) * partition_size)
            kp = k[lo:hi].repeat_interleave(g, dim=1)
            vp = v[lo:hi].repeat_interleave(g, dim=1)
            scores = torch.einsum("hd,shd->hs", qs, kp)
            m = scores.max(dim=-1).values
            if sinks is not None and p == 0:
                m = torch.maximum(m, sinks.to(torch.float32))
            e = torch.exp(scores - m[:, None])
            l = e.sum(dim=-1)
            if sinks is not None and p == 0:
                l = l + torch.exp(sinks.to(torch.float32) - m)
            max_logits[i, :, p] = m
            exp_sums[i, :, p] = l
            tmp_out[i, :, p] = torch.einsum("hs,shd->hd", e / l[:, None], vp)
            written[i, p] = True
    return max_logits, exp_sums, tmp_out, written


def merge_partitions_ref(max_logits, exp_sums, tmp_out, context_lens, partition_size: int) -> torch.Tensor:
    """Second kernel of the split variant: fp16 [S, H, D].

    M = max_p m_p; w_p = l_p * exp(m_p - M); out = sum_p (w_p / sum w) * tmp_out[p], over
    p < ceil(ctx / P) only
    (paged_attention_reduce/paged_attention_kernel_v2.hpp:679,736-764,813-863,924-932).
    """
    s, h, npart = max_logits.shape
    d = tmp_out.shape[-1]
    out = torch.zeros(s, h, d, dtype=torch.float16)
    for i in range(s):
        n = min(npart, (int(context_lens[i]) + partition_size - 1) // partition_size)
        if n == 0:
            continue
        m = max_logits[i, :, :n].float()
        gmax = m.max(dim=-1, keepdim=True).values
        w = exp_sums[i, :, :n].float() * torch.exp(m - gmax)
        w = w / w.sum(dim=-1, keepdim=True)
        out[i] = torch.einsum("hp,hpd->hd", w, tmp_out[i, :, :n].float()).to(torch.float16)
    return out


def kv_bytes(context_lens: Sequence[int], num_kv_heads: int, head_size: int, elt_bytes: int) -> int:
    """Algorithmic HBM bytes of one call: every cached K and V element once."""
    return int(sum(int(c) for c in context_lens)) * num_kv_heads * head_size * 2 * elt_bytes


def reshape_and_cache_ref(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                          value_cache: torch.Tensor, slot_mapping: torch.Tensor, fp8_scale: float = 1.0,
                          k_scales: Optional[torch.Tensor] = None, v_scales: Optional[torch.Tensor] = None):
    """CPU statement of the cache append: returns new (key_cache, value_cache).

    Token t goes to flat slot slot_mapping[t] = block_id * block_size + row of the
    [num_blocks, block_size, kv_heads, head_size] cache (layout of
    paged_attention_loop/paged_attention_kernel_loop.hpp:50-51); negative slots are skipped.
    The cast is the reference fixture's: `x.to(fp8_dtype)` on the fp16 data
    (test_paged_fp8cache.py:201-203), after dividing by the per-tensor scale in fp32.
    `k_scales` / `v_scales` (an extension over the reference's single scalar) replace the
    scalar: shape [kv_heads] = one scale per KV head, [num_blocks, kv_heads] = one per block
    and KV head, the inverse of what `paged_attention_ref` multiplies by.
    """
    kc, vc = key_cache.clone(), value_cache.clone()
    dt = kc.dtype
    flat_k = kc.view(-1, *kc.shape[2:])
    flat_v = vc.view(-1, *vc.shape[2:])
    block_size = kc.shape[1]

    def divisor(scales, slot):
        if scales is None:
            return fp8_scale
        per_head = scales if scales.dim() == 1 else scales[slot // block_size]
        return per_head.float().view(-1, 1)  # [kv_heads, 1] against a [kv_heads, head_size] row

    for t, slot in enumerate(slot_mapping.tolist()):
        if slot < 0 or slot >= flat_k.shape[0]:
            continue
        if dt == torch.float16:
            flat_k[slot], flat_v[slot] = key[t], value[t]
        else:
            flat_k[slot] = (key[t].float() / divisor(k_scales, slot)).to(dt)
            flat_v[slot] = (value[t].float() / divisor(v_scales, slot)).to(dt)
    return kc, vc


def paged_attention_ref_fp16(query, key_cache, value_cache, block_tables, context_lens,
                             sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The reference's second oracle: the same attention in pure fp16 with reordered scaling
    (`attention_ref(..., upcast=False, reorder_ops=True)`, test_paged.py:88-91,432-447).

    Its error against the fp32 oracle is the yardstick of the reference's acceptance test:
    max|out - ref| <= 3 * max|out_fp16 - ref| + 1e-5 (test_paged.py:603-604).
    """
    s, h, d = query.shape
    out = torch.zeros(s, h, d, dtype=torch.float16)
    for i in range(s):
        n = int(context_lens[i])
        if n == 0:
            continue
        k = gather_sequence(key_cache, block_tables[i], n).to(torch.float16)  # test_paged_fp8cache.py:80-81
        v = gather_sequence(value_cache, block_tables[i], n).to(torch.float16)
        g = h // k.shape[1]
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        scores = torch.einsum("hd,shd->hs", query[i], k / math.sqrt(d))  # reorder_ops: k is scaled
        sf = scores.to(torch.float32)  # test_paged.py:112
        smax = sf.max(dim=-1, keepdim=True).values
        if sinks is not None:
            sk = sinks.reshape(h, 1)
            m = torch.maximum(sk, smax)
            e = torch.exp(sf - m)
            denom = e.sum(dim=-1, keepdim=True) + torch.exp(sk - m)
        else:
            e = torch.exp(sf - smax)
            denom = e.sum(dim=-1, keepdim=True)
        p = (e / denom).to(torch.float16)  # test_paged.py:119,123
        out[i] = torch.einsum("hs,shd->hd", p, v)
    return out
