"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own CPU code.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It loads the reference's two test files (test_paged.py, test_paged_fp8cache.py) with
the missing ``lib`` extension package stubbed out, builds fixtures with the reference's
own generators (`_generate_block_kvcache`, `_generate_block_fp8kvcache`,
`generate_random_padding_mask`) under the reference's seed (torch.random.manual_seed(0),
test_paged.py:291) following the order of random draws of its test body
(test_paged.py:298-341), and stores inputs together with the outputs of the reference's
`attention_ref` / `attention_ref_fp8kv` called exactly as the test calls them
(test_paged.py:418-447): `out_ref` (fp32 math) and `out_pt` (fp16 math, reordered).
Each case is one compressed .npz of a few hundred KB; fp16 / fp8 tensors are stored as
their raw uint16 / uint8 bits.
"""
from __future__ import annotations

import importlib.util
import math
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# (name, fp8_dtype or None, batch, nheads, nheads_k, d, seqlen_k, block, sinks, varlen)
CASES = [
    ("f16_b2_h8k2_d128_s339_bs64_sink_varlen", None, 2, 8, 2, 128, 339, 64, True, True),
    ("f16_b1_h8k1_d128_s1024_bs64_nosink_full", None, 1, 8, 1, 128, 1024, 64, False, False),
    ("f16_b2_h6k2_d64_s800_bs64_nosink_varlen", None, 2, 6, 2, 64, 800, 64, False, True),
    ("f16_b2_h10k2_d64_s256_bs64_sink_full", None, 2, 10, 2, 64, 256, 64, True, False),
    ("f16_b2_h4k4_d128_s200_bs16_nosink_varlen", None, 2, 4, 4, 128, 200, 16, False, True),
    ("e5m2_b2_h14k2_d128_s799_bs64_sink_varlen", "float8_e5m2", 2, 14, 2, 128, 799, 64, True, True),
    ("e5m2_b1_h12k2_d64_s2048_bs64_nosink_full", "float8_e5m2", 1, 12, 2, 64, 2048, 64, False, False),
    ("e5m2_b2_h8k2_d128_s530_bs16_nosink_varlen", "float8_e5m2", 2, 8, 2, 128, 530, 16, False, True),
]


def load_reference_module(path: Path, name: str):
    """Imports a reference test file; `from lib import ...` is satisfied by empty stubs."""
    lib = types.ModuleType("lib")
    for sub in ("paged_attention_loop", "paged_attention_reduce", "paged_attention_fp8_loop",
                "paged_attention_fp8_reduce"):
        mod = types.ModuleType(f"lib.{sub}")
        setattr(lib, sub, mod)
        sys.modules[f"lib.{sub}"] = mod
    sys.modules["lib"] = lib
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e5m2, torch.float8_e4m3fn):
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def make_case(ref16, ref8, name, fp8_dtype, batch, nheads, nheads_k, d, seqlen_k, block, sinks, varlen):
    from einops import repeat

    torch.random.manual_seed(0)  # test_paged.py:291
    dtype = torch.float16
    q = torch.randn(batch, 1, nheads, d, dtype=dtype)  # test_paged.py:298
    if fp8_dtype is None:
        k_cache, v_cache, block_table, k_paged, v_paged, _ = ref16._generate_block_kvcache(
            seqlen_k, block, batch, nheads_k, d, "cpu", dtype)
        attention = ref16.attention_ref
    else:
        k_cache, v_cache, block_table, k_paged, v_paged, _ = ref8._generate_block_fp8kvcache(
            seqlen_k, block, batch, nheads_k, d, "cpu", dtype, getattr(torch, fp8_dtype))
        attention = ref8.attention_ref_fp8kv
    # the test draws cache_seqlens here although it never uses them (test_paged.py:320-331)
    torch.randint(1, seqlen_k + 1, (batch,), dtype=torch.int32)
    gen_mask = (ref16 if fp8_dtype is None else ref8).generate_random_padding_mask
    key_padding_mask, seq_lens = gen_mask(seqlen_k, batch, "cpu", mode="random" if varlen else "full")
    k_rep = repeat(k_cache, "b s h d -> b s (h g) d", g=nheads // nheads_k)  # test_paged.py:408-409
    v_rep = repeat(v_cache, "b s h d -> b s (h g) d", g=nheads // nheads_k)
    learnable_sinks = torch.ones(nheads, dtype=dtype) * 10 if sinks else None  # test_paged.py:414-417
    mask = key_padding_mask if varlen else None
    out_ref, _, _ = attention(q, k_rep, v_rep, learnable_sinks, None, mask, None, 0.0, None,
                              causal=False, window_size=(-1, -1), key_leftpad=None)
    out_pt, _, _ = attention(q, k_rep, v_rep, learnable_sinks, None, mask, None, 0.0, None,
                             causal=False, window_size=(-1, -1), upcast=False, reorder_ops=True,
                             key_leftpad=None)
    context_lens = seq_lens.squeeze(1).to(torch.int32)
    arrays = dict(
        query=bits(q.view(batch, nheads, d)),
        key_cache=bits(k_paged),
        value_cache=bits(v_paged),
        block_tables=block_table.to(torch.int32).numpy(),
        context_lens=context_lens.numpy(),
        out_ref=bits(out_ref.squeeze(1)),
        out_pt=bits(out_pt.squeeze(1)),
        has_sinks=np.array(int(sinks)),
        sm_scale=np.array(1.0 / math.sqrt(d), dtype=np.float64),
        kv_dtype=np.array(fp8_dtype or "float16"),
    )
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    print(f"{name}: ctx={context_lens.tolist()} |out_ref|max={out_ref.abs().max().item():.4f}")


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of baodii/flash_attention_factory>")
    ref_root = Path(sys.argv[1])
    ref16 = load_reference_module(ref_root / "test_paged.py", "ref_test_paged")
    ref8 = load_reference_module(ref_root / "test_paged_fp8cache.py", "ref_test_paged_fp8cache")
    for case in CASES:
        make_case(ref16, ref8, *case)


if __name__ == "__main__":
    main()
