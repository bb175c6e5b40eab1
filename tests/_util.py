"""Helpers shared by the tests: golden-vector loading, seeded fixtures, comparisons."""
from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

# tolerance BASELINE.json's north_star states for every entry point
ATOL, RTOL = 1e-3, 1e-2

FP8_DTYPES = {"float8_e5m2": torch.float8_e5m2, "float8_e4m3fn": torch.float8_e4m3fn}


def golden_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.npz"))


def load_golden(name: str) -> dict:
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    kv_dtype = str(z["kv_dtype"])

    def f16(a):
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.float16)

    if kv_dtype == "float16":
        k, v = f16(z["key_cache"]), f16(z["value_cache"])
    else:
        k = torch.from_numpy(z["key_cache"].copy()).view(FP8_DTYPES[kv_dtype])
        v = torch.from_numpy(z["value_cache"].copy()).view(FP8_DTYPES[kv_dtype])
    q = f16(z["query"])
    sinks = torch.ones(q.shape[1], dtype=torch.float16) * 10 if int(z["has_sinks"]) else None
    return dict(
        query=q, key_cache=k, value_cache=v,
        block_tables=torch.from_numpy(z["block_tables"].copy()),
        context_lens=torch.from_numpy(z["context_lens"].copy()),
        out_ref=f16(z["out_ref"]), out_pt=f16(z["out_pt"]), sinks=sinks,
        sm_scale=float(z["sm_scale"]), kv_dtype=kv_dtype,
    )


def make_case(seed, num_seqs, num_heads, num_kv_heads, head_size, block_size, context_lens,
              kv_dtype="float16", sinks=False, fp8_scale=1.0, extra_blocks=0, integer_valued=False):
    """Seeded synthetic inputs in the reference's layouts (CPU tensors).

    Follows the reference fixture generator (test_paged.py:170-194): N(0,1) fp16 pages,
    block table = random permutation of the physical blocks cut into rows.  For FP8 the
    fp16 pages are cast with torch's round-to-nearest-even cast
    (test_paged_fp8cache.py:201-203); with ``fp8_scale == 'amax'`` the pages are divided
    by amax/448 first and that scale is returned.
    """
    g = torch.Generator().manual_seed(seed)
    ctx = torch.as_tensor(context_lens, dtype=torch.int32)
    assert ctx.numel() == num_seqs
    max_blocks = max(1, (int(ctx.max()) + block_size - 1) // block_size)
    num_blocks = max_blocks * num_seqs + extra_blocks
    shape = (num_blocks, block_size, num_kv_heads, head_size)
    if integer_valued:
        q = torch.randint(-2, 3, (num_seqs, num_heads, head_size), generator=g).to(torch.float16)
        k = torch.randint(-2, 3, shape, generator=g).to(torch.float16)
        v = torch.randint(-4, 5, shape, generator=g).to(torch.float16)
    else:
        q = torch.randn(num_seqs, num_heads, head_size, generator=g).to(torch.float16)
        k = torch.randn(shape, generator=g).to(torch.float16)
        v = torch.randn(shape, generator=g).to(torch.float16)
    scale = 1.0
    if kv_dtype != "float16":
        dt = FP8_DTYPES[kv_dtype]
        if fp8_scale == "amax":
            scale = float(max(k.abs().max(), v.abs().max())) / 448.0
        else:
            scale = float(fp8_scale)
        if scale != 1.0:
            k = (k.float() / scale).to(dt)
            v = (v.float() / scale).to(dt)
        else:
            k, v = k.to(dt), v.to(dt)
    perm = torch.randperm(num_blocks, generator=g)[: max_blocks * num_seqs]
    block_tables = perm.to(torch.int32).view(num_seqs, max_blocks)
    sink_t = None
    if sinks:
        sink_t = (torch.randn(num_heads, generator=g) * 2 + 3).to(torch.float16)
    return dict(query=q, key_cache=k, value_cache=v, block_tables=block_tables, context_lens=ctx,
                sinks=sink_t, sm_scale=1.0 / math.sqrt(head_size), fp8_scale=scale, kv_dtype=kv_dtype,
                block_size=block_size)


def run_entry(variant: str, case: dict, device, max_num_partitions=None, poison=None):
    """Runs one of the four operators through flash_attention_factory_b200.lib on `device`.

    Returns dict(out, max_logits, exp_sums, tmp_out, times).  Scratch buffers are filled
    with `poison` first so that untouched entries can be recognised.
    """
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import lib

    fp8 = case["kv_dtype"] != "float16"
    q = case["query"].to(device)
    k = case["key_cache"].to(device)
    v = case["value_cache"].to(device)
    bt = case["block_tables"].to(device)
    cl = case["context_lens"].to(device)
    sinks = case["sinks"].to(device) if case.get("sinks") is not None else None
    s, h, d = q.shape
    block_size = k.shape[1]
    psize = pkg.partition_size(d)
    max_ctx = int(case["context_lens"].max()) if case["context_lens"].numel() else 0
    npart = max_num_partitions or max(1, (max_ctx + psize - 1) // psize)
    fill = float("nan") if poison is None else poison
    max_logits = torch.full((s, h, npart), fill, dtype=torch.float32, device=device)
    exp_sums = torch.full((s, h, npart), fill, dtype=torch.float32, device=device)
    tmp_out = torch.full((s, h, npart, d), fill, dtype=torch.float16, device=device)
    out = torch.full((s, h, d), fill, dtype=torch.float16, device=device)
    debug = torch.zeros((s, h, npart * d), dtype=torch.float32, device=device)
    alibi = torch.ones(h, dtype=torch.float32, device=device)
    group = h // k.shape[2]
    name = f"paged_attention_{'fp8_' if fp8 else ''}{variant}"
    mod = getattr(lib, name)
    args = [max_logits, exp_sums, tmp_out, out, debug, q, k, v, bt, cl, group, case["sm_scale"]]
    if fp8:
        args.append(case.get("fp8_scale", 1.0))
    args += [block_size, max_ctx, alibi, sinks, -1.0]
    times = mod.run(*args)
    torch.cuda.synchronize(device)
    return dict(out=out.cpu(), max_logits=max_logits.cpu(), exp_sums=exp_sums.cpu(),
                tmp_out=tmp_out.cpu(), times=times)


def assert_close(actual, expected, atol=ATOL, rtol=RTOL, what=""):
    a, e = actual.float(), expected.float()
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values in the result"
    err = (a - e).abs()
    tol = atol + rtol * e.abs()
    bad = err > tol
    assert not bad.any(), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements outside atol={atol} rtol={rtol}; "
        f"max abs err {err.max().item():.3e} at {np.unravel_index(int(err.argmax()), a.shape)}")
