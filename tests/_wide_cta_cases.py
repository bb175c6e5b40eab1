"""Cases of tests/test_wide_cta_gpu.py, runnable as a script.

`python tests/_wide_cta_cases.py out.pt` runs every case through the FP8 split entry point on
cuda:0 and stores the outputs.  The CTA shape is whatever the process environment selects
(PA_WIDE_CTA=1 forces the 8-warp shape wherever the KV heads come in eights), which is why
the test runs this file in a child process.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from _util import make_case  # noqa: E402

# name -> (kv, head_size, block_size, num_heads, num_kv_heads, context_lens, sinks, extras)
CASES = {
    "e4m3_d128_b16_g1_ragged": ("float8_e4m3fn", 128, 16, 8, 8, [1500, 17, 512, 513, 1, 2049], False, ()),
    "e5m2_d128_b16_g4_sinks": ("float8_e5m2", 128, 16, 32, 8, [700, 3000, 31], True, ()),
    "e4m3_d64_b16_g8": ("float8_e4m3fn", 64, 16, 64, 8, [1000, 255, 257, 40], False, ()),
    "e5m2_d64_b64_g2_sinks": ("float8_e5m2", 64, 64, 32, 16, [900, 64, 65], True, ()),
    "e4m3_d128_b128_g2": ("float8_e4m3fn", 128, 128, 32, 16, [1300, 129, 5], False, ()),
    "e5m2_d128_b32_scales": ("float8_e5m2", 128, 32, 16, 8, [800, 1600, 90], True, ("scales",)),
    "e4m3_d128_b16_modifiers": ("float8_e4m3fn", 128, 16, 16, 8, [777, 40, 1300], True, ("alibi", "softcap")),
    "e5m2_d128_b16_subset": ("float8_e5m2", 128, 16, 16, 8, [600, 50, 1100, 2000, 513], False, ("subset",)),
    "e4m3_d128_b16_block_scales": ("float8_e4m3fn", 128, 16, 16, 8, [900, 33, 1600], True, ("block_scales",)),
}
SUBSET = [3, 0, 4]  # sequence ids of the "subset" case, in launch order


def build(name):
    kv, d, bs, h, hk, ctx, sinks, extras = CASES[name]
    c = make_case(seed=300 + list(CASES).index(name), num_seqs=len(ctx), num_heads=h, num_kv_heads=hk, head_size=d,
                  block_size=bs, context_lens=ctx, kv_dtype=kv, sinks=sinks, fp8_scale=0.5)
    g = torch.Generator().manual_seed(9)
    c["k_scales"] = torch.rand(hk, generator=g) + 0.5 if "scales" in extras else None
    c["v_scales"] = torch.rand(hk, generator=g) * 2 + 0.25 if "scales" in extras else None
    c["alibi"] = torch.linspace(0.01, 0.2, h) if "alibi" in extras else None
    c["softcap"] = 6.0 if "softcap" in extras else 0.0
    c["subset"] = SUBSET if "subset" in extras else None
    nb = c["key_cache"].size(0)
    c["k_block_scales"] = torch.rand(nb, hk, generator=g) + 0.5 if "block_scales" in extras else None
    c["v_block_scales"] = torch.rand(nb, hk, generator=g) * 2 + 0.25 if "block_scales" in extras else None
    return c


def run_case(name, dev):
    """Output [S, H, D] (fp16, CPU) of the FP8 split variant for one case."""
    from flash_attention_factory_b200 import _cabi
    from flash_attention_factory_b200.lib import _shim
    from flash_attention_factory_b200.lib import paged_attention_fp8_reduce as mod

    c = build(name)
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    s, h, d = q.shape
    psize = _cabi.partition_size(d)
    npart = (int(c["context_lens"].max()) + psize - 1) // psize
    ml = torch.full((s, h, npart), -7.0, dtype=torch.float32, device=dev)
    es = torch.full_like(ml, -7.0)
    tmp = torch.full((s, h, npart, d), -7.0, dtype=torch.float16, device=dev)
    out = torch.full((s, h, d), -7.0, dtype=torch.float16, device=dev)
    alibi = (c["alibi"] if c["alibi"] is not None else torch.ones(h)).to(dev)
    sinks = c["sinks"].to(dev) if c["sinks"] is not None else None
    ks = c["k_scales"].to(dev) if c["k_scales"] is not None else None
    vs = c["v_scales"].to(dev) if c["v_scales"] is not None else None
    kb = c["k_block_scales"].to(dev) if c["k_block_scales"] is not None else None
    vb = c["v_block_scales"].to(dev) if c["v_block_scales"] is not None else None
    p = mod.params(ml, es, tmp, out, torch.zeros(1, device=dev), q, k, v, bt, cl, h // k.size(2), c["sm_scale"],
                   c["fp8_scale"], k.size(1), int(c["context_lens"].max()), alibi, sinks, c["softcap"] or -1.0,
                   k_scale_per_head=ks, v_scale_per_head=vs, use_alibi=c["alibi"] is not None,
                   use_softcap=c["softcap"] > 0, k_scale_per_block=kb, v_scale_per_block=vb)
    keep = None
    if c["subset"] is not None:
        keep = torch.tensor(c["subset"], dtype=torch.int32, device=dev)
        p.num_seqs = keep.numel()
        p.seq_indices = keep.data_ptr()
    _shim.enqueue_entry(mod.ENTRY, p, dev)
    torch.cuda.synchronize(dev)
    return out.cpu()


if __name__ == "__main__":
    device = torch.device("cuda:0")
    results = {name: run_case(name, device) for name in CASES}
    import flash_attention_factory_b200 as pkg

    pkg.device_status()
    torch.save(results, sys.argv[1])
