"""Per-block FP8 scales (an extension over the reference's scalar fp8_scale): every (block, KV
head) of the cache has its own K and V dequantisation scale, fetched with the block."""
import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def _run(mod, dev, c, ctx, h, d, bs, group, **scales):
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    s = len(ctx)
    psize = 512 if d == 128 else 256
    npart = (max(ctx) + psize - 1) // psize
    ml = torch.empty(s, h, npart, dtype=torch.float32, device=dev)
    es = torch.empty_like(ml)
    tmp = torch.empty(s, h, npart, d, dtype=torch.float16, device=dev)
    out = torch.zeros(s, h, d, dtype=torch.float16, device=dev)
    sinks = c["sinks"].to(dev) if c["sinks"] is not None else None
    mod.enqueue(ml, es, tmp, out, torch.zeros(1, device=dev), q, k, v, bt, cl, group, c["sm_scale"],
                123.0,  # the scalar must be ignored when per-block scales are given
                bs, max(ctx), torch.ones(h, device=dev), sinks, -1.0,
                **{name: t.to(dev) for name, t in scales.items()})
    torch.cuda.synchronize(dev)
    return out.cpu()


# (kv, kv heads, head size, block size, group): 1 / 2 / 4 KV heads per CTA and stages of 1, 2 and 4
# tiles; the 8-warp CTA is covered by tests/test_wide_cta_gpu.py (case "e4m3_d128_b16_block_scales")
@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv,hk,d,bs,group", [("float8_e4m3fn", 4, 128, 16, 4), ("float8_e5m2", 2, 64, 16, 2),
                                              ("float8_e4m3fn", 1, 128, 16, 8), ("float8_e5m2", 4, 128, 64, 2),
                                              ("float8_e4m3fn", 4, 64, 64, 5), ("float8_e5m2", 8, 128, 32, 1)])
def test_per_block_scales_match_the_oracle(cuda_device, variant, kv, hk, d, bs, group):
    from flash_attention_factory_b200 import lib

    ctx = [700, 90, 1537, 1, 513]
    h = hk * group
    c = make_case(seed=195, num_seqs=len(ctx), num_heads=h, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    g = torch.Generator().manual_seed(4)
    nb = c["key_cache"].size(0)
    k_scales = torch.rand(nb, hk, generator=g) * 1.5 + 0.25
    v_scales = torch.rand(nb, hk, generator=g) * 3.0 + 0.1
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      k_block_scales=k_scales, v_block_scales=v_scales)
    mod = getattr(lib, f"paged_attention_fp8_{variant}")
    got = _run(mod, cuda_device, c, ctx, h, d, bs, group, k_scale_per_block=k_scales, v_scale_per_block=v_scales)
    # outputs scale with the V scales (up to 3x): the relative tolerance carries the check
    assert_close(got, want, atol=3e-3, rtol=1e-2, what=f"per-block scales {variant}/{kv}/bs{bs}")
    # all-equal block scales are the scalar scale: same answer as fp8_scale within rounding of the order of operations
    flat = _run(mod, cuda_device, c, ctx, h, d, bs, group, k_scale_per_block=torch.full((nb, hk), 0.5),
                v_scale_per_block=torch.full((nb, hk), 0.5))
    want_flat = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                           c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"], fp8_scale=0.5)
    assert_close(flat, want_flat, what="constant per-block scales")


def test_per_block_scales_argument_checks():
    import ctypes

    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    p = _cabi.PaParams()
    p.head_size, p.block_size, p.num_queries_per_tokens = 128, 16, 1
    p.sm_scale, p.fp8_scale, p.kv_dtype, p.k_scale_per_block = 0.1, 1.0, _cabi.KV_F16, 0x1000
    assert lib.launch_kernels_loop(ctypes.byref(p), None, None) == _cabi.PA_ERR_BAD_ARG  # fp16 entry point
    p.kv_dtype = _cabi.KV_FP8_E5M2
    assert lib.launch_kernels_fp8_loop(ctypes.byref(p), None, None) == _cabi.PA_ERR_BAD_ARG  # V scales missing
    assert "together" in lib.pa_last_error().decode()
    p.v_scale_per_block, p.k_scale_per_head = 0x2000, 0x3000
    assert lib.launch_kernels_fp8_loop(ctypes.byref(p), None, None) == _cabi.PA_ERR_BAD_ARG  # both kinds
    assert "exclude" in lib.pa_last_error().decode()
