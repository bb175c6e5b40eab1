"""pa_reshape_and_cache: bit-exact against the CPU statement of the reference's fixture casts."""
import pytest
import torch

from _util import FP8_DTYPES, assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16) if t.dtype == torch.float16 else t.view(torch.uint8)


@pytest.mark.parametrize("kv,scale", [("float16", 1.0), ("float8_e5m2", 1.0), ("float8_e4m3fn", 1.0),
                                      ("float8_e4m3fn", 0.0123), ("float8_e5m2", 3.0),
                                      ("float8_e4m3fn", 0.25), ("float8_e5m2", 8.0)])
@pytest.mark.parametrize("hk,d,bs", [(8, 128, 16), (2, 64, 64), (1, 128, 32)])
def test_append_is_bit_exact(cuda_device, kv, scale, hk, d, bs):
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    g = torch.Generator().manual_seed(hk * 1000 + d + bs)
    nb, t = 12, 37
    dt = torch.float16 if kv == "float16" else FP8_DTYPES[kv]
    # values stay inside the format's range after scaling: |x / scale| < 448 for e4m3
    key = (torch.randn(t, hk, d, generator=g) * (scale if scale != 1.0 else 1.0) * 20).to(torch.float16)
    value = (torch.randn(t, hk, d, generator=g) * (scale if scale != 1.0 else 1.0) * 20).to(torch.float16)
    kc = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16).to(dt)
    vc = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16).to(dt)
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int64)
    slots[5] = -1  # padding token: skipped
    want_k, want_v = oracle.reshape_and_cache_ref(key, value, kc, vc, slots, scale)
    dk, dv = kc.to(cuda_device), vc.to(cuda_device)
    reshape_and_cache(key.to(cuda_device), value.to(cuda_device), dk, dv, slots.to(cuda_device), scale)
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(_bits(dk.cpu()), _bits(want_k))
    assert torch.equal(_bits(dv.cpu()), _bits(want_v))


def test_fp8_overflow_saturates(cuda_device):
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    key = torch.full((1, 1, 8), 1000.0, dtype=torch.float16)
    key[0, 0, 1] = -60000.0
    kc = torch.zeros(1, 16, 1, 8, dtype=torch.float8_e4m3fn, device=cuda_device)
    vc = torch.zeros_like(kc)
    reshape_and_cache(key.to(cuda_device), key.to(cuda_device), kc, vc,
                      torch.zeros(1, dtype=torch.int64, device=cuda_device), 1.0)
    got = kc[0, 0, 0].float().cpu()
    assert got[0] == 448.0 and got[1] == -448.0  # largest finite e4m3 code, not NaN


@pytest.mark.parametrize("kv", ["float8_e5m2", "float8_e4m3fn"])
def test_decode_step_append_then_attend(cuda_device, kv):
    """One decode step end to end: the kernel appends token ctx of every sequence, attention
    over ctx + 1 tokens then equals the oracle on a cache built with torch casts."""
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    ctx = [100, 511, 512, 37]
    c = make_case(seed=77, num_seqs=4, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[n + 1 for n in ctx], kv_dtype=kv, fp8_scale=0.05)
    g = torch.Generator().manual_seed(3)
    new_k = (torch.randn(4, 2, 128, generator=g)).to(torch.float16)
    new_v = (torch.randn(4, 2, 128, generator=g)).to(torch.float16)
    slots = torch.tensor([int(c["block_tables"][i, n // 16]) * 16 + n % 16 for i, n in enumerate(ctx)])
    want_k, want_v = oracle.reshape_and_cache_ref(new_k, new_v, c["key_cache"], c["value_cache"], slots,
                                                  c["fp8_scale"])
    dk, dv = c["key_cache"].to(cuda_device), c["value_cache"].to(cuda_device)
    reshape_and_cache(new_k.to(cuda_device), new_v.to(cuda_device), dk, dv, slots.to(cuda_device),
                      c["fp8_scale"])
    c2 = dict(c)
    c2["key_cache"], c2["value_cache"] = dk.cpu(), dv.cpu()
    want = oracle.paged_attention_ref(c["query"], want_k, want_v, c["block_tables"], c["context_lens"],
                                      sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    for variant in ("loop", "reduce"):
        assert_close(run_entry(variant, c2, cuda_device)["out"], want, what=f"append+attend/{kv}/{variant}")


@pytest.mark.parametrize("kv,scale", [("float16", 1.0), ("float8_e4m3fn", 0.5), ("float8_e5m2", 0.3)])
def test_prefill_sized_append_is_bit_exact(cuda_device, kv, scale):
    """More than 4096 tokens take the plain (not launch-chained) form of the kernel."""
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    g = torch.Generator().manual_seed(77)
    hk, d, bs, nb, t = 4, 128, 16, 400, 5000
    dt = torch.float16 if kv == "float16" else FP8_DTYPES[kv]
    key = (torch.randn(t, hk, d, generator=g) * scale * 20).to(torch.float16)
    value = (torch.randn(t, hk, d, generator=g) * scale * 20).to(torch.float16)
    kc = torch.zeros(nb, bs, hk, d, dtype=torch.float16).to(dt)
    vc = torch.zeros(nb, bs, hk, d, dtype=torch.float16).to(dt)
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int64)
    want_k, want_v = oracle.reshape_and_cache_ref(key, value, kc, vc, slots, scale)
    dk, dv = kc.to(cuda_device), vc.to(cuda_device)
    reshape_and_cache(key.to(cuda_device), value.to(cuda_device), dk, dv, slots.to(cuda_device), scale)
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(_bits(dk.cpu()), _bits(want_k))
    assert torch.equal(_bits(dv.cpu()), _bits(want_v))


@pytest.mark.parametrize("kv", ["float8_e5m2", "float8_e4m3fn"])
@pytest.mark.parametrize("kind", ["per_head", "per_block"])
@pytest.mark.parametrize("hk,d,bs,t", [(8, 128, 16, 37), (2, 64, 64, 21), (4, 128, 16, 5000)])
def test_append_with_scale_arrays_is_bit_exact(cuda_device, kv, kind, hk, d, bs, t):
    """Per-head and per-block scale arrays take the place of the scalar: stored = x / scale of
    the token's KV head (and block), in the arithmetic of the oracle's torch division."""
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    g = torch.Generator().manual_seed(hk * 31 + d + bs + t)
    nb = (t + bs - 1) // bs + 11
    dt = FP8_DTYPES[kv]
    shape = (hk,) if kind == "per_head" else (nb, hk)
    # |x / scale| stays inside e4m3's range (448): torch's cast turns overflow into NaN, the kernel saturates
    k_scales = torch.rand(shape, generator=g) * 1.5 + 0.05
    v_scales = torch.rand(shape, generator=g) * 3.0 + 0.1
    key = (torch.randn(t, hk, d, generator=g) * 2).to(torch.float16)
    value = (torch.randn(t, hk, d, generator=g) * 2).to(torch.float16)
    kc = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16).to(dt)
    vc = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16).to(dt)
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int64)
    slots[3] = -1
    want_k, want_v = oracle.reshape_and_cache_ref(key, value, kc, vc, slots, 123.0, k_scales, v_scales)
    dk, dv = kc.to(cuda_device), vc.to(cuda_device)
    names = {f"k_scale_{kind}": k_scales.to(cuda_device), f"v_scale_{kind}": v_scales.to(cuda_device)}
    # the scalar must be ignored when arrays are given
    reshape_and_cache(key.to(cuda_device), value.to(cuda_device), dk, dv, slots.to(cuda_device), 123.0, **names)
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(_bits(dk.cpu()), _bits(want_k))
    assert torch.equal(_bits(dv.cpu()), _bits(want_v))


@pytest.mark.parametrize("kv", ["float8_e5m2", "float8_e4m3fn"])
def test_decode_step_with_per_block_scales_append_then_attend(cuda_device, kv):
    """Writer and reader agree on per-block scales: the kernel appends one token per sequence with
    the scale of its block, attention with the same arrays equals the oracle on the oracle's cache."""
    from flash_attention_factory_b200 import lib
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    ctx = [100, 511, 512, 37]
    hk, h, d, bs = 2, 8, 128, 16
    c = make_case(seed=78, num_seqs=4, num_heads=h, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=[n + 1 for n in ctx], kv_dtype=kv)
    g = torch.Generator().manual_seed(5)
    nb = c["key_cache"].size(0)
    k_scales = torch.rand(nb, hk, generator=g) * 1.5 + 0.25
    v_scales = torch.rand(nb, hk, generator=g) * 3.0 + 0.1
    new_k = torch.randn(4, hk, d, generator=g).to(torch.float16)
    new_v = torch.randn(4, hk, d, generator=g).to(torch.float16)
    slots = torch.tensor([int(c["block_tables"][i, n // bs]) * bs + n % bs for i, n in enumerate(ctx)])
    want_k, want_v = oracle.reshape_and_cache_ref(new_k, new_v, c["key_cache"], c["value_cache"], slots, 1.0,
                                                  k_scales, v_scales)
    dev = cuda_device
    dk, dv = c["key_cache"].to(dev), c["value_cache"].to(dev)
    ks, vs = k_scales.to(dev), v_scales.to(dev)
    reshape_and_cache(new_k.to(dev), new_v.to(dev), dk, dv, slots.to(dev), 1.0,
                      k_scale_per_block=ks, v_scale_per_block=vs)
    assert torch.equal(_bits(dk.cpu()), _bits(want_k)) and torch.equal(_bits(dv.cpu()), _bits(want_v))
    want = oracle.paged_attention_ref(c["query"], want_k, want_v, c["block_tables"], c["context_lens"],
                                      sm_scale=c["sm_scale"], k_block_scales=k_scales, v_block_scales=v_scales)
    npart = (max(ctx) + 1 + 511) // 512
    for variant in ("loop", "reduce"):
        ml = torch.empty(4, h, npart, dtype=torch.float32, device=dev)
        es, tmp = torch.empty_like(ml), torch.empty(4, h, npart, d, dtype=torch.float16, device=dev)
        out = torch.zeros(4, h, d, dtype=torch.float16, device=dev)
        getattr(lib, f"paged_attention_fp8_{variant}").enqueue(
            ml, es, tmp, out, torch.zeros(1, device=dev), c["query"].to(dev), dk, dv, c["block_tables"].to(dev),
            c["context_lens"].to(dev), h // hk, c["sm_scale"], 1.0, bs, max(ctx) + 1, torch.ones(h, device=dev),
            None, -1.0, k_scale_per_block=ks, v_scale_per_block=vs)
        torch.cuda.synchronize(dev)
        assert_close(out.cpu(), want, atol=3e-3, rtol=1e-2, what=f"append+attend per-block scales/{kv}/{variant}")
