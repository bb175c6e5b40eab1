"""Per-KV-head FP8 scales (an extension over the reference's scalar fp8_scale)."""
import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv,hk,d", [("float8_e4m3fn", 4, 128), ("float8_e5m2", 2, 64), ("float8_e4m3fn", 1, 128)])
def test_per_head_scales_match_the_oracle(cuda_device, variant, kv, hk, d):
    from flash_attention_factory_b200 import lib

    dev = cuda_device
    ctx = [700, 90, 1537]
    h = hk * 4
    c = make_case(seed=95, num_seqs=3, num_heads=h, num_kv_heads=hk, head_size=d, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    g = torch.Generator().manual_seed(2)
    k_scales = (torch.rand(hk, generator=g) * 1.5 + 0.25)
    v_scales = (torch.rand(hk, generator=g) * 3.0 + 0.1)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      k_scales=k_scales, v_scales=v_scales)
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    psize = 512 if d == 128 else 256
    npart = (max(ctx) + psize - 1) // psize
    ml = torch.empty(3, h, npart, dtype=torch.float32, device=dev)
    es = torch.empty_like(ml)
    tmp = torch.empty(3, h, npart, d, dtype=torch.float16, device=dev)
    out = torch.zeros(3, h, d, dtype=torch.float16, device=dev)
    mod = getattr(lib, f"paged_attention_fp8_{variant}")
    mod.enqueue(ml, es, tmp, out, torch.zeros(1, device=dev), q, k, v, bt, cl, 4, c["sm_scale"],
                123.0,  # the scalar must be ignored when both per-head arrays are given
                16, max(ctx), torch.ones(h, device=dev), c["sinks"].to(dev), -1.0,
                k_scale_per_head=k_scales.to(dev), v_scale_per_head=v_scales.to(dev))
    torch.cuda.synchronize(dev)
    # outputs scale with v_scales (up to 3x): relative tolerance carries the check
    assert_close(out.cpu(), want, atol=3e-3, rtol=1e-2, what=f"per-head scales {variant}/{kv}")


def test_per_head_scales_are_refused_for_fp16():
    import ctypes

    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    p = _cabi.PaParams()
    p.head_size, p.block_size, p.num_queries_per_tokens = 128, 16, 1
    p.sm_scale, p.kv_dtype, p.k_scale_per_head = 0.1, _cabi.KV_F16, 0x1000
    assert lib.launch_kernels_loop(ctypes.byref(p), None, None) == _cabi.PA_ERR_BAD_ARG
    assert "per-head" in lib.pa_last_error().decode()
