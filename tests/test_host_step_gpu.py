"""One decode step with host buffers as a single library call (pa_decode_step_host)."""
import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("direct_out", [False, True])
@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_host_step_matches_oracle_and_enqueue(cuda_device, variant, kv, direct_out):
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import lib
    from flash_attention_factory_b200.host_io import DecodeStepIO

    dev = cuda_device
    ctx = [900, 17, 512, 1300, 1]
    s, h, hk, d, bs = len(ctx), 8, 4, 128, 16
    c = make_case(seed=91, num_seqs=s, num_heads=h, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=ctx, kv_dtype=kv)
    fp8 = kv != "float16"
    k, v = c["key_cache"].to(dev), c["value_cache"].to(dev)
    npart = 3
    ml = torch.empty(s, h, npart, dtype=torch.float32, device=dev)
    es = torch.empty_like(ml)
    tmp = torch.empty(s, h, npart, d, dtype=torch.float16, device=dev)
    dbg = torch.zeros(1, dtype=torch.float32, device=dev)
    alibi = torch.ones(h, dtype=torch.float32, device=dev)
    mod = getattr(lib, f"paged_attention_{'fp8_' if fp8 else ''}{variant}")

    io = DecodeStepIO(s, h, d, c["block_tables"].size(1), dev)

    def args(out, q, bt, cl):
        a = [ml, es, tmp, out, dbg, q, k, v, bt, cl, h // hk, c["sm_scale"]]
        if fp8:
            a.append(c["fp8_scale"])
        return a + [bs, max(ctx), alibi, None, -1.0]

    # reference run of the same operator on device-resident inputs
    want_dev = torch.zeros(s, h, d, dtype=torch.float16, device=dev)
    mod.enqueue(*args(want_dev, c["query"].to(dev), c["block_tables"].to(dev), c["context_lens"].to(dev)))
    torch.cuda.synchronize(dev)

    step = io.bind(mod.ENTRY, mod.params(*args(io.out, io.query, io.block_tables, io.context_lens)),
                   direct_out=direct_out)
    io.query_host.copy_(c["query"])
    io.block_tables_host.copy_(c["block_tables"])
    io.context_lens_host.copy_(c["context_lens"])
    io.out_host.fill_(7.0)
    got = step.run()  # returns after the stream has drained: the host buffer holds the result
    assert torch.equal(got, want_dev.cpu()), "host step and enqueue disagree"
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    assert_close(got, want, what=f"host step {variant}/{kv}/direct={direct_out}")

    # a second step with other inputs in the same staging buffer
    io.query_host.mul_(-0.5)
    got2 = step.run().clone()
    want2 = oracle.paged_attention_ref(io.query_host.clone(), c["key_cache"], c["value_cache"], c["block_tables"],
                                       c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    assert_close(got2, want2, what="second host step")
    pkg.device_status()


def test_host_step_rejects_bad_arguments(cuda_device):
    import ctypes

    from flash_attention_factory_b200 import _cabi

    lib = _cabi.load_library()
    p, io = _cabi.PaParams(), _cabi.PaHostStep()
    with torch.cuda.device(cuda_device):
        assert lib.pa_decode_step_host(9, ctypes.byref(p), ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
        io.in_bytes = 16  # size without buffers
        assert lib.pa_decode_step_host(0, ctypes.byref(p), ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
        assert lib.pa_decode_step_host(0, None, ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
