"""Opt-in soft-cap and ALiBi (ignored by default, as in the reference)."""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def _call(variant, c, dev, alibi, softcap, use_alibi, use_softcap):
    from flash_attention_factory_b200 import lib

    fp8 = c["kv_dtype"] != "float16"
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    s, h, d = q.shape
    npart = (int(c["context_lens"].max()) + 511) // 512
    ml = torch.empty(s, h, npart, dtype=torch.float32, device=dev)
    es = torch.empty_like(ml)
    tmp = torch.empty(s, h, npart, d, dtype=torch.float16, device=dev)
    out = torch.zeros(s, h, d, dtype=torch.float16, device=dev)
    mod = getattr(lib, f"paged_attention_{'fp8_' if fp8 else ''}{variant}")
    args = [ml, es, tmp, out, torch.zeros(1, device=dev), q, k, v, bt, cl, h // k.size(2), c["sm_scale"]]
    if fp8:
        args.append(c["fp8_scale"])
    sinks = c["sinks"].to(dev) if c["sinks"] is not None else None
    args += [k.size(1), int(c["context_lens"].max()), alibi.to(dev), sinks, softcap]
    mod.enqueue(*args, use_alibi=use_alibi, use_softcap=use_softcap)
    torch.cuda.synchronize(dev)
    return out.cpu()


@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
@pytest.mark.parametrize("use_alibi,use_softcap", [(True, False), (False, True), (True, True)])
def test_modifiers_match_the_oracle(cuda_device, variant, kv, use_alibi, use_softcap):
    ctx = [777, 40, 1300, 513]
    c = make_case(seed=97, num_seqs=4, num_heads=12, num_kv_heads=4, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    c["query"] = (c["query"].float() * 3).half()  # large logits so that the cap bites
    alibi = torch.linspace(0.01, 0.3, 12)
    softcap = 5.0
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      fp8_scale=c["fp8_scale"], softcap=softcap if use_softcap else 0.0,
                                      alibi_slopes=alibi if use_alibi else None)
    got = _call(variant, c, cuda_device, alibi, softcap, use_alibi, use_softcap)
    assert_close(got, want, what=f"modifiers {variant}/{kv}/{use_alibi}/{use_softcap}")


@pytest.mark.parametrize("variant", ["loop", "reduce"])
def test_modifiers_are_ignored_by_default(cuda_device, variant):
    """run() with alibi_slopes = ones and softcap = 30 must equal the plain result: the reference
    never reads either (paged_attention_kernel_loop.hpp:329-342)."""
    c = make_case(seed=98, num_seqs=2, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[600, 70])
    plain = run_entry(variant, c, cuda_device)["out"]
    got = _call(variant, c, cuda_device, torch.ones(8), 30.0, False, False)
    assert torch.equal(got, plain)
