"""paged_attention_auto: loop kernel for short sequences, split-context pair for long ones."""
import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_auto_matches_oracle_and_single_variant_bits(cuda_device, kv):
    from flash_attention_factory_b200.serving import AutoDecodePlan, paged_attention_auto
    from flash_attention_factory_b200.sharding import choose_variant
    from _util import run_entry

    ctx = [30, 5000, 700, 2048, 1, 2047, 3100]
    c = make_case(seed=61, num_seqs=len(ctx), num_heads=16, num_kv_heads=4, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    dev = cuda_device
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    sinks = c["sinks"].to(dev)
    out = torch.full_like(q, float("nan"))
    plan = AutoDecodePlan(ctx, 16, 128, 16, bt.size(1), dev)
    assert plan.loop is not None and plan.reduce is not None
    for _ in range(2):  # the plan is reusable
        paged_attention_auto(plan, out, q, k, v, bt, cl, 4, c["sm_scale"], c["fp8_scale"], sinks)
    torch.cuda.synchronize(dev)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      fp8_scale=c["fp8_scale"])
    assert_close(out.cpu(), want, what=f"auto/{kv}")
    # every sequence carries exactly the bits of the variant chosen for it alone
    by_variant = {vname: run_entry(vname, c, dev)["out"] for vname in ("loop", "reduce")}
    for i, n in enumerate(ctx):
        assert torch.equal(out[i].cpu(), by_variant[choose_variant(n)][i]), f"sequence {i}"
