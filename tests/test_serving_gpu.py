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
    plan = AutoDecodePlan(ctx, 16, 128, 16, bt.size(1), dev, fold_short_fraction=0.0)  # strictly per sequence
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
    # default plan: the three short sequences hold 5 % of the tokens and are folded into the split launch
    folded = AutoDecodePlan(ctx, 16, 128, 16, bt.size(1), dev)
    assert folded.loop is None and folded.reduce.count == len(ctx)
    out2 = torch.full_like(q, float("nan"))
    paged_attention_auto(folded, out2, q, k, v, bt, cl, 4, c["sm_scale"], c["fp8_scale"], sinks)
    torch.cuda.synchronize(dev)
    assert torch.equal(out2.cpu(), by_variant["reduce"])
    # a batch of short sequences only is one loop launch
    short = AutoDecodePlan([30, 500, 1, 400], 16, 128, 16, bt.size(1), dev)
    assert short.reduce is None and short.loop.count == 4


def test_decode_step_io_round_trip(cuda_device):
    """Packed upload -> operator -> download gives the oracle's answer from host buffers."""
    from flash_attention_factory_b200 import lib
    from flash_attention_factory_b200.host_io import DecodeStepIO

    ctx = [300, 45, 1025]
    c = make_case(seed=62, num_seqs=3, num_heads=8, num_kv_heads=2, head_size=64, block_size=32,
                  context_lens=ctx)
    dev = cuda_device
    io = DecodeStepIO(3, 8, 64, c["block_tables"].size(1), dev)
    io.query_host.copy_(c["query"])
    io.block_tables_host.copy_(c["block_tables"])
    io.context_lens_host.copy_(c["context_lens"])
    k, v = c["key_cache"].to(dev), c["value_cache"].to(dev)
    ml = torch.empty(3, 8, 5, dtype=torch.float32, device=dev)
    tmp = torch.empty(3, 8, 5, 64, dtype=torch.float16, device=dev)
    io.upload()
    lib.paged_attention_reduce.enqueue(ml, torch.empty_like(ml), tmp, io.out, torch.zeros(1, device=dev),
                                       io.query, k, v, io.block_tables, io.context_lens, 4, c["sm_scale"],
                                       32, max(ctx), torch.ones(8, device=dev), None, -1.0)
    got = io.download().clone()
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"])
    assert_close(got, want, what="DecodeStepIO")
