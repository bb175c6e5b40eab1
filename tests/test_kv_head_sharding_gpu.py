"""Sharding by KV head (few very long sequences): each shard holds a slice of the KV heads of
both caches and the matching query heads, and writes a disjoint slice of the output."""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["reduce", "loop"])
@pytest.mark.parametrize("kv,world", [("float8_e4m3fn", 2), ("float16", 4)])
def test_head_shards_concatenate_to_the_unsharded_result(cuda_device, variant, kv, world):
    from flash_attention_factory_b200.sharding import shard_kv_heads

    hk, group, d = 8, 4, 128
    ctx = [5000, 1200]
    c = make_case(seed=71, num_seqs=len(ctx), num_heads=hk * group, num_kv_heads=hk, head_size=d, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True, fp8_scale=0.5 if kv != "float16" else 1.0)
    whole = run_entry(variant, c, cuda_device)["out"]
    pieces = []
    for lo, hi in shard_kv_heads(hk, world):
        shard = dict(c)
        shard["key_cache"] = c["key_cache"][:, :, lo:hi, :].contiguous()  # what the rank keeps in its HBM
        shard["value_cache"] = c["value_cache"][:, :, lo:hi, :].contiguous()
        shard["query"] = c["query"][:, lo * group:hi * group, :].contiguous()
        shard["sinks"] = c["sinks"][lo * group:hi * group].contiguous()
        pieces.append(run_entry(variant, shard, cuda_device)["out"])
    glued = torch.cat(pieces, dim=1)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      fp8_scale=c["fp8_scale"])
    assert_close(glued, want, what=f"head shards {variant}/{kv}/{world}")
    if variant == "reduce" and (hk // world) % 4 == 0:
        # with heads in fours a warp owns a head: a (sequence, head) pair is computed the same
        # way whatever else the launch holds
        assert torch.equal(glued, whole)
    else:
        assert_close(glued, whole, what="head shards vs unsharded")
