"""The multi-GPU driver on real devices: logical shards of one batch run together and their
gathered outputs are the unsharded result.  With one GPU the shards share it (separate streams,
separate host threads); with several visible GPUs they are spread over them."""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scheme,parts", [("contiguous", 3), ("lpt", 4), ("heads", 2)])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_shards_run_together_and_gather_to_the_unsharded_result(cuda_device, scheme, parts, kv):
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200.multi_gpu import shard_reference_batch

    ctx = [900, 17, 2100, 1300, 1, 2049, 640, 77, 3000, 333, 512]
    c = make_case(seed=211, num_seqs=len(ctx), num_heads=32, num_kv_heads=8, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    n_dev = torch.cuda.device_count()
    devices = [torch.device("cuda", i % n_dev) for i in range(parts)]
    job = shard_reference_batch(c, devices, scheme, "reduce")
    worst, each = job.run(calls=3, warmup=1)
    assert len(each) == parts and worst == pytest.approx(max(each)) and min(each) > 0.0
    got = job.gather(torch.full((len(ctx), 32, 128), 7.0, dtype=torch.float16, device=cuda_device)).cpu()
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"])
    assert_close(got, want, what=f"{scheme}/{parts} shards")
    # a warp owns a KV head in every shard here (heads in fours), so a (sequence, head) pair is
    # computed the same way however the batch is cut
    whole = run_entry("reduce", c, cuda_device)["out"]
    assert torch.equal(got, whole)
    pkg.device_status()
