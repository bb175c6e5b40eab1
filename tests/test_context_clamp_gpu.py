"""A context length larger than the block-table row can address is cut to what the row holds.

The reference checks head size, block size and group on the host
(paged_attention_loop/launch_kernels_loop.h:114-115,170-172) and trusts context_lens.  Here
a value beyond max_blocks_per_seq * block_size would walk the producer past the sequence's
row of block_tables; the kernels cut it to that limit instead, and the result is attention
over the clamped prefix.  The oversized entry sits in a row that is not the last one of
block_tables, so even an unclamped read would stay inside the tensor.
"""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
@pytest.mark.parametrize("block_size,limit_blocks", [(16, 70), (64, 9)])
def test_context_length_beyond_the_table_row_is_clamped(cuda_device, variant, kv, block_size, limit_blocks):
    limit = block_size * limit_blocks  # 1120 / 576 tokens: crosses a partition boundary
    honest = [limit - 3, limit, 200, limit - block_size]
    c = make_case(seed=77, num_seqs=4, num_heads=8, num_kv_heads=2, head_size=128, block_size=block_size,
                  context_lens=honest, kv_dtype=kv, sinks=True)
    assert c["block_tables"].shape[1] == limit_blocks
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"])
    lying = dict(c)
    lying["context_lens"] = torch.tensor([limit - 3, limit + 5000, 200, limit - block_size], dtype=torch.int32)
    # scratch sized for what the caller claims; rows past the clamped context must stay untouched
    res = run_entry(variant, lying, cuda_device, poison=-9.0)
    assert_close(res["out"], want, what=f"clamped/{variant}/{kv}")
    honest_res = run_entry(variant, c, cuda_device, poison=-9.0)
    assert torch.equal(res["out"], honest_res["out"]), "clamping must give the bits of the honest length"
    if variant == "reduce":
        psize = 512
        used = (limit + psize - 1) // psize
        assert (res["max_logits"][1, :, used:] == -9.0).all() and (res["tmp_out"][1, :, used:] == -9.0).all()
