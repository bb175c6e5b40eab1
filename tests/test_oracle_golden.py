"""Pins the CPU oracle against golden vectors produced by the reference's own
`attention_ref` / `attention_ref_fp8kv` (tests/golden/make_golden.py)."""
import pytest
import torch

from _util import golden_cases, load_golden
from oracle import paged_attention_oracle as oracle


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_matches_reference_fp32_path(name):
    c = load_golden(name)
    out = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                     c["context_lens"], sm_scale=None, sinks=c["sinks"])
    ref = c["out_ref"]
    # same fp32 math as the reference; only the summation order inside einsum may differ,
    # which can flip the final fp16 rounding by one unit in the last place
    err = (out.float() - ref.float()).abs()
    assert (err <= 2.0 ** -10 * ref.float().abs() + 1e-7).all(), err.max().item()
    assert (err == 0).float().mean().item() > 0.98
    diff = err.max().item()
    # and it satisfies the reference's own acceptance criterion (test_paged.py:603-604)
    bound = 3 * (c["out_pt"].float() - ref.float()).abs().max().item() + 1e-5
    assert diff <= bound


@pytest.mark.parametrize("name", golden_cases())
def test_partition_restatement_merges_to_the_same_answer(name):
    """merge(partition stats) must equal the one-shot softmax for 512- and 256-token partitions."""
    c = load_golden(name)
    d = c["query"].shape[-1]
    psize = 512 if d == 128 else 256
    ml, es, tmp, written = oracle.partition_stats_ref(
        c["query"], c["key_cache"], c["value_cache"], c["block_tables"], c["context_lens"], psize,
        sm_scale=None, sinks=c["sinks"])
    merged = oracle.merge_partitions_ref(ml, es, tmp, c["context_lens"], psize)
    assert (merged.float() - c["out_ref"].float()).abs().max().item() <= 1e-3 * 0.5
    for i, ctx in enumerate(c["context_lens"].tolist()):
        n = (ctx + psize - 1) // psize
        assert written[i, :n].all() and not written[i, n:].any()


def test_empty_context_gives_zeros():
    q = torch.randn(1, 4, 64).half()
    k = torch.randn(2, 16, 2, 64).half()
    out = oracle.paged_attention_ref(q, k, k, torch.zeros(1, 1, dtype=torch.int32), [0])
    assert torch.count_nonzero(out) == 0


def test_fp8_scale_is_applied_once():
    """K_deq = fp16(k8) * s and V_deq = fp16(v8) * s, each exactly once."""
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, 2, 64, generator=g).half()
    k16 = torch.randn(4, 16, 1, 64, generator=g).half()
    k8 = k16.to(torch.float8_e4m3fn)
    bt = torch.arange(4, dtype=torch.int32).view(1, 4)
    a = oracle.paged_attention_ref(q, k8, k8, bt, [50], fp8_scale=0.5)
    kd = (k8.to(torch.float16).float() * 0.5).half()  # 0.5 * x is exact in fp16
    b = oracle.paged_attention_ref(q, kd, kd, bt, [50])
    assert torch.equal(a, b)


@pytest.mark.parametrize("name", golden_cases())
def test_fp16_oracle_matches_reference_fp16_path(name):
    """The pure-fp16 restatement is pinned to the reference's `out_pt` (upcast=False, reorder_ops=True)."""
    c = load_golden(name)
    pt = oracle.paged_attention_ref_fp16(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                         c["context_lens"], sinks=c["sinks"])
    err = (pt.float() - c["out_pt"].float()).abs()
    assert (err <= 2.0 ** -10 * c["out_pt"].float().abs() + 1e-7).all(), err.max().item()
