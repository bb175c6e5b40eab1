"""Parity of the four CUDA entry points with the CPU oracle (run on a B200).

Every case goes through flash_attention_factory_b200.lib.*.run, i.e. through the C ABI.
Tolerance: atol 1e-3 / rtol 1e-2 against the fp32 oracle (for FP8: the oracle applied to
the identically dequantised cache), plus the reference's own acceptance criterion
max|out-ref| <= 3 max|out_pt-ref| + 1e-5 (test_paged.py:603-604) on the golden cases.
"""
import pytest
import torch

from _util import assert_close, golden_cases, load_golden, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu

VARIANTS = ["loop", "reduce"]


def oracle_out(case):
    return oracle.paged_attention_ref(case["query"], case["key_cache"], case["value_cache"],
                                      case["block_tables"], case["context_lens"],
                                      sm_scale=case["sm_scale"], sinks=case.get("sinks"),
                                      fp8_scale=case.get("fp8_scale", 1.0))


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name", golden_cases())
def test_golden_vectors(cuda_device, name, variant):
    c = load_golden(name)
    c["fp8_scale"] = 1.0
    res = run_entry(variant, c, cuda_device)
    assert_close(res["out"], c["out_ref"], what=f"{name}/{variant}")
    err = (res["out"].float() - c["out_ref"].float()).abs().max().item()
    bound = 3 * (c["out_pt"].float() - c["out_ref"].float()).abs().max().item() + 1e-5
    assert err <= bound, f"reference criterion: {err} > {bound}"
    assert len(res["times"]) == (2 if variant == "reduce" else 1)
    assert all(t > 0 for t in res["times"])


# (kv_dtype, heads, kv_heads, head_size, block_size, context_lens, sinks)
SHAPES = [
    ("float16", 8, 8, 128, 16, [1, 15, 16, 17], False),
    ("float16", 8, 8, 128, 16, [511, 512, 513, 64], True),
    ("float16", 8, 1, 128, 64, [128, 339], True),
    ("float16", 10, 2, 128, 64, [1024, 800], False),
    ("float16", 14, 2, 64, 64, [256, 799], True),
    ("float16", 12, 2, 64, 16, [255, 256, 257], False),
    ("float16", 6, 2, 128, 32, [2048, 1000], False),
    ("float16", 3, 1, 128, 128, [700, 129], True),
    ("float16", 32, 32, 128, 16, [4096], False),
    ("float8_e5m2", 32, 8, 128, 16, [1024, 3000, 2047], False),
    ("float8_e5m2", 40, 8, 64, 64, [1500, 1490], True),
    ("float8_e5m2", 5, 1, 128, 16, [1, 31, 33, 600], True),
    ("float8_e5m2", 16, 2, 64, 16, [300, 257], False),
    ("float8_e4m3fn", 64, 8, 128, 16, [5000, 4097], False),
    ("float8_e4m3fn", 14, 2, 64, 64, [777], True),
    ("float8_e4m3fn", 7, 1, 128, 32, [65, 64, 63], False),
]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}-h{s[1]}k{s[2]}-d{s[3]}-bs{s[4]}-{'sink' if s[6] else 'nosink'}-{len(s[5])}seq")
def test_shapes_against_oracle(cuda_device, shape, variant):
    kv, h, hk, d, bs, ctx, sinks = shape
    c = make_case(seed=100 + SHAPES.index(shape), num_seqs=len(ctx), num_heads=h, num_kv_heads=hk,
                  head_size=d, block_size=bs, context_lens=ctx, kv_dtype=kv, sinks=sinks, extra_blocks=3)
    res = run_entry(variant, c, cuda_device)
    assert_close(res["out"], oracle_out(c), what=f"{shape}/{variant}")


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("kv,scale", [("float8_e4m3fn", "amax"), ("float8_e5m2", 0.5), ("float8_e4m3fn", 2.0)])
def test_fp8_scale(cuda_device, kv, scale, variant):
    c = make_case(seed=5, num_seqs=2, num_heads=16, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[1234, 515], kv_dtype=kv, fp8_scale=scale)
    res = run_entry(variant, c, cuda_device)
    assert_close(res["out"], oracle_out(c), what=f"{kv}/{scale}/{variant}")


@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_every_group_size(cuda_device, kv, group):
    c = make_case(seed=group, num_seqs=2, num_heads=2 * group, num_kv_heads=2, head_size=128,
                  block_size=16, context_lens=[700, 90], kv_dtype=kv, sinks=(group % 2 == 0))
    want = oracle_out(c)
    for variant in VARIANTS:
        assert_close(run_entry(variant, c, cuda_device)["out"], want, what=f"G={group}/{variant}")


def test_baseline_config_1(cuda_device):
    """Loop variant, fp16, S=4, H=HK=8, D=128, bs=16, ctx uniform in [1,512], seed 0."""
    g = torch.Generator().manual_seed(0)
    ctx = torch.randint(1, 513, (4,), generator=g).tolist()
    c = make_case(seed=0, num_seqs=4, num_heads=8, num_kv_heads=8, head_size=128, block_size=16,
                  context_lens=ctx)
    assert c["key_cache"].shape[0] == 4 * 32 or max(ctx) <= 496
    want = oracle_out(c)
    for variant in VARIANTS:
        assert_close(run_entry(variant, c, cuda_device)["out"], want, what=f"C1/{variant}")


def test_scaled_down_baseline_configs(cuda_device):
    """C2 / C3 / C4 shapes with fewer sequences (the oracle has to finish in seconds)."""
    g = torch.Generator().manual_seed(3)
    c2 = make_case(seed=2, num_seqs=2, num_heads=32, num_kv_heads=32, head_size=128, block_size=16,
                   context_lens=[4096, 4096])
    assert_close(run_entry("reduce", c2, cuda_device)["out"], oracle_out(c2), what="C2")
    ctx3 = torch.randint(1024, 8193, (3,), generator=g).tolist()
    c3 = make_case(seed=3, num_seqs=3, num_heads=32, num_kv_heads=8, head_size=128, block_size=16,
                   context_lens=ctx3, kv_dtype="float8_e5m2")
    assert_close(run_entry("loop", c3, cuda_device)["out"], oracle_out(c3), what="C3")
    c4 = make_case(seed=4, num_seqs=1, num_heads=64, num_kv_heads=8, head_size=128, block_size=16,
                   context_lens=[32768], kv_dtype="float8_e4m3fn", fp8_scale="amax")
    want4 = oracle_out(c4)
    assert_close(run_entry("reduce", c4, cuda_device)["out"], want4, what="C4/reduce")
    assert_close(run_entry("loop", c4, cuda_device)["out"], want4, what="C4/loop")


def test_long_contexts_of_the_reference_matrix(cuda_device):
    """seqlen_k 20000 / 40000 / 50000 of test_paged.py:238-240, block 64, varlen."""
    for kv, d, h, hk, ctx in (("float16", 128, 8, 1, [20000, 19985]), ("float8_e5m2", 64, 4, 2, [40000]),
                              ("float16", 64, 2, 2, [50000])):
        c = make_case(seed=ctx[0], num_seqs=len(ctx), num_heads=h, num_kv_heads=hk, head_size=d,
                      block_size=64, context_lens=ctx, kv_dtype=kv, sinks=True)
        want = oracle_out(c)
        for variant in VARIANTS:
            assert_close(run_entry(variant, c, cuda_device)["out"], want, what=f"{ctx}/{variant}")


def test_empty_context_writes_zeros(cuda_device):
    c = make_case(seed=9, num_seqs=3, num_heads=4, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[0, 40, 0])
    want = oracle_out(c)
    for variant in VARIANTS:
        res = run_entry(variant, c, cuda_device, poison=7.0)
        assert torch.count_nonzero(res["out"][0]) == 0 and torch.count_nonzero(res["out"][2]) == 0
        assert_close(res["out"], want, what=f"ctx0/{variant}")


@pytest.mark.parametrize("kv", ["float16", "float8_e5m2", "float8_e4m3fn"])
def test_garbage_past_the_context_is_ignored(cuda_device, kv):
    """NaN / Inf codes in the unused tail of the last block and in unused blocks never leak."""
    ctx = [37, 130]
    c = make_case(seed=11, num_seqs=2, num_heads=8, num_kv_heads=2, head_size=128, block_size=64,
                  context_lens=ctx, kv_dtype=kv)
    want = oracle_out(c)
    for name in ("key_cache", "value_cache"):
        raw = c[name].view(torch.int16 if kv == "float16" else torch.uint8)
        nan_bits = 0x7E00 if kv == "float16" else (0x7F if kv == "float8_e4m3fn" else 0x7E)
        for i, n in enumerate(ctx):
            blk = int(c["block_tables"][i, n // 64])
            raw[blk, n % 64:] = nan_bits
    for variant in VARIANTS:
        assert_close(run_entry(variant, c, cuda_device)["out"], want, what=f"garbage/{kv}/{variant}")


@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_ragged_batch_with_one_long_sequence(cuda_device, kv):
    """A few hundred units and a long context-length hint: the loop variant takes clusters of 8, so
    that the long sequence is spread over 8 CTAs, and most CTAs of the short sequences' clusters get
    no token.  The block tables draw from a small shared pool (sequences may read the same blocks)."""
    g = torch.Generator().manual_seed(123)
    n, long_ctx, pool = 200, 24000, 2048
    ctx = [long_ctx] + torch.randint(1, 600, (n - 1,), generator=g).tolist()
    ctx[7], ctx[8], ctx[9] = 0, 1, 16
    c = make_case(seed=321, num_seqs=1, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[16 * pool], kv_dtype=kv, sinks=True)  # one sequence's worth of blocks = the pool
    c["query"] = torch.randn(n, 8, 128, generator=g).to(torch.float16)
    c["block_tables"] = torch.randint(0, pool, (n, long_ctx // 16), generator=g).to(torch.int32)
    c["context_lens"] = torch.tensor(ctx, dtype=torch.int32)
    want = oracle_out(c)
    for variant in VARIANTS:
        assert_close(run_entry(variant, c, cuda_device)["out"], want, what=f"ragged/{kv}/{variant}")
