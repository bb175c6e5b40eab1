"""Bit-exact checks of block-table indexing and partition bookkeeping (run on a B200)."""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def one_hot_value_case(kv_dtype, block_size, ctx, head_size=128, seed=0):
    """K = 0 (uniform softmax), V[token t] = one-hot at dim (t % head_size) times 2^(t // head_size):
    out[d] * ctx is then an exact integer code of WHICH tokens were read."""
    c = make_case(seed=seed, num_seqs=len(ctx), num_heads=2, num_kv_heads=1, head_size=head_size,
                  block_size=block_size, context_lens=ctx, kv_dtype="float16", extra_blocks=5)
    c["key_cache"].zero_()
    v = c["value_cache"]
    v.fill_(3.0)  # unread rows would show up as 3s
    for i, n in enumerate(ctx):
        for t in range(n):
            blk = int(c["block_tables"][i, t // block_size])
            row = v[blk, t % block_size, 0]
            row.zero_()
            row[t % head_size] = 2.0 ** (t // head_size)
    if kv_dtype != "float16":
        dt = {"float8_e5m2": torch.float8_e5m2, "float8_e4m3fn": torch.float8_e4m3fn}[kv_dtype]
        c["key_cache"] = c["key_cache"].to(dt)
        c["value_cache"] = c["value_cache"].to(dt)
        c["kv_dtype"] = kv_dtype
    return c


@pytest.mark.parametrize("kv", ["float16", "float8_e5m2", "float8_e4m3fn"])
@pytest.mark.parametrize("block_size,ctx", [(16, [128, 64, 256]), (64, [512, 128]), (32, [1024])])
@pytest.mark.parametrize("variant", ["loop", "reduce"])
def test_every_token_is_read_exactly_once(cuda_device, kv, block_size, ctx, variant):
    # ctx values are powers of two, so 1/ctx and every partial sum are exact in fp16/fp32
    c = one_hot_value_case(kv, block_size, ctx)
    res = run_entry(variant, c, cuda_device)
    for i, n in enumerate(ctx):
        expect = torch.zeros(128)
        for t in range(n):
            expect[t % 128] += 2.0 ** (t // 128)
        expect = (expect / n).to(torch.float16)
        for h in range(2):
            assert torch.equal(res["out"][i, h], expect), f"seq {i} head {h}"


@pytest.mark.parametrize("variant", ["loop", "reduce"])
def test_block_table_permutation_does_not_change_the_result(cuda_device, variant):
    c = make_case(seed=21, num_seqs=3, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=[700, 33, 512], kv_dtype="float8_e5m2")
    a = run_entry(variant, c, cuda_device)["out"]
    # move every physical block somewhere else and rewrite the table accordingly
    nb = c["key_cache"].shape[0]
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(1))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb)
    c2 = dict(c)
    c2["key_cache"] = c["key_cache"].view(torch.uint8)[perm].view(torch.float8_e5m2)
    c2["value_cache"] = c["value_cache"].view(torch.uint8)[perm].view(torch.float8_e5m2)
    c2["block_tables"] = inv[c["block_tables"].long()].to(torch.int32)
    b = run_entry(variant, c2, cuda_device)["out"]
    assert torch.equal(a, b)


@pytest.mark.parametrize("kv", ["float16", "float8_e4m3fn"])
def test_partition_scratch_layout_and_untouched_rows(cuda_device, kv):
    """max_logits / exp_sums / tmp_out: rows p < ceil(ctx/P) hold the partition statistics,
    rows p >= ceil(ctx/P) keep the caller's bytes; strides follow max_logits.size(2)."""
    ctx = [1300, 512, 1, 513]
    c = make_case(seed=31, num_seqs=4, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype=kv, sinks=True)
    npart = 5  # larger than needed (3): the stride must come from the tensor shape
    res = run_entry("reduce", c, cuda_device, max_num_partitions=npart, poison=-123.0)
    ml, es, tmp, written = oracle.partition_stats_ref(
        c["query"], c["key_cache"], c["value_cache"], c["block_tables"], c["context_lens"], 512,
        sm_scale=c["sm_scale"], sinks=c["sinks"], fp8_scale=c["fp8_scale"], max_num_partitions=npart)
    for i, n in enumerate(ctx):
        k = (n + 511) // 512
        assert written[i, :k].all()
        # untouched: exactly the poison value
        assert (res["max_logits"][i, :, k:] == -123.0).all()
        assert (res["exp_sums"][i, :, k:] == -123.0).all()
        assert (res["tmp_out"][i, :, k:] == -123.0).all()
        torch.testing.assert_close(res["max_logits"][i, :, :k], ml[i, :, :k], atol=1e-3, rtol=1e-3)
        torch.testing.assert_close(res["exp_sums"][i, :, :k], es[i, :, :k], atol=1e-3, rtol=1e-2)
        torch.testing.assert_close(res["tmp_out"][i, :, :k].float(), tmp[i, :, :k], atol=1e-3, rtol=1e-2)
    merged = oracle.merge_partitions_ref(res["max_logits"], res["exp_sums"], res["tmp_out"], ctx, 512)
    torch.testing.assert_close(res["out"].float(), merged.float(), atol=2e-3, rtol=1e-2)


def test_loop_leaves_the_scratch_buffers_alone(cuda_device):
    """The loop entry point accepts max_logits / exp_sums / tem_output and never writes them
    (launch_kernels_loop.h:39-47)."""
    c = make_case(seed=41, num_seqs=2, num_heads=4, num_kv_heads=4, head_size=64, block_size=16,
                  context_lens=[600, 10])
    res = run_entry("loop", c, cuda_device, poison=55.0)
    assert (res["max_logits"] == 55.0).all() and (res["exp_sums"] == 55.0).all()
    assert (res["tmp_out"] == 55.0).all()


def test_out_of_range_block_ids_read_zeros_without_faulting(cuda_device):
    """A block id >= num_blocks is outside the TMA descriptor and reads as zeros."""
    c = make_case(seed=51, num_seqs=1, num_heads=2, num_kv_heads=1, head_size=128, block_size=16,
                  context_lens=[64])
    c["block_tables"][0, 2] = 10_000
    k = c["key_cache"].clone()
    v = c["value_cache"].clone()
    zero = torch.zeros(1, *k.shape[1:], dtype=k.dtype)
    cz = dict(c)
    cz["key_cache"] = torch.cat([k, zero])
    cz["value_cache"] = torch.cat([v, zero])
    cz["block_tables"] = c["block_tables"].clone()
    cz["block_tables"][0, 2] = k.shape[0]
    want = run_entry("loop", cz, cuda_device)["out"]
    got = run_entry("loop", c, cuda_device)["out"]
    assert torch.equal(got, want)
    import flash_attention_factory_b200 as pkg

    pkg.device_status()


@pytest.mark.parametrize("d,kv", [(128, "float16"), (64, "float8_e5m2")])
def test_both_merge_kernels_give_the_same_bits(cuda_device, d, kv):
    """The launcher picks the warp-per-head merge for large batches and the CTA-per-head one
    otherwise; a sequence must not change its bits with the size of the batch it sits in."""
    import os
    import subprocess
    import sys
    import textwrap

    # the kernel choice is read once per process: compare two child processes
    code = textwrap.dedent(f"""
        import sys, torch
        sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parent)!r})
        from _util import make_case, run_entry
        ctx = [3000, 513, 140 * {512 if d == 128 else 256}, 1, 7000, 2049]
        c = make_case(seed=91, num_seqs=len(ctx), num_heads=8, num_kv_heads=2, head_size={d}, block_size=16,
                      context_lens=ctx, kv_dtype={kv!r}, sinks=True)
        out = run_entry("reduce", c, torch.device("cuda:0"))["out"]
        torch.save(out, sys.argv[1])
    """)
    outs = []
    for which in ("cta", "warp"):
        path = f"/tmp/merge_{which}_{d}.pt"
        env = dict(os.environ, PA_MERGE_KERNEL=which)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=600)
        outs.append(torch.load(path))
    assert torch.isfinite(outs[0].float()).all()
    assert torch.equal(outs[0], outs[1])


def test_large_batch_takes_the_warp_merge_and_matches_the_oracle(cuda_device):
    from _util import assert_close

    ctx = [600 + 37 * (i % 40) for i in range(1024)]  # 1024 x 8 heads = 8192 (sequence, head) pairs
    c = make_case(seed=92, num_seqs=1024, num_heads=8, num_kv_heads=8, head_size=64, block_size=64,
                  context_lens=ctx, kv_dtype="float8_e5m2")
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"])
    assert_close(run_entry("reduce", c, cuda_device)["out"], want, what="large batch")


@pytest.mark.parametrize("d,kv", [(64, "float16"), (128, "float8_e4m3fn")])
def test_bits_do_not_depend_on_the_position_in_a_large_batch(cuda_device, d, kv):
    """More work than two rounds of the persistent grid: which CTA computes an item, and when, is
    decided at run time.  A sequence must get the same bits at the front of the batch and at
    the back, and both must match the oracle."""
    import flash_attention_factory_b200 as pkg

    psize = pkg.partition_size(d)
    props = torch.cuda.get_device_properties(cuda_device)
    # items = num_seqs * (kv heads / 4) * partitions: a little more than two per resident CTA
    s, hk = 8, 8
    parts = -(-4 * props.multi_processor_count // (s * (hk // 4))) + 1
    ctx = [parts * psize - 7] * s
    c = make_case(seed=61, num_seqs=s, num_heads=hk * 2, num_kv_heads=hk, head_size=d, block_size=16,
                  context_lens=ctx, kv_dtype=kv, fp8_scale=0.5 if kv != "float16" else 1.0)
    fwd = run_entry("reduce", c, cuda_device, poison=-3.0)
    r = dict(c)
    flip = torch.arange(s - 1, -1, -1)
    r["query"] = c["query"][flip].contiguous()
    r["block_tables"] = c["block_tables"][flip].contiguous()
    r["context_lens"] = c["context_lens"][flip].contiguous()
    rev = run_entry("reduce", r, cuda_device, poison=-3.0)
    for name in ("out", "max_logits", "exp_sums", "tmp_out"):
        assert torch.equal(fwd[name], rev[name][flip]), f"{name}: bits depend on the position in the batch"
    # alone, the sequence is a small launch (FP8: the default CTA shape instead of the wide one)
    solo = dict(c)
    solo["query"] = c["query"][3:4].contiguous()
    solo["block_tables"] = c["block_tables"][3:4].contiguous()
    solo["context_lens"] = c["context_lens"][3:4].contiguous()
    alone = run_entry("reduce", solo, cuda_device, poison=-3.0)
    for name in ("out", "max_logits", "exp_sums", "tmp_out"):
        assert torch.equal(fwd[name][3:4], alone[name]), f"{name}: bits depend on the rest of the batch"
    for i in (0, s - 1):
        want = oracle.paged_attention_ref(c["query"][i:i + 1], c["key_cache"], c["value_cache"],
                                          c["block_tables"][i:i + 1], c["context_lens"][i:i + 1],
                                          sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
        assert_close(fwd["out"][i:i + 1], want, what=f"sequence {i}")
    pkg.device_status()
