"""launch_kernels_reduce_static_scratch: the split variant for hosts that cannot allocate.

Some callers of this library have no allocator to offer: their device memory belongs to a
pool they do not control, or allocation is off limits once serving has started.  The entry
point keeps the per-partition scratch in an array built into the library instead.  This
test drives it through the C ABI (ctypes, no scratch tensors passed) and compares it with
launch_kernels_reduce on the same inputs -- same kernels, fixed summation order, so the bits
must be equal -- and with the CPU oracle, twice in a row with different shapes so that the
second call runs over whatever the first one left in the shared array.  Further cases: the
largest problem the array holds (accepted, right answers) and one row more (refused), and a
subset launch (refused: its scratch rows are addressed by sequence ids the host cannot see).

The file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes

import pytest
import torch

from _util import ATOL, RTOL, assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def _run_static(case, device, npart=None):
    """Calls the no-allocation entry point directly over the C ABI; returns `out` on the CPU."""
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    q = case["query"].to(device)
    k = case["key_cache"].to(device)
    v = case["value_cache"].to(device)
    bt = case["block_tables"].to(device)
    cl = case["context_lens"].to(device)
    sinks = case["sinks"].to(device) if case.get("sinks") is not None else None
    s, h, d = q.shape
    psize = pkg.partition_size(d)
    max_ctx = int(case["context_lens"].max())
    npart = npart or max(1, (max_ctx + psize - 1) // psize)
    out = torch.full((s, h, d), float("nan"), dtype=torch.float16, device=device)
    p = _cabi.PaParams()
    p.out, p.query = out.data_ptr(), q.data_ptr()
    p.key_cache, p.value_cache = k.data_ptr(), v.data_ptr()
    p.block_tables, p.context_lens = bt.data_ptr(), cl.data_ptr()
    p.sinks = sinks.data_ptr() if sinks is not None else None
    p.max_logits = p.exp_sums = p.tmp_out = None  # nothing to pass: that is the point
    p.num_seqs, p.num_heads, p.head_size = s, h, d
    p.num_kv_heads = k.size(2)
    p.max_num_partitions = npart
    p.max_blocks_per_seq = bt.size(1)
    p.block_size = k.size(1)
    p.num_queries_per_tokens = h // k.size(2)
    p.max_context_len = max_ctx
    p.num_blocks = k.size(0)
    p.sm_scale, p.fp8_scale, p.kv_dtype = case["sm_scale"], 1.0, _cabi.KV_F16
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), ctypes.c_void_p(stream))
    assert rc == _cabi.PA_OK, lib.pa_last_error().decode()
    torch.cuda.synchronize(device)
    return out.cpu()


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row(cuda_device):
    # two different problems back to back: the second one reuses the array the first one filled
    first = make_case(seed=71, num_seqs=3, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                      context_lens=[1500, 700, 40], sinks=True)
    second = make_case(seed=72, num_seqs=2, num_heads=12, num_kv_heads=4, head_size=64, block_size=64,
                       context_lens=[300, 2100])
    for case in (first, second):
        same_kernels = run_entry("reduce", case, cuda_device)["out"]
        got = _run_static(case, cuda_device)
        assert torch.equal(got, same_kernels), "static scratch must give the bits of launch_kernels_reduce"
        want = oracle.paged_attention_ref(case["query"], case["key_cache"], case["value_cache"],
                                          case["block_tables"], case["context_lens"], sm_scale=case["sm_scale"],
                                          sinks=case.get("sinks"))
        assert_close(got, want, atol=ATOL, rtol=RTOL, what="static scratch vs oracle")


def _shared_pool_case(seed, num_seqs, num_heads, num_kv_heads, context_lens, pool_blocks=4096):
    """Many sequences over one small pool of blocks (rows of the table may name the same
    physical block: attention only reads), so that a batch of a thousand sequences stays small."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.as_tensor(context_lens, dtype=torch.int32)
    mb = (int(ctx.max()) + 15) // 16
    return dict(query=torch.randn(num_seqs, num_heads, 128, generator=g).to(torch.float16),
                key_cache=torch.randn(pool_blocks, 16, num_kv_heads, 128, generator=g).to(torch.float16),
                value_cache=torch.randn(pool_blocks, 16, num_kv_heads, 128, generator=g).to(torch.float16),
                block_tables=torch.randint(0, pool_blocks, (num_seqs, mb), generator=g, dtype=torch.int32),
                context_lens=ctx, sinks=None, sm_scale=128 ** -0.5, fp8_scale=1.0, kv_dtype="float16",
                block_size=16)


def test_static_scratch_at_its_capacity(cuda_device):
    """rows = num_seqs * num_heads * max_num_partitions = 127100 with head size 128 needs
    2 * align256(4 * rows) + 256 * rows = 33554432 bytes, exactly the array; 127101 rows do not fit."""
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    s, h, npart = 1271, 4, 25
    assert 2 * ((4 * s * h * npart + 255) // 256 * 256) + 256 * s * h * npart == _cabi.STATIC_SCRATCH_BYTES
    g = torch.Generator().manual_seed(5)
    ctx = torch.randint(1, 700, (s,), generator=g).tolist()
    ctx[0], ctx[s // 2], ctx[-1] = 25 * 512, 25 * 512 - 1, 24 * 512 + 1  # the last partition row is in use
    case = _shared_pool_case(seed=6, num_seqs=s, num_heads=h, num_kv_heads=2, context_lens=ctx)
    got = _run_static(case, cuda_device, npart=npart)
    same_kernels = run_entry("reduce", case, cuda_device, max_num_partitions=npart)["out"]
    assert torch.equal(got, same_kernels)
    sample = [0, 1, 2, s // 2, s - 2, s - 1]
    want = oracle.paged_attention_ref(case["query"][sample], case["key_cache"], case["value_cache"],
                                      case["block_tables"][sample], case["context_lens"][sample],
                                      sm_scale=case["sm_scale"])
    assert_close(got[sample], want, atol=ATOL, rtol=RTOL, what="static scratch at capacity vs oracle")
    # one row more: 127101 = 3259 * 3 * 13
    lib = pkg.load_library()
    p = _cabi.PaParams()
    p.num_seqs, p.num_heads, p.head_size, p.num_kv_heads, p.max_num_partitions = 3259, 3, 128, 3, 13
    p.max_blocks_per_seq, p.block_size, p.num_queries_per_tokens = 512, 16, 1
    p.num_blocks, p.sm_scale, p.kv_dtype = 1 << 12, 0.1, _cabi.KV_F16
    assert lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), None) == _cabi.PA_ERR_BAD_ARG
    assert "127101 rows" in lib.pa_last_error().decode()


def test_static_scratch_refuses_subset_launches(cuda_device):
    """With seq_indices the kernels address scratch rows by sequence id; the library cannot
    bound ids it cannot read, so the fixed array is not offered to subset launches."""
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    ids = torch.tensor([5, 9], dtype=torch.int32, device=cuda_device)
    p = _cabi.PaParams()
    p.num_seqs, p.num_heads, p.head_size, p.num_kv_heads, p.max_num_partitions = 2, 8, 128, 2, 4
    p.max_blocks_per_seq, p.block_size, p.num_queries_per_tokens = 128, 16, 4
    p.num_blocks, p.sm_scale, p.kv_dtype = 1 << 12, 0.1, _cabi.KV_F16
    p.seq_indices = ids.data_ptr()
    assert lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), None) == _cabi.PA_ERR_BAD_ARG
    assert "seq_indices" in lib.pa_last_error().decode()


def test_static_scratch_rejects_problems_beyond_its_capacity(cuda_device):
    """Too many (sequence, head, partition) rows for the built-in array: refused on the host."""
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    p = _cabi.PaParams()
    p.num_seqs, p.num_heads, p.head_size, p.num_kv_heads = 4096, 64, 128, 8
    p.max_num_partitions, p.max_blocks_per_seq, p.block_size = 64, 2048, 16
    p.num_queries_per_tokens, p.num_blocks, p.sm_scale, p.kv_dtype = 8, 1 << 20, 0.1, _cabi.KV_F16
    rc = lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), None)
    assert rc == _cabi.PA_ERR_BAD_ARG
    msg = lib.pa_last_error().decode()
    assert "static scratch too small" in msg and str(_cabi.STATIC_SCRATCH_BYTES) in msg
