"""The pipelined decode step with host buffers (pa_decode_step_host_batch) and packed block tables.

Packed tables (`pa_params.block_table_offsets`) are another way to hand the kernels the same
block ids, so every entry point must give the bits of the dense form; the pipelined step cuts
the batch into sub-batches of consecutive sequences, which for the reduce entry points gives
the bits of one launch over the whole batch.
"""
import ctypes

import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu

CTX = [900, 17, 512, 1300, 1, 2049, 0, 640, 77, 1536, 333]


def _setup(dev, kv, variant, io, case, npart, h, hk, d, bs):
    from flash_attention_factory_b200 import lib

    fp8 = kv != "float16"
    k, v = case["key_cache"].to(dev), case["value_cache"].to(dev)
    s = len(CTX)
    ml = torch.full((s, h, npart), -5.0, dtype=torch.float32, device=dev)
    es = torch.full_like(ml, -5.0)
    tmp = torch.full((s, h, npart, d), -5.0, dtype=torch.float16, device=dev)
    dbg = torch.zeros(1, dtype=torch.float32, device=dev)
    alibi = torch.ones(h, dtype=torch.float32, device=dev)
    mod = getattr(lib, f"paged_attention_{'fp8_' if fp8 else ''}{variant}")

    def args(out, q, bt, cl):
        a = [ml, es, tmp, out, dbg, q, k, v, bt, cl, h // hk, case["sm_scale"]]
        if fp8:
            a.append(case["fp8_scale"])
        return a + [bs, max(CTX), alibi, None, -1.0]

    return mod, args, (ml, es, tmp, k, v)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("sub_batches", [0, 1, 3, 8])
@pytest.mark.parametrize("variant,kv", [("reduce", "float16"), ("reduce", "float8_e5m2"), ("loop", "float8_e4m3fn")])
def test_pipelined_host_step_matches_enqueue_and_oracle(cuda_device, variant, kv, sub_batches, packed):
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200.host_io import DecodeBatchIO

    dev = cuda_device
    s, h, hk, d, bs = len(CTX), 8, 4, 128, 16
    c = make_case(seed=123, num_seqs=s, num_heads=h, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=CTX, kv_dtype=kv, fp8_scale=(0.5 if kv != "float16" else 1.0))
    npart = 5
    io = DecodeBatchIO(s, h, d, c["block_tables"].size(1), dev,
                       packed_capacity=(sum((x + bs - 1) // bs for x in CTX) + 7 if packed else 0))
    mod, args, keep = _setup(dev, kv, variant, io, c, npart, h, hk, d, bs)

    # the same operator on device-resident dense inputs, one launch over the whole batch
    want_dev = torch.zeros(s, h, d, dtype=torch.float16, device=dev)
    mod.enqueue(*args(want_dev, c["query"].to(dev), c["block_tables"].to(dev), c["context_lens"].to(dev)))
    torch.cuda.synchronize(dev)
    scratch_whole = [t.clone() for t in keep[:3]]

    step = io.bind(mod.ENTRY, mod.params(*args(io.out, io.query, io.block_tables if not packed else
                                               c["block_tables"].to(dev), io.context_lens)),
                   sub_batches=sub_batches)
    io.query_host.copy_(c["query"])
    io.context_lens_host.copy_(c["context_lens"])
    io.set_block_tables(c["block_tables"], c["context_lens"], bs)
    io.out_host.fill_(7.0)
    for t in keep[:3]:
        t.fill_(-5.0)
    got = step.run().clone()
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    assert_close(got, want, what=f"pipelined step {variant}/{kv}/n={sub_batches}/packed={packed}")
    if variant == "reduce":
        assert torch.equal(got, want_dev.cpu()), "sub-batches must give the bits of one launch over the batch"
        for name, a, b in zip(("max_logits", "exp_sums", "tmp_out"), keep[:3], scratch_whole):
            assert torch.equal(a, b), f"{name} differs from the single launch"
    # a second step with other inputs through the same buffers
    io.query_host.mul_(-0.5)
    got2 = step.run().clone()
    want2 = oracle.paged_attention_ref(io.query_host.clone(), c["key_cache"], c["value_cache"], c["block_tables"],
                                       c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    assert_close(got2, want2, what="second pipelined step")
    pkg.device_status()


@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_packed_block_tables_give_the_bits_of_dense_tables(cuda_device, variant, kv):
    from flash_attention_factory_b200.host_io import pack_block_tables
    from flash_attention_factory_b200.lib import _shim

    dev = cuda_device
    s, h, hk, d, bs = len(CTX), 8, 4, 128, 16
    c = make_case(seed=321, num_seqs=s, num_heads=h, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=CTX, kv_dtype=kv)
    mod, args, keep = _setup(dev, kv, variant, None, c, 5, h, hk, d, bs)
    q, bt, cl = c["query"].to(dev), c["block_tables"].to(dev), c["context_lens"].to(dev)
    dense = torch.zeros(s, h, d, dtype=torch.float16, device=dev)
    mod.enqueue(*args(dense, q, bt, cl))
    torch.cuda.synchronize(dev)
    ids, offsets = pack_block_tables(c["block_tables"], c["context_lens"], bs)
    ids_dev, off_dev = ids.to(dev), offsets.to(dev)
    out = torch.zeros_like(dense)
    p = mod.params(*args(out, q, bt, cl))
    p.block_tables = ids_dev.data_ptr()
    p.block_table_offsets = off_dev.data_ptr()
    p.max_blocks_per_seq = 0  # not used with packed tables
    _shim.enqueue_entry(mod.ENTRY, p, dev)
    torch.cuda.synchronize(dev)
    assert torch.equal(out, dense)
    # a context length beyond its packed row is cut to the row (here: sequence 3 claims 5000 tokens)
    lying = c["context_lens"].clone()
    lying[3] = 5000
    cl2 = lying.to(dev)
    p2 = mod.params(*args(out, q, bt, cl2))
    p2.block_tables, p2.block_table_offsets, p2.max_blocks_per_seq = ids_dev.data_ptr(), off_dev.data_ptr(), 0
    out.zero_()
    _shim.enqueue_entry(mod.ENTRY, p2, dev)
    torch.cuda.synchronize(dev)
    honest3 = (CTX[3] + bs - 1) // bs * bs  # the row holds whole blocks: 1312 tokens
    c3 = dict(c)
    c3["context_lens"] = c["context_lens"].clone()
    c3["context_lens"][3] = honest3
    want = oracle.paged_attention_ref(c3["query"], c3["key_cache"], c3["value_cache"], c3["block_tables"],
                                      c3["context_lens"], sm_scale=c["sm_scale"])
    assert_close(out.cpu(), want, what="packed row limit")


def test_pipelined_host_step_rejects_bad_arguments(cuda_device):
    from flash_attention_factory_b200 import _cabi

    lib = _cabi.load_library()
    p, io = _cabi.PaParams(), _cabi.PaHostBatch()
    with torch.cuda.device(cuda_device):
        assert lib.pa_decode_step_host_batch(9, ctypes.byref(p), ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
        p.num_seqs = 4  # buffers missing
        assert lib.pa_decode_step_host_batch(1, ctypes.byref(p), ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
        p.seq_indices = 0x1000
        assert lib.pa_decode_step_host_batch(1, ctypes.byref(p), ctypes.byref(io), None, 1) == _cabi.PA_ERR_BAD_ARG
        assert "seq_indices" in lib.pa_last_error().decode()
