"""Loop variant on batches of many short sequences: the persistent kernel with whole-context items.

With at least four (sequence, head group) units per SM and a context-length hint that keeps the
longest possible item at 2 MiB or less, the loop entry points run the split variant's persistent
kernel, one work item per unit, results written straight to `out` (no scratch, no merge): the reference's loop semantics
(paged_attention_loop/launch_kernels_loop.h:16-54: one launch, no global scratch), without one
cluster launch per unit.  The batches here are large enough to take that path by themselves; a child
process forces it (PA_PERSISTENT_LOOP=1) for the ordinary parity and bookkeeping suites.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _contexts(n, hi, seed):
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(1, hi + 1, (n,), generator=g).tolist()
    # an empty context, single tokens, whole blocks and the longest length, away from the ends too
    for pos, val in ((0, 0), (1, 1), (2, 16), (3, hi), (n // 2, 0), (n // 2 + 1, 64), (n - 1, 1)):
        ctx[pos] = val
    return ctx


@pytest.mark.parametrize("kv,hk,group,d,bs,hi", [
    ("float16", 2, 4, 128, 16, 300),        # 2 heads per CTA: the warps of a head split its tokens
    ("float8_e5m2", 4, 2, 128, 16, 260),    # a warp per head
    ("float8_e4m3fn", 1, 8, 128, 64, 200),  # one head per CTA, blocks of 64: stages of two tiles
    ("float16", 4, 1, 64, 64, 520),         # head 64, crosses the 256-token partition size of the split variant
    ("float8_e5m2", 8, 5, 64, 32, 150),     # group 5, head 64
])
def test_many_short_sequences_match_the_oracle(cuda_device, kv, hk, group, d, bs, hi):
    hpc = 4 if hk % 4 == 0 else (2 if hk % 2 == 0 else 1)
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    n = (4 * sms * hpc + hk - 1) // hk + 8  # units = n * hk / hpc: just past four per SM
    ctx = _contexts(n, hi, seed=hk * 100 + d + bs)
    c = make_case(seed=31 + hk, num_seqs=n, num_heads=hk * group, num_kv_heads=hk, head_size=d, block_size=bs,
                  context_lens=ctx, kv_dtype=kv, sinks=True, fp8_scale=("amax" if kv == "float8_e4m3fn" else 1.0))
    res = run_entry("loop", c, cuda_device, poison=-5.0)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"],
                                      sinks=c["sinks"])
    assert_close(res["out"], want, what=f"persistent loop {kv}/hk{hk}/d{d}/bs{bs}")
    empty = [i for i, v in enumerate(ctx) if v == 0]
    assert empty and all(torch.count_nonzero(res["out"][i]) == 0 for i in empty)
    # the loop variant owns no scratch: whatever the caller passes stays as it was
    for name in ("max_logits", "exp_sums", "tmp_out"):
        assert (res[name] == -5.0).all(), name
    # same answer as the split-context pair on the same inputs, within the tolerance of the two summation orders
    assert_close(res["out"], run_entry("reduce", c, cuda_device)["out"], what="loop vs reduce")


def test_subset_launch_and_packed_tables(cuda_device):
    """seq_indices and packed block tables through the whole-context items."""
    from flash_attention_factory_b200 import lib
    from flash_attention_factory_b200.host_io import pack_block_tables

    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    n = 4 * sms + 40
    ctx = _contexts(n, 280, seed=5)
    c = make_case(seed=77, num_seqs=n, num_heads=8, num_kv_heads=4, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype="float8_e5m2")
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"])
    dev = cuda_device
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    cl = c["context_lens"].to(dev)
    ids, offsets = pack_block_tables(c["block_tables"], c["context_lens"], 16)
    subset = torch.arange(n - 1, -1, -1, dtype=torch.int32)[: n - 13]  # reversed order, 13 sequences left out
    out = torch.full((n, 8, 128), 9.0, dtype=torch.float16, device=dev)
    mod = lib.paged_attention_fp8_loop
    stats = torch.empty(n, 8, 1, device=dev)
    p = mod.params(stats, stats.clone(), torch.empty(n, 8, 1, 128, dtype=torch.float16, device=dev),
                   out, torch.zeros(1, device=dev), q, k, v, c["block_tables"].to(dev), cl, 2, c["sm_scale"], 1.0, 16,
                   max(ctx), torch.ones(8, device=dev), None, -1.0)
    ids_d, off_d, sub_d = ids.to(dev), offsets.to(dev), subset.to(dev)
    p.block_tables, p.block_table_offsets = ids_d.data_ptr(), off_d.data_ptr()
    p.num_seqs, p.seq_indices = subset.numel(), sub_d.data_ptr()
    from flash_attention_factory_b200.lib import _shim

    _shim.enqueue_entry(mod.ENTRY, p, dev)
    torch.cuda.synchronize(dev)
    got = out.cpu()
    covered = subset.long()
    assert_close(got[covered], want[covered], what="subset + packed tables")
    left_out = torch.tensor(sorted(set(range(n)) - set(subset.tolist())))
    assert (got[left_out] == 9.0).all()


def test_parity_suites_with_the_persistent_loop_forced(cuda_device):
    """The ordinary parity, bookkeeping, modifier, graph-capture, host-step and selector suites once
    more with every loop launch that carries a context-length hint sent through the persistent kernel."""
    env = dict(os.environ, PA_PERSISTENT_LOOP="1")
    files = ["tests/test_parity_gpu.py", "tests/test_bookkeeping_gpu.py", "tests/test_score_modifiers_gpu.py",
             "tests/test_per_head_scales_gpu.py", "tests/test_per_block_scales_gpu.py", "tests/test_context_clamp_gpu.py",
             "tests/test_cuda_graph_gpu.py", "tests/test_host_step_gpu.py", "tests/test_serving_gpu.py"]
    res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-k", "not persistent", *files],
                         cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=1500)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
