"""The asynchronous launch path can be recorded into a CUDA graph and replayed."""
import pytest
import torch

from _util import assert_close, make_case
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["loop", "reduce"])
@pytest.mark.parametrize("kv", ["float16", "float8_e4m3fn"])
def test_enqueue_is_graph_capturable(cuda_device, variant, kv):
    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import lib

    dev = cuda_device
    ctx = [300, 1100, 16, 513]
    c = make_case(seed=81, num_seqs=4, num_heads=8, num_kv_heads=4, head_size=128, block_size=16,
                  context_lens=ctx, kv_dtype=kv, fp8_scale=0.25 if kv != "float16" else 1.0)
    q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
    bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
    npart = 3
    ml = torch.empty(4, 8, npart, dtype=torch.float32, device=dev)
    es = torch.empty_like(ml)
    tmp = torch.empty(4, 8, npart, 128, dtype=torch.float16, device=dev)
    out = torch.zeros(4, 8, 128, dtype=torch.float16, device=dev)
    dbg = torch.zeros(1, dtype=torch.float32, device=dev)
    alibi = torch.ones(8, dtype=torch.float32, device=dev)
    fp8 = kv != "float16"
    mod = getattr(lib, f"paged_attention_{'fp8_' if fp8 else ''}{variant}")
    args = [ml, es, tmp, out, dbg, q, k, v, bt, cl, 2, c["sm_scale"]]
    if fp8:
        args.append(c["fp8_scale"])
    args += [16, max(ctx), alibi, None, -1.0]
    mod.enqueue(*args)  # first call outside capture: sets kernel attributes
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            mod.enqueue(*args)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], fp8_scale=c["fp8_scale"])
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize(dev)
        assert_close(out.cpu(), want, what=f"graph replay {variant}/{kv}")
    pkg.device_status()


def test_torch_custom_ops(cuda_device):
    """torch.ops.paged_attention_b200.* are registered and give the operators' results."""
    import flash_attention_factory_b200.torch_ops  # noqa: F401  (registers the ops)

    dev = cuda_device
    ctx = [700, 33]
    for kv, op in (("float16", "reduce"), ("float16", "loop"), ("float8_e5m2", "fp8_reduce"),
                   ("float8_e5m2", "fp8_loop")):
        c = make_case(seed=83, num_seqs=2, num_heads=8, num_kv_heads=2, head_size=128, block_size=16,
                      context_lens=ctx, kv_dtype=kv)
        q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
        bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
        ml = torch.empty(2, 8, 2, dtype=torch.float32, device=dev)
        es = torch.empty_like(ml)
        tmp = torch.empty(2, 8, 2, 128, dtype=torch.float16, device=dev)
        out = torch.zeros(2, 8, 128, dtype=torch.float16, device=dev)
        alibi = torch.ones(8, dtype=torch.float32, device=dev)
        fn = getattr(torch.ops.paged_attention_b200, op)
        if op.startswith("fp8"):
            fn(ml, es, tmp, out, q, k, v, bt, cl, 4, c["sm_scale"], 1.0, 16, max(ctx), alibi, None, -1.0)
        else:
            fn(ml, es, tmp, out, q, k, v, bt, cl, 4, c["sm_scale"], 16, max(ctx), alibi, None, -1.0)
        torch.cuda.synchronize(dev)
        want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                          c["context_lens"], sm_scale=c["sm_scale"])
        assert_close(out.cpu(), want, what=f"torch op {op}")
