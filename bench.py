"""Benchmark of the paged-attention decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl ours|reference]

A step is one call of the operator over one batch.  At N=1 the default workload is
BASELINE.json's configs[1] (reduce variant, fp16 KV, 64 sequences x 4096 tokens, 32 heads);
`--config c1|c3|c4|c5` select the other BASELINE configurations.  With N>1 (torchrun, one
rank per GPU) every rank runs the same configuration on its own shard with its own KV pool
and block tables (weak scaling, no data-path collective); `c5` instead splits one batch of
1024 ragged sequences over the ranks by cumulative KV length (strong scaling).

Rank 0 prints ONE JSON line.  `value` is KV bytes / time with all inputs resident in HBM;
`e2e` is the same metric through flash_attention_factory_b200.lib.*.run with the per-step
inputs (query, block tables, context lengths) copied from pinned host memory and the output
copied back inside the timed region.  The KV cache is state of the serving process, like
weights, and stays resident.  `--impl reference` times the CPU oracle (the reference's own
CPU algorithm, oracle/paged_attention_oracle.py) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


# ----------------------------------------------------------------------------- workloads
def config_spec(name: str) -> dict:
    """Shapes of BASELINE.json's configs (all head_size 128, block_size 16)."""
    specs = {
        "c1": dict(variant="loop", kv="float16", num_seqs=4, heads=8, kv_heads=8, ctx=("uniform", 1, 512)),
        "c2": dict(variant="reduce", kv="float16", num_seqs=64, heads=32, kv_heads=32, ctx=("const", 4096)),
        "c3": dict(variant="loop", kv="float8_e5m2", num_seqs=128, heads=32, kv_heads=8,
                   ctx=("uniform", 1024, 8192)),
        "c4": dict(variant="reduce", kv="float8_e4m3fn", num_seqs=16, heads=64, kv_heads=8,
                   ctx=("const", 32768)),
        "c5": dict(variant="auto", kv="float8_e5m2", num_seqs=1024, heads=32, kv_heads=8,
                   ctx=("lognormal", 7.5, 1.0, 16, 32768)),
    }
    s = dict(specs[name])
    s.update(name=name, head_size=128, block_size=16)
    return s


def draw_context_lens(spec: dict, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    kind = spec["ctx"][0]
    n = spec["num_seqs"]
    if kind == "const":
        return torch.full((n,), spec["ctx"][1], dtype=torch.int32)
    if kind == "uniform":
        return torch.randint(spec["ctx"][1], spec["ctx"][2] + 1, (n,), generator=g).to(torch.int32)
    mu, sigma, lo, hi = spec["ctx"][1:]
    x = torch.exp(torch.randn(n, generator=g) * sigma + mu).round().clamp(lo, hi)
    return x.to(torch.int32)


class Workload:
    """Device-resident inputs of one rank plus pinned host copies of the per-step inputs."""

    def __init__(self, spec: dict, ctx: torch.Tensor, device, seed: int, variant: str):
        import flash_attention_factory_b200 as pkg

        self.spec, self.device, self.variant = spec, device, variant
        d, bs = spec["head_size"], spec["block_size"]
        h, hk = spec["heads"], spec["kv_heads"]
        s = int(ctx.numel())
        self.num_seqs, self.ctx = s, ctx
        self.fp8 = spec["kv"] != "float16"
        self.elt = 1 if self.fp8 else 2
        max_ctx = int(ctx.max()) if s else 0
        self.max_ctx = max_ctx
        mb = max(1, (max_ctx + bs - 1) // bs)
        blocks_needed = [(int(c) + bs - 1) // bs for c in ctx.tolist()]
        num_blocks = max(1, sum(blocks_needed))
        g = torch.Generator(device=device).manual_seed(seed)
        gc = torch.Generator().manual_seed(seed)
        # block tables: a random permutation of the physical blocks, cut into rows
        perm = torch.randperm(num_blocks, generator=gc).to(torch.int32)
        if spec.get("block_order") == "sequential":
            perm = torch.arange(num_blocks, dtype=torch.int32)
        bt = torch.zeros(s, mb, dtype=torch.int32)
        pos = 0
        for i, nb in enumerate(blocks_needed):
            bt[i, :nb] = perm[pos:pos + nb]
            pos += nb
        shape = (num_blocks, bs, hk, d)
        cache_bytes = 2 * num_blocks * bs * hk * d * self.elt
        # rotate over several cache copies when one copy could live in L2
        self.copies = 1 if cache_bytes >= 4 * L2_BYTES else min(50, math.ceil(4 * L2_BYTES / cache_bytes))
        if spec.get("cache_copies"):
            self.copies = int(spec["cache_copies"])  # diagnostic: 1 copy of a small cache stays in L2
        self.fp8_scale = 1.0
        self.k, self.v = [], []
        for _ in range(self.copies):
            k = torch.randn(shape, generator=g, device=device, dtype=torch.float16)
            v = torch.randn(shape, generator=g, device=device, dtype=torch.float16)
            if spec["kv"] == "float8_e5m2":
                k, v = k.to(torch.float8_e5m2), v.to(torch.float8_e5m2)
            elif spec["kv"] == "float8_e4m3fn":
                self.fp8_scale = float(max(k.abs().max(), v.abs().max())) / 448.0
                k = (k.float() / self.fp8_scale).to(torch.float8_e4m3fn)
                v = (v.float() / self.fp8_scale).to(torch.float8_e4m3fn)
            self.k.append(k)
            self.v.append(v)
        self.q_host = torch.randn(s, h, d, generator=gc).to(torch.float16).pin_memory()
        self.bt_host = bt.pin_memory()
        self.ctx_host = ctx.clone().pin_memory()
        self.q = self.q_host.to(device)
        self.bt = self.bt_host.to(device)
        self.cl = self.ctx_host.to(device)
        psize = pkg.partition_size(d)
        self.npart = max(1, (max_ctx + psize - 1) // psize)
        self.max_logits = torch.empty(s, h, self.npart, dtype=torch.float32, device=device)
        self.exp_sums = torch.empty_like(self.max_logits)
        self.tmp_out = torch.empty(s, h, self.npart, d, dtype=torch.float16, device=device)
        self.out = torch.zeros(s, h, d, dtype=torch.float16, device=device)
        self.out_host = torch.empty(s, h, d, dtype=torch.float16).pin_memory()
        self.debug = torch.zeros(1, dtype=torch.float32, device=device)
        self.alibi = torch.ones(h, dtype=torch.float32, device=device)
        self.sm_scale = 1.0 / math.sqrt(d)
        self.group = h // hk
        self.kv_bytes = int(ctx.to(torch.int64).sum()) * hk * d * 2 * self.elt
        self.h2d_bytes = self.q_host.numel() * 2 + self.bt_host.numel() * 4 + self.ctx_host.numel() * 4
        self.d2h_bytes = self.out_host.numel() * 2

    def module(self):
        from flash_attention_factory_b200 import lib

        return getattr(lib, f"paged_attention_{'fp8_' if self.fp8 else ''}{self.variant}")

    def args(self, step: int, q=None, bt=None, cl=None):
        i = step % self.copies
        a = [self.max_logits, self.exp_sums, self.tmp_out, self.out, self.debug,
             self.q if q is None else q, self.k[i], self.v[i], self.bt if bt is None else bt,
             self.cl if cl is None else cl, self.group, self.sm_scale]
        if self.fp8:
            a.append(self.fp8_scale)
        a += [self.spec["block_size"], self.max_ctx, self.alibi, None, -1.0]
        return a

    def enqueue(self, step: int, q=None, bt=None, cl=None) -> None:
        """One asynchronous call of the operator on the current stream."""
        if self.variant != "auto":
            if q is not None or bt is not None or cl is not None:
                self.module().enqueue(*self.args(step, q, bt, cl))
                return
            # the argument block of a cache copy is checked and built once, like a serving loop
            # would do; a call then is one call into the library
            from flash_attention_factory_b200.lib import _shim

            cache = self.__dict__.setdefault("_params", {})
            i = step % self.copies
            if i not in cache:
                cache[i] = self.module().params(*self.args(i))
            _shim.enqueue_entry(self.module().ENTRY, cache[i], self.device)
            return
        from flash_attention_factory_b200.serving import AutoDecodePlan, paged_attention_auto

        if getattr(self, "plan", None) is None:
            self.plan = AutoDecodePlan(self.ctx.tolist(), self.spec["heads"], self.spec["head_size"],
                                       self.spec["block_size"], self.bt.size(1), self.device)
        i = step % self.copies
        paged_attention_auto(self.plan, self.out, self.q if q is None else q, self.k[i], self.v[i],
                             self.bt if bt is None else bt, self.cl if cl is None else cl, self.group,
                             self.sm_scale, self.fp8_scale)

    @property
    def launches_per_step(self) -> int:
        if self.variant == "auto":
            plan = getattr(self, "plan", None)
            return (1 if plan is None or plan.loop is not None else 0) + \
                   (2 if plan is None or plan.reduce is not None else 0)
        return 2 if self.variant == "reduce" else 1


def shard_by_kv_length(ctx: torch.Tensor, world: int, rank: int, scheme: str = "contiguous") -> torch.Tensor:
    """This rank's sequences: the contiguous range whose cumulative KV length falls in its share,
    or (scheme "lpt") the ids dealt longest-first to the lightest rank."""
    from flash_attention_factory_b200.sharding import shard_sequences_by_kv_length, shard_sequences_lpt

    if scheme == "lpt":
        return ctx[torch.tensor(shard_sequences_lpt(ctx.tolist(), world)[rank], dtype=torch.long)].clone()
    lo, hi = shard_sequences_by_kv_length(ctx.tolist(), world)[rank]
    return ctx[lo:hi].clone()


# --------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------ CPU oracle
def cpu_sample_inputs(w: Workload, n_seq: int):
    """A bounded sample of the rank's workload for the CPU oracle: the first n_seq sequences
    with their blocks compacted into a small cache (block ids renumbered)."""
    n_seq = min(n_seq, w.num_seqs)
    bs = w.spec["block_size"]
    rows, tables, pos = [], [], 0
    mb = w.bt.shape[1]
    for i in range(n_seq):
        nb = (int(w.ctx[i]) + bs - 1) // bs
        rows.append(w.bt_host[i, :nb].long())
        t = torch.zeros(mb, dtype=torch.int32)
        t[:nb] = torch.arange(pos, pos + nb, dtype=torch.int32)
        tables.append(t)
        pos += nb
    idx = torch.cat(rows).to(w.device)
    k = w.k[0][idx].cpu()
    v = w.v[0][idx].cpu()
    return dict(query=w.q_host[:n_seq].clone(), key_cache=k, value_cache=v,
                block_tables=torch.stack(tables), context_lens=w.ctx[:n_seq].clone(),
                sm_scale=w.sm_scale, fp8_scale=w.fp8_scale)


def use_all_host_threads() -> None:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core."""
    n = os.cpu_count() or 1
    if torch.get_num_threads() != n:
        torch.set_num_threads(n)


def time_cpu_oracle(sample: dict) -> float:
    from oracle import paged_attention_oracle as oracle

    use_all_host_threads()

    t0 = time.perf_counter()
    oracle.paged_attention_ref(sample["query"], sample["key_cache"], sample["value_cache"],
                               sample["block_tables"], sample["context_lens"], sm_scale=sample["sm_scale"],
                               fp8_scale=sample["fp8_scale"])
    return time.perf_counter() - t0


def sample_kv_bytes(sample: dict, w: Workload) -> int:
    return int(sample["context_lens"].to(torch.int64).sum()) * w.spec["kv_heads"] * w.spec["head_size"] * 2 * w.elt


# ----------------------------------------------------------------------------------- main
def measured_hbm_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


def describe_config(a, spec: dict, variant: str, world: int, ctx) -> dict:
    """The `config` object of the JSON line; identical for the two --impl arms."""
    by_heads = getattr(a, "shard", "") == "heads" and world > 1
    strong = a.config == "c5" or by_heads
    fp8 = spec["kv"] != "float16"
    elt = 1 if fp8 else 2
    bs = spec["block_size"]
    blocks = sum((int(c) + bs - 1) // bs for c in ctx.tolist())
    cache_bytes = 2 * max(1, blocks) * bs * spec["kv_heads"] * spec["head_size"] * elt
    copies = 1 if cache_bytes >= 4 * L2_BYTES else min(50, math.ceil(4 * L2_BYTES / cache_bytes))
    forced = spec.get("cache_copies")
    if forced:
        copies = int(forced)
    kv_bytes = int(ctx.to(torch.int64).sum()) * spec["kv_heads"] * spec["head_size"] * 2 * elt
    return {
        "workload": f"BASELINE config {a.config[1]}: {variant} variant, KV {spec['kv']}, "
                    f"num_seqs={spec['num_seqs']}{' per GPU' if not strong and world > 1 else ''}, "
                    f"heads={spec['heads']}/{spec['kv_heads']}, head_size={spec['head_size']}, "
                    f"block_size={spec['block_size']}, ctx={spec['ctx']}",
        "entry_point": (f"launch_kernels_{'fp8_' if fp8 else ''}{variant}" if variant != "auto" else
                        f"launch_kernels_{'fp8_' if fp8 else ''}loop + launch_kernels_{'fp8_' if fp8 else ''}reduce, "
                        "chosen per sequence (serving.paged_attention_auto)"),
        "kv_bytes_per_call_per_gpu": kv_bytes, "cache_copies_rotated": copies,
        "l2_policy": (f"DIAGNOSTIC: {copies} cache copies forced, inputs may stay in L2" if forced else
                      "inputs larger than L2" if copies == 1 else
                      f"rotating over {copies} cache copies (> 4x L2 in total)"),
        "block_order": spec.get("block_order", "random"),
        "launch": "cuda graph replay" if getattr(a, "cuda_graph", False) else "direct",
        "sharding": "none" if world == 1 else
                    ("KV heads split evenly over the GPUs (heads shown are per GPU)" if by_heads else
                     ("sequences dealt longest-first to the lightest GPU" if getattr(a, "shard", "") == "lpt"
                      else "sequences split by cumulative KV length") if strong else "one shard per GPU"),
    }


def pick_variant(spec: dict) -> str:
    return spec["variant"]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4", "c5", "kvwrite"],
                    help="c1..c5: BASELINE configs of the attention path; kvwrite: the cache-append kernel")
    ap.add_argument("--variant", default=None, choices=["loop", "reduce", "auto"],
                    help="override the entry point the configuration names")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fp8-scale", type=float, default=0.05, help="kvwrite: per-tensor scale of the cache")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="record one call per rotated cache copy into CUDA graphs and replay them "
                         "in the device-resident timing loop (hides launch latency of tiny batches)")
    ap.add_argument("--kv", default=None, choices=["float16", "float8_e5m2", "float8_e4m3fn"],
                    help="override the KV cache type of the configuration")
    ap.add_argument("--head-size", type=int, default=None, choices=[64, 128])
    ap.add_argument("--heads", type=int, default=None, help="override the number of query heads")
    ap.add_argument("--kv-heads", type=int, default=None, help="override the number of KV heads")
    ap.add_argument("--block-size", type=int, default=None, choices=[16, 32, 64, 128])
    ap.add_argument("--e2e-mode", default="direct", choices=["torch", "step", "direct"],
                    help="end-to-end leg: torch copies + enqueue, one pa_decode_step_host call per step, "
                         "or the same with the kernels writing the result into pinned host memory")
    ap.add_argument("--shard", default="contiguous", choices=["contiguous", "lpt", "heads"],
                    help="several GPUs: config c5 is split by sequence, in contiguous ranges balanced on "
                         "cumulative KV length (default) or longest-first to the lightest GPU (lpt); "
                         "'heads' splits any config by KV head instead (few very long sequences): every "
                         "GPU holds num_kv_heads / N heads of all sequences")
    ap.add_argument("--cache-copies", type=int, default=None,
                    help="diagnostic: number of KV-cache copies the steps rotate over (1 with a small cache "
                         "measures the kernel fed from L2, not an HBM figure)")
    ap.add_argument("--block-order", default=None, choices=["random", "sequential"],
                    help="physical placement of a sequence's blocks (default: a random permutation)")
    ap.add_argument("--num-seqs", type=int, default=None,
                    help="override the number of sequences (small cases for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.config == "kvwrite":
        if rank == 0:
            bench_cache_write(a)
        return
    spec = config_spec(a.config)
    if a.num_seqs is not None:
        spec["num_seqs"] = a.num_seqs
    if a.kv is not None:
        spec["kv"] = a.kv
    for key, val in (("head_size", a.head_size), ("heads", a.heads), ("kv_heads", a.kv_heads),
                     ("block_size", a.block_size)):
        if val is not None:
            spec[key] = val
    if a.block_order is not None:
        spec["block_order"] = a.block_order
    if a.cache_copies is not None:
        spec["cache_copies"] = a.cache_copies
    overridden = any(v is not None for v in (a.num_seqs, a.kv, a.head_size, a.heads, a.kv_heads, a.block_size, a.block_order, a.cache_copies))
    variant = a.variant or pick_variant(spec)

    if a.impl == "reference":
        if rank != 0:
            return
        run_reference_arm(a, spec, variant, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group(backend="nccl", device_id=device)

    ctx_all = draw_context_lens(spec, seed=int(a.config[1]))
    by_heads = a.shard == "heads" and world > 1
    if by_heads:
        from flash_attention_factory_b200.sharding import shard_kv_heads

        lo, hi = shard_kv_heads(spec["kv_heads"], world)[rank]
        if (hi - lo) * world != spec["kv_heads"]:
            raise SystemExit("--shard heads needs num_kv_heads divisible by the number of GPUs")
        group = spec["heads"] // spec["kv_heads"]
        spec["kv_heads"], spec["heads"] = hi - lo, (hi - lo) * group  # this rank's slice of both caches
    strong = a.config == "c5" or by_heads
    ctx = shard_by_kv_length(ctx_all, world, rank, a.shard) if (a.config == "c5" and world > 1 and not by_heads) else ctx_all
    w = Workload(spec, ctx, device, seed=1000 * int(a.config[1]) + rank, variant=variant)

    def sync_all():
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(device)

    # ---- device-resident throughput: K asynchronous calls between two events
    for i in range(a.warmup):
        w.enqueue(i)
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    graphs = None
    if a.cuda_graph:
        graphs = []
        side = torch.cuda.Stream(device)
        for i in range(w.copies):
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(gph, stream=side):
                    w.enqueue(i)
            graphs.append(gph)
        for gph in graphs[:3]:
            gph.replay()
        sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        if graphs is not None:
            graphs[i % w.copies].replay()
        else:
            w.enqueue(i)
    e1.record()
    sync_all()
    ms_total = e0.elapsed_time(e1)

    # ---- per-kernel durations (blocking form: events around each kernel)
    attn_us, merge_us = [], []
    if variant == "auto":
        attn_us = [ms_total / a.steps * 1e3]  # two kernels on two streams: the call is the unit
    else:
        for i in range(min(a.steps, 30)):
            t = w.module().run(*w.args(i))
            attn_us.append(t[0])
            if len(t) > 1:
                merge_us.append(t[1])

    # ---- end to end: host buffers in, host buffer out, every step
    from flash_attention_factory_b200.host_io import DecodeStepIO

    io = DecodeStepIO(w.num_seqs, spec["heads"], spec["head_size"], w.bt.size(1), device)
    io.query_host.copy_(w.q_host)
    io.block_tables_host.copy_(w.bt_host)
    io.context_lens_host.copy_(w.ctx_host)
    out_resident = w.out
    w.out = io.out  # the step writes into the buffer that is downloaded

    bound = None
    if variant != "auto" and a.e2e_mode != "torch":
        # one library call per step: upload, launch, download, wait (pa_decode_step_host)
        bound = [io.bind(w.module().ENTRY, w.module().params(*w.args(i, io.query, io.block_tables, io.context_lens)),
                         direct_out=(a.e2e_mode == "direct")) for i in range(w.copies)]

    def e2e_step(i):
        if bound is not None:
            bound[i % w.copies].run()
            return
        io.upload()  # query + block tables + context lengths: one copy from pinned memory
        w.enqueue(i, io.query, io.block_tables, io.context_lens)
        io.download()  # the caller reads the result now

    for i in range(3):
        e2e_step(i)
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(a.steps):
        e2e_step(i)
    e3.record()
    sync_all()
    ms_e2e = e2.elapsed_time(e3)
    w.out = out_resident
    w.h2d_bytes, w.d2h_bytes = io.h2d_bytes, io.d2h_bytes
    clocks = sampler.stop() if rank == 0 else None

    import flash_attention_factory_b200 as pkg

    pkg.device_status()

    # ---- read rate of a kernel that only reads, same pools, one launch, this GPU, this run
    read_gbs, bulk_gbs, read_bytes = None, None, 0
    if rank == 0:
        from flash_attention_factory_b200 import _test_aids as _cabi

        kp, vp = w.k[0], w.v[0]
        read_bytes = (kp.numel() + vp.numel()) * kp.element_size()
        if read_bytes >= 4 * L2_BYTES:  # several times L2, else the figure is not an HBM figure
            cur = torch.cuda.current_stream(device).cuda_stream
            read_gbs = _cabi.measure_read_bandwidth(kp.data_ptr(), read_bytes // 2, 10, cur,
                                                    vp.data_ptr(), read_bytes // 2, method=0)
            bulk_gbs = _cabi.measure_read_bandwidth(kp.data_ptr(), read_bytes // 2, 10, cur,
                                                    vp.data_ptr(), read_bytes // 2, method=1)

    # ---- max over ranks, whole-job aggregate
    stats = torch.tensor([ms_total, ms_e2e, statistics.mean(attn_us)], dtype=torch.float64, device=device)
    total_bytes = torch.tensor([float(w.kv_bytes)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    ms_total, ms_e2e, attn_mean_us = [float(x) for x in stats.tolist()]
    job_bytes = float(total_bytes.item())
    ms_per_step = ms_total / a.steps
    value = job_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = job_bytes / (ms_e2e / a.steps * 1e-3) / 1e9

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        achieved = w.kv_bytes / (attn_mean_us * 1e-6) / 1e9
        line = {
            "metric": "decode_attention_kv_GBps", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_per_step, 5),
            "us_per_call": round(ms_per_step * 1e3, 2), "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 x f16 -> f32 (mma.sync), KV stored as " + spec["kv"], "data": "synthetic",
            "config": describe_config(a, spec, variant, world, ctx_all),
            "pct_of_8TBps": round(100 * value / (NOMINAL_HBM_GBS * world), 2),
            "roofline": {"bound": "hbm", "kernel": "paged_attention_kernel",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                         "frac_of_8TBps": round(achieved / NOMINAL_HBM_GBS, 4),
                         "read_only_stream_gbs": round(read_gbs, 1) if read_gbs else None,
                         "read_only_bulk_copy_gbs": round(bulk_gbs, 1) if bulk_gbs else None,
                         "read_only_stream_bytes": read_bytes if read_gbs else None,
                         "frac_of_read_only_stream": round(achieved / max(read_gbs, bulk_gbs), 4) if read_gbs else None,
                         "kernel_us": round(attn_mean_us, 2),
                         "merge_kernel_us": round(statistics.mean(merge_us), 2) if merge_us else None,
                         "traffic": TRAFFIC_BYTES.get((a.config, variant)) if not overridden else None},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": w.h2d_bytes,
                    "d2h_bytes_per_step": w.d2h_bytes, "us_per_call": round(ms_e2e / a.steps * 1e3, 2)},
            "gpu_launches": a.steps * w.launches_per_step,
            "clocks": clocks,
        }
        if not a.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one attention-kernel launch, from the ncu
# captures summarised under profiles/ (None until a capture exists for the workload)
TRAFFIC_BYTES: dict = {
    # profiles/paged_attention_kernel_split_fp16_c2_small.md: 4 x (1073.96 + 3.82) MB
    ("c2", "reduce"): 4_311_100_000,
    # profiles/paged_attention_kernel_split_e4m3_c4_small.md: 2 x (537.13 + 5.65) MB
    ("c4", "reduce"): 1_085_600_000,
}


def bench_cache_write(a) -> None:
    """`--config kvwrite`: pa_reshape_and_cache on 64k new tokens of a Llama-3-8B-shaped cache
    (8 KV heads x 128, block 16), fp16 input -> e4m3 cache.  HBM-bound: per token it reads
    2 x 2 KB of fp16 K/V and writes 2 x 1 KB of FP8."""
    from flash_attention_factory_b200.cache_ops import reshape_and_cache

    dev = torch.device("cuda", 0)
    tokens, hk, d, bs = 65536, 8, 128, 16
    kv = a.kv or "float8_e4m3fn"
    dt = {"float16": torch.float16, "float8_e5m2": torch.float8_e5m2, "float8_e4m3fn": torch.float8_e4m3fn}[kv]
    g = torch.Generator(device=dev).manual_seed(0)
    key = torch.randn(tokens, hk, d, generator=g, device=dev, dtype=torch.float16)
    value = torch.randn(tokens, hk, d, generator=g, device=dev, dtype=torch.float16)
    nb = 2 * tokens // bs
    kc = torch.zeros(nb, bs, hk, d, device=dev, dtype=torch.float16).to(dt)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * bs, generator=g, device=dev)[:tokens].to(torch.int64)
    elt = 2 if kv == "float16" else 1
    nbytes = tokens * hk * d * (2 * 2 + 2 * elt)
    for _ in range(max(3, a.warmup)):
        reshape_and_cache(key, value, kc, vc, slots, a.fp8_scale)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        reshape_and_cache(key, value, kc, vc, slots, a.fp8_scale)
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / a.steps
    peak, kind = measured_hbm_peak()
    val = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "kv_cache_write_GBps", "value": round(val, 1), "unit": "GB/s", "n_gpus": 1,
        "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": round(ms, 5), "higher_is_better": True,
        "dtype": f"fp16 -> {kv}", "data": "synthetic",
        "config": {"workload": f"pa_reshape_and_cache: {tokens} tokens, {hk} KV heads x {d}, block {bs}, "
                               f"random slots, cache {kv}; {nbytes} bytes moved per call (402 MB, larger than L2)"},
        "roofline": {"bound": "hbm", "kernel": "reshape_and_cache_kernel", "achieved": round(val, 1),
                     "peak": peak, "unit": "GB/s", "frac": round(val / peak, 4), "peak_kind": f"of {kind}",
                     "traffic": None},
        "gpu_launches": a.steps}), flush=True)


def cpu_baseline(w: Workload) -> dict:
    """Times the CPU oracle on a sample sized for roughly 10-30 s of host work."""
    probe = cpu_sample_inputs(w, 1)
    t1 = time_cpu_oracle(probe)
    n = max(1, min(w.num_seqs, int(15.0 / max(t1, 1e-3))))
    sample = cpu_sample_inputs(w, n)
    t = time_cpu_oracle(sample)
    reps = 1 + max(0, min(20, int(10.0 / max(t, 1e-3)) - 1))
    for _ in range(reps - 1):
        t += time_cpu_oracle(sample)
    return {"value": round(reps * sample_kv_bytes(sample, w) / t / 1e9, 4), "unit": "GB/s",
            "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(), "kind": "port",
            "seconds": round(t, 2),
            "sample": f"first {n} of {w.num_seqs} sequences of the workload, {reps} passes, CPU oracle "
                      f"(torch fp32, {torch.get_num_threads()} threads)"}


def run_reference_arm(a, spec: dict, variant: str, world: int) -> None:
    """`--impl reference`: the reference's CPU algorithm (oracle port) on the host cores.

    The reference's GPU kernels are Intel SYCL/ESIMD and cannot be built for this machine; its
    CPU implementation of the path is the torch code of its tests, restated in oracle/.  Every
    step runs the oracle on a bounded sample of the configured workload."""
    ctx = draw_context_lens(spec, seed=int(a.config[1]))
    d, bs, hk, h = spec["head_size"], spec["block_size"], spec["kv_heads"], spec["heads"]
    elt = 1 if spec["kv"] != "float16" else 2
    g = torch.Generator().manual_seed(7)

    def build(n):
        c = ctx[:n]
        nbs = [(int(x) + bs - 1) // bs for x in c.tolist()]
        nb, mb = sum(nbs), max(nbs)
        k = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16)
        v = torch.randn(nb, bs, hk, d, generator=g).to(torch.float16)
        scale = 1.0
        if spec["kv"] == "float8_e5m2":
            k, v = k.to(torch.float8_e5m2), v.to(torch.float8_e5m2)
        elif spec["kv"] == "float8_e4m3fn":
            scale = float(max(k.abs().max(), v.abs().max())) / 448.0
            k, v = (k.float() / scale).to(torch.float8_e4m3fn), (v.float() / scale).to(torch.float8_e4m3fn)
        perm = torch.randperm(nb, generator=g).to(torch.int32)
        bt = torch.zeros(n, mb, dtype=torch.int32)
        pos = 0
        for i, x in enumerate(nbs):
            bt[i, :x] = perm[pos:pos + x]
            pos += x
        q = torch.randn(n, h, d, generator=g).to(torch.float16)
        return dict(query=q, key_cache=k, value_cache=v, block_tables=bt, context_lens=c,
                    sm_scale=1.0 / math.sqrt(d), fp8_scale=scale)

    probe = build(1)
    t1 = time_cpu_oracle(probe)
    budget = 150.0 / (a.steps + a.warmup)
    n = max(1, min(spec["num_seqs"], int(budget / max(t1, 1e-3))))
    sample = build(n)
    nbytes = int(sample["context_lens"].to(torch.int64).sum()) * hk * d * 2 * elt
    for _ in range(a.warmup):
        time_cpu_oracle(sample)
    t0 = time.perf_counter()
    for _ in range(a.steps):
        time_cpu_oracle(sample)
    dt = (time.perf_counter() - t0) / a.steps
    value = nbytes / dt / 1e9
    desc = (f"{n} of {spec['num_seqs']} sequences of the workload per step, CPU oracle "
            f"(torch fp32, {torch.get_num_threads()} threads)")
    print(json.dumps({
        "impl": "reference", "metric": "decode_attention_kv_GBps", "value": round(value, 4), "unit": "GB/s",
        "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (CPU)",
        "data": "synthetic",
        "config": describe_config(a, spec, variant, world, ctx),
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


if __name__ == "__main__":
    main()
