"""Benchmark of the paged-attention decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c5] [--impl ours|reference]

A call is one invocation of the operator over one batch; a step is `calls_per_step` calls back
to back, chosen so that the K timed steps last at least `--min-seconds` (default 1 s): a
decode call takes 0.1-1 ms, and a timed region of a few milliseconds measures a GPU that has
barely left its idle clocks.

The default workload, at every N, is BASELINE.json's configs[4] ("c5": 1024 sequences with
log-normal context lengths, FP8 e5m2 KV cache, 32 query / 8 KV heads): the largest single-GPU
configuration and the one the path shards by sequence.  With N>1 (torchrun, one rank per GPU)
the one batch is split over the ranks (strong scaling, no data-path collective) and each rank
holds its own shard's KV pool; `--config c1..c4` select the other BASELINE configurations (one
copy per rank: weak scaling), `--config refperf16|refperf8` the two shapes the reference's own
perf mode times (test_paged.py:607-631, test_paged_fp8cache.py:612-636).

Rank 0 prints ONE JSON line.  `value` is KV bytes / time with all inputs resident in HBM; `e2e`
is the same metric through the library's host-buffer call (`pa_decode_step_host_batch`): every
step uploads the step's inputs (query, packed block tables, context lengths) from pinned host
memory and delivers the result to pinned host memory inside the timed region.  The KV cache is
state of the serving process, like weights, and stays resident.  At N=1 `roofline.variants`
holds the same measurement for each of the four entry points on the long-context FP8 GQA shape
(c4) and for c3, c2, c1 and the reference's perf shapes; at N>1 it holds the c4 batch split by
KV head and by sequence.  `roofline.errors` compares outputs of the timed workloads with the CPU
oracle on a sample of sequences.  `--impl reference` times the CPU oracle (the reference's own
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
    """Shapes of BASELINE.json's configs (head_size 128, block_size 16) and of the reference's perf mode."""
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
    # the two shapes the reference's perf mode times (test_paged.py:607-631,
    # test_paged_fp8cache.py:612-636): head 64, block 64, ctx 1500, sinks, groups 8 and 5
    ref = dict(variant="loop", num_seqs=64, kv_heads=8, ctx=("const", 1500), head_size=64, block_size=64, sinks=True)
    specs["refperf16"] = dict(ref, kv="float16", heads=64)
    specs["refperf8"] = dict(ref, kv="float8_e5m2", heads=40)
    # many short sequences (no BASELINE counterpart): the batch shape of short-prompt serving, where the
    # loop variant runs its persistent form (one work item per sequence and head group)
    specs["short"] = dict(variant="loop", kv="float8_e5m2", num_seqs=4096, heads=32, kv_heads=8,
                          ctx=("uniform", 64, 512))
    s = dict(head_size=128, block_size=16, sinks=False)
    s.update(specs[name])
    s["name"] = name
    return s


CONFIG_SEEDS = {"c1": 1, "c2": 2, "c3": 3, "c4": 4, "c5": 5, "refperf16": 6, "refperf8": 7, "short": 8}
CONFIG_TITLES = {"c1": "BASELINE config 1", "c2": "BASELINE config 2", "c3": "BASELINE config 3",
                 "c4": "BASELINE config 4", "c5": "BASELINE config 5",
                 "refperf16": "reference perf-mode shape (fp16)", "refperf8": "reference perf-mode shape (fp8)",
                 "short": "4096 sequences of 64..512 tokens (no BASELINE counterpart)"}


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
        self.sinks_host = (torch.randn(h, generator=gc) * 2 + 3).to(torch.float16) if spec.get("sinks") else None
        self.sinks = self.sinks_host.to(device) if self.sinks_host is not None else None
        self.sm_scale = 1.0 / math.sqrt(d)
        self.group = h // hk
        self.kv_bytes = int(ctx.to(torch.int64).sum()) * hk * d * 2 * self.elt
        self.h2d_bytes = self.q_host.numel() * 2 + self.bt_host.numel() * 4 + self.ctx_host.numel() * 4
        self.d2h_bytes = self.out_host.numel() * 2

    def module(self):
        from flash_attention_factory_b200 import lib

        return getattr(lib, f"paged_attention_{'fp8_' if self.fp8 else ''}{self.entry_variant()}")

    def auto_plan(self):
        from flash_attention_factory_b200.serving import AutoDecodePlan

        if getattr(self, "plan", None) is None:
            self.plan = AutoDecodePlan(self.ctx.tolist(), self.spec["heads"], self.spec["head_size"],
                                       self.spec["block_size"], self.bt.size(1), self.device)
        return self.plan

    def entry_variant(self) -> str:
        """The single entry point a step goes through; for "auto" the one the selector folds the
        whole batch into (None if the batch is launched as a loop and a reduce part)."""
        if self.variant != "auto":
            return self.variant
        plan = self.auto_plan()
        if plan.loop is not None and plan.reduce is not None:
            return None
        return "reduce" if plan.reduce is not None else "loop"

    def args(self, step: int, q=None, bt=None, cl=None):
        i = step % self.copies
        a = [self.max_logits, self.exp_sums, self.tmp_out, self.out, self.debug,
             self.q if q is None else q, self.k[i], self.v[i], self.bt if bt is None else bt,
             self.cl if cl is None else cl, self.group, self.sm_scale]
        if self.fp8:
            a.append(self.fp8_scale)
        a += [self.spec["block_size"], self.max_ctx, self.alibi, self.sinks, -1.0]
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
        from flash_attention_factory_b200.serving import paged_attention_auto

        i = step % self.copies
        paged_attention_auto(self.auto_plan(), self.out, self.q if q is None else q, self.k[i], self.v[i],
                             self.bt if bt is None else bt, self.cl if cl is None else cl, self.group,
                             self.sm_scale, self.fp8_scale, self.sinks)

    @property
    def launches_per_step(self) -> int:
        if self.variant == "auto":
            plan = self.auto_plan()
            return (1 if plan.loop is not None else 0) + (2 if plan.reduce is not None else 0)
        return 2 if self.variant == "reduce" else 1

    def free(self) -> None:
        """Drops the device tensors (the variants table builds one workload after another)."""
        for name in ("k", "v", "q", "bt", "cl", "max_logits", "exp_sums", "tmp_out", "out", "plan", "_params"):
            self.__dict__.pop(name, None)
        torch.cuda.empty_cache()


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
def cpu_sample_inputs(w: Workload, n_seq, copy: int = 0):
    """A bounded sample of the rank's workload for the CPU oracle: the first n_seq sequences (or
    the sequences of an index list) with their blocks compacted into a small cache (block ids
    renumbered)."""
    picks = list(range(min(n_seq, w.num_seqs))) if isinstance(n_seq, int) else list(n_seq)
    bs = w.spec["block_size"]
    rows, tables, pos = [], [], 0
    mb = w.bt.shape[1]
    for i in picks:
        nb = (int(w.ctx[i]) + bs - 1) // bs
        rows.append(w.bt_host[i, :nb].long())
        t = torch.zeros(mb, dtype=torch.int32)
        t[:nb] = torch.arange(pos, pos + nb, dtype=torch.int32)
        tables.append(t)
        pos += nb
    idx = torch.cat(rows).to(w.device)
    k = w.k[copy][idx].cpu()
    v = w.v[copy][idx].cpu()
    sel = torch.tensor(picks, dtype=torch.long)
    return dict(query=w.q_host[sel].clone(), key_cache=k, value_cache=v,
                block_tables=torch.stack(tables), context_lens=w.ctx[sel].clone(),
                sm_scale=w.sm_scale, fp8_scale=w.fp8_scale, sinks=w.sinks_host)


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
                               fp8_scale=sample["fp8_scale"], sinks=sample.get("sinks"))
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


def describe_config(a, spec: dict, variant: str, world: int, ctx, shard: str) -> dict:
    """The `config` object of the JSON line; identical for the two --impl arms."""
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
    sharding = {"none": "none", "replicas": "one copy of the batch per GPU",
                "heads": "KV heads split evenly over the GPUs",
                "lpt": "sequences dealt longest-first to the lightest GPU",
                "contiguous": "consecutive sequences with equal shares of the KV tokens per GPU"}[shard]
    return {
        "workload": f"{CONFIG_TITLES[spec['name']]}: {variant} variant, KV {spec['kv']}, "
                    f"num_seqs={spec['num_seqs']}{' per GPU' if shard == 'replicas' else ''}, "
                    f"heads={spec['heads']}/{spec['kv_heads']}, head_size={spec['head_size']}, "
                    f"block_size={spec['block_size']}, ctx={spec['ctx']}",
        "entry_point": (f"launch_kernels_{'fp8_' if fp8 else ''}{variant}" if variant != "auto" else
                        f"launch_kernels_{'fp8_' if fp8 else ''}loop / launch_kernels_{'fp8_' if fp8 else ''}reduce, "
                        "chosen per sequence (serving.paged_attention_auto; short sequences that hold under a "
                        "quarter of the tokens are folded into the reduce launch)"),
        "kv_bytes_per_call": kv_bytes, "cache_copies_rotated": copies,
        "l2_policy": (f"DIAGNOSTIC: {copies} cache copies forced, inputs may stay in L2" if forced else
                      "inputs larger than L2" if copies == 1 else
                      f"rotating over {copies} cache copies (> 4x L2 in total)"),
        "block_order": spec.get("block_order", "random"),
        "launch": "cuda graph replay" if getattr(a, "cuda_graph", False) else "direct",
        "sharding": sharding,
    }


class Group:
    """The ranks of the run: barrier, max and sum over ranks (a single rank is its own group)."""

    def __init__(self, dist, device):
        self.dist, self.device = dist, device

    def sync(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize(self.device)

    def _reduce(self, values, op):
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        if self.dist is not None:
            self.dist.all_reduce(t, op=op)
        return [float(x) for x in t.tolist()]

    def max(self, *values):
        return self._reduce(values, self.dist.ReduceOp.MAX if self.dist is not None else None)

    def sum(self, *values):
        return self._reduce(values, self.dist.ReduceOp.SUM if self.dist is not None else None)


def timed_calls(call, steps: int, warmup: int, min_seconds: float, group: Group):
    """W warm-up calls, then `steps` steps of `calls_per_step` calls between two CUDA events on
    the launching stream, a barrier and a device synchronisation on both sides.  The number of
    calls per step is chosen from a short probe so that the timed region lasts `min_seconds`,
    the same on every rank.  Returns (milliseconds of the timed region, calls_per_step)."""
    for i in range(warmup):
        call(i)
    group.sync()
    probe = 4
    t0 = time.perf_counter()
    for i in range(probe):
        call(i)
    torch.cuda.synchronize()
    per_call = (time.perf_counter() - t0) / probe
    per_call = group.max(per_call)[0]
    cps = max(1, math.ceil(min_seconds / max(per_call * steps, 1e-9)))
    group.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n = 0
    for _ in range(steps):
        for _ in range(cps):
            call(n)
            n += 1
    e1.record()
    group.sync()
    return e0.elapsed_time(e1), cps


def timed_launches_from_c(w: Workload, steps: int, warmup: int, min_seconds: float, group: Group):
    """The same protocol as timed_calls with the calls issued from C (`pa_aid_time_launches`): what
    a C or C++ host of the library sees.  A Python loop adds several microseconds of interpreter
    time per call, which hides the kernels of small batches.  One argument block per rotated
    cache copy, built and checked once."""
    from flash_attention_factory_b200 import _test_aids

    keep = w.variant
    w.variant = w.entry_variant()
    entry = w.module().ENTRY
    blocks = [w.module().params(*w.args(i)) for i in range(w.copies)]
    w.variant = keep
    stream = torch.cuda.current_stream(w.device).cuda_stream
    _test_aids.time_launches(entry, blocks, max(warmup, 3), stream)
    group.sync()
    per_call = _test_aids.time_launches(entry, blocks, 8, stream) * 1e-6
    per_call = group.max(per_call)[0]
    cps = max(1, math.ceil(min_seconds / max(per_call * steps, 1e-9)))
    group.sync()
    us = _test_aids.time_launches(entry, blocks, steps * cps, stream)
    group.sync()
    return us * steps * cps / 1e3, cps


def e2e_binding(w: Workload):
    """The host-buffer step of the workload: pinned inputs (query, packed block tables, context
    lengths) and a pinned result, one `pa_decode_step_host_batch` call per step.  Returns
    (io, list of bound steps, one per rotated cache copy) or None when the batch is launched as
    two parts (strict per-sequence selection), which goes through torch copies instead."""
    from flash_attention_factory_b200.host_io import DecodeBatchIO

    variant = w.entry_variant()
    if variant is None:
        return None
    spec = w.spec
    bs = spec["block_size"]
    cap = sum((int(c) + bs - 1) // bs for c in w.ctx.tolist()) + 8
    io = DecodeBatchIO(w.num_seqs, spec["heads"], spec["head_size"], w.bt.size(1), w.device, packed_capacity=cap)
    io.query_host.copy_(w.q_host)
    io.context_lens_host.copy_(w.ctx_host)
    io.set_block_tables(w.bt_host, w.ctx_host, bs)
    keep = (w.out, w.variant)
    w.out, w.variant = io.out, variant
    # the merge kernel writes whole rows, so the last sub-batch's result can go straight to the
    # host; the loop kernel's epilogue writes scattered halves and is better served by a copy
    steps = [io.bind(w.module().ENTRY, w.module().params(*w.args(i, io.query, w.bt, io.context_lens)),
                     last_out_direct=(variant == "reduce")) for i in range(w.copies)]
    w.out, w.variant = keep
    return io, steps


def check_errors(w: Workload, max_seqs: int = 6, e2e=None) -> dict:
    """Outputs of the timed workload against the CPU oracle, on a sample of its sequences: the
    shortest, the longest, the one nearest to a partition boundary and a few drawn at random.
    Tolerance: atol 1e-3, rtol 1e-2 (BASELINE.json's north_star).  The oracle is the checker
    here, after the timed regions; nothing timed touches it."""
    from oracle import paged_attention_oracle as oracle

    lens = w.ctx.tolist()
    if not lens:
        return {"checked_seqs": 0, "within_tol": True, "max_abs": 0.0, "max_rel": 0.0}
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    psize = 512 if w.spec["head_size"] == 128 else 256
    near = min(range(len(lens)), key=lambda i: (min(lens[i] % psize, psize - lens[i] % psize), i))
    rnd = torch.randperm(len(lens), generator=torch.Generator().manual_seed(11)).tolist()
    picks = []
    for i in [order[0], order[-1], near] + rnd:
        if i not in picks:
            picks.append(i)
        if len(picks) >= max_seqs:
            break
    w.out.fill_(float("nan"))
    w.enqueue(0)
    torch.cuda.synchronize(w.device)
    got = w.out[torch.tensor(picks, device=w.device)].float().cpu()
    sample = cpu_sample_inputs(w, picks, copy=0)
    want = oracle.paged_attention_ref(sample["query"], sample["key_cache"], sample["value_cache"],
                                      sample["block_tables"], sample["context_lens"], sm_scale=sample["sm_scale"],
                                      fp8_scale=sample["fp8_scale"], sinks=sample.get("sinks")).float()
    err = (got - want).abs()
    ok = bool(torch.isfinite(got).all()) and bool((err <= 1e-3 + 1e-2 * want.abs()).all())
    res = {"checked_seqs": len(picks), "checked_ctx": [lens[i] for i in picks], "within_tol": ok,
           "max_abs": float(err.max()), "max_rel": float((err / want.abs().clamp_min(1e-2)).max()),
           "atol": 1e-3, "rtol": 1e-2}
    if e2e is not None:
        io, steps = e2e
        io.out_host.fill_(float("nan"))
        host = steps[0].run().clone()
        same = torch.equal(host, w.out.cpu()) if w.entry_variant() == "reduce" else None
        herr = (host[torch.tensor(picks)].float() - want).abs()
        res["e2e_within_tol"] = bool(torch.isfinite(host).all()) and bool((herr <= 1e-3 + 1e-2 * want.abs()).all())
        res["e2e_bits_equal_resident"] = same
    return res


def measure_workload(w: Workload, a, group: Group, min_seconds: float, e2e_seconds: float, with_errors: bool,
                     kernel_reps: int = 20, graph: bool = False, error_seqs: int = 6, sampler=None) -> dict:
    """Times one workload on this rank (and, through `group`, on all ranks): device-resident
    calls, the attention kernel alone, and the host-buffer step."""
    graphs = None
    if graph:
        graphs = []
        side = torch.cuda.Stream(w.device)
        for i in range(w.copies):
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(gph, stream=side):
                    w.enqueue(i)
            graphs.append(gph)

    def call(i):
        if graphs is not None:
            graphs[i % w.copies].replay()
        else:
            w.enqueue(i)

    if graphs is None and w.entry_variant() is not None:
        ms_total, cps = timed_launches_from_c(w, a.steps, a.warmup, min_seconds, group)
    else:
        ms_total, cps = timed_calls(call, a.steps, a.warmup, min_seconds, group)
    # ---- per-kernel durations (blocking form of the entry point: events around each kernel)
    attn_us, merge_us = [], []
    if w.entry_variant() is not None:
        keep = w.variant
        w.variant = w.entry_variant()
        for i in range(kernel_reps):
            t = w.module().run(*w.args(i))
            attn_us.append(t[0])
            if len(t) > 1:
                merge_us.append(t[1])
        w.variant = keep
    # ---- end to end: host buffers in, host buffer out, every call
    e2e = e2e_binding(w)
    if e2e is not None:
        io, bound = e2e
        plan = bound[0].plan()

        def e2e_call(i):
            bound[i % w.copies].run()
    else:
        from flash_attention_factory_b200.host_io import DecodeStepIO

        sio = DecodeStepIO(w.num_seqs, w.spec["heads"], w.spec["head_size"], w.bt.size(1), w.device)
        sio.query_host.copy_(w.q_host)
        sio.block_tables_host.copy_(w.bt_host)
        sio.context_lens_host.copy_(w.ctx_host)
        plan = {"sub_batches": 1, "h2d_bytes": sio.h2d_bytes, "d2h_bytes": sio.d2h_bytes}
        resident_out = w.out

        def e2e_call(i):
            w.out = sio.out
            sio.upload()
            w.enqueue(i, sio.query, sio.block_tables, sio.context_lens)
            sio.download()
            w.out = resident_out

    ms_e2e, cps_e2e = timed_calls(e2e_call, a.steps, 3, e2e_seconds, group)
    clocks = sampler.stop() if sampler is not None else None  # the clock record covers the timed regions only
    errors = check_errors(w, max_seqs=error_seqs, e2e=e2e) if with_errors else None
    calls, calls_e2e = a.steps * cps, a.steps * cps_e2e
    kernel = statistics.mean(attn_us) if attn_us else ms_total / calls * 1e3
    ms_total, ms_e2e, kernel = group.max(ms_total, ms_e2e, kernel)
    (job_bytes,) = group.sum(float(w.kv_bytes))
    return {
        "ms_total": ms_total, "calls_per_step": cps, "us_per_call": ms_total / calls * 1e3,
        "gbs": job_bytes / (ms_total / calls * 1e-3) / 1e9, "job_bytes": job_bytes,
        "kernel_us": kernel, "kernel_gbs": w.kv_bytes / (kernel * 1e-6) / 1e9,
        "merge_us": statistics.mean(merge_us) if merge_us else None,
        "e2e_us_per_call": ms_e2e / calls_e2e * 1e3, "e2e_gbs": job_bytes / (ms_e2e / calls_e2e * 1e-3) / 1e9,
        "e2e_calls_per_step": cps_e2e, "e2e_plan": plan, "errors": errors, "clocks": clocks,
        "launches": calls * w.launches_per_step,
    }


def variant_row(m: dict, peak: float, world: int = 1) -> dict:
    row = {"us_per_call": round(m["us_per_call"], 2), "gbs": round(m["gbs"], 1),
           "frac": round(m["kernel_gbs"] / peak, 4), "frac_of_8TBps": round(m["gbs"] / (NOMINAL_HBM_GBS * world), 4),
           "kernel_us": round(m["kernel_us"], 2), "kernel_gbs": round(m["kernel_gbs"], 1),
           "merge_kernel_us": round(m["merge_us"], 2) if m["merge_us"] else None,
           "e2e_gbs": round(m["e2e_gbs"], 1), "e2e_us_per_call": round(m["e2e_us_per_call"], 2),
           "e2e_sub_batches": m["e2e_plan"]["sub_batches"], "timed_ms": round(m["ms_total"], 1)}
    if m["errors"] is not None:
        row["errors"] = {k: (round(v, 6) if isinstance(v, float) else v) for k, v in m["errors"].items()
                         if k != "checked_ctx"}
    return row


def timeline_report(w: Workload, calls: int) -> None:
    """`--timeline`: per-CTA time stamps of the attention kernel of the last of `calls` back-to-back
    calls, summarised: microseconds from the first CTA's entry to each event, over the CTAs."""
    import ctypes

    from flash_attention_factory_b200 import _cabi

    lib = _cabi.load_library()
    variant = w.entry_variant() or "reduce"
    reader = getattr(lib, f"pa_debug_timeline_{'fp8_' if w.fp8 else ''}{variant}")
    for i in range(max(3, calls)):
        w.enqueue(i)
    torch.cuda.synchronize(w.device)
    rows = 4096
    buf = (ctypes.c_ulonglong * (rows * 8))()
    _cabi.check(reader(buf, rows))
    t = torch.tensor(list(buf), dtype=torch.float64).view(rows, 8)
    t = t[t[:, 0] > 0]
    t = t[t[:, 5] >= t[:, 0]]  # rows of the last launch only
    newest = t[:, 0].max()
    t = t[t[:, 0] > newest - 5e6]
    t0 = t[:, 0].min()
    names = ["entry", "after_wait_for_previous_kernel", "first_copy_issued", "first_stage_complete",
             "last_stage_consumed", "exit", None, "cluster_met_for_merge"]
    print(f"{w.spec['name']} {variant}: {t.size(0)} CTAs, kernel span "
          f"{(t[:, 5].max() - t0) / 1e3:.1f} us, KV bytes {w.kv_bytes}")
    print(f"{'event (us after first entry)':34s} {'min':>8s} {'p10':>8s} {'median':>8s} {'p90':>8s} {'max':>8s}")
    for k, name in enumerate(names):
        if name is None:
            continue
        col = t[:, k]
        col = (col[col > 0] - t0) / 1e3
        if col.numel() == 0:
            continue
        q = torch.quantile(col, torch.tensor([0.0, 0.1, 0.5, 0.9, 1.0], dtype=torch.float64))
        print(f"{name:34s} " + " ".join(f"{x:8.1f}" for x in q.tolist()))
    end = (t[:, 5] - t0) / 1e3
    last = (t[:, 4] - t0) / 1e3
    span = float(end.max())
    for back in (5.0, 10.0, 20.0):
        idle = int((last < span - back).sum())
        print(f"CTAs that had consumed their last stage {back:.0f} us before the end: {idle} of {t.size(0)}")
    items = t[:, 6]
    for k in sorted(set(int(x) for x in items.tolist())):
        sel = items == k
        print(f"CTAs with {k} work items: {int(sel.sum())}, last stage consumed at median "
              f"{float(last[sel].median()):.1f} us (min {float(last[sel].min()):.1f}, max {float(last[sel].max()):.1f})")


# name -> (config, variant, KV type override)
VARIANT_TABLE = [
    ("c4_launch_kernels_fp8_reduce", "c4", "reduce", None),
    ("c4_launch_kernels_fp8_loop", "c4", "loop", None),
    ("c4_launch_kernels_reduce_f16kv", "c4", "reduce", "float16"),
    ("c4_launch_kernels_loop_f16kv", "c4", "loop", "float16"),
    ("c3_launch_kernels_fp8_loop", "c3", "loop", None),
    ("c3_launch_kernels_fp8_reduce", "c3", "reduce", None),
    ("c2_launch_kernels_reduce", "c2", "reduce", None),
    ("c1_launch_kernels_loop", "c1", "loop", None),
    ("refperf16_launch_kernels_loop", "refperf16", "loop", None),
    ("refperf16_launch_kernels_reduce", "refperf16", "reduce", None),
    ("refperf8_launch_kernels_fp8_loop", "refperf8", "loop", None),
    ("short_launch_kernels_fp8_loop", "short", "loop", None),
    ("short_launch_kernels_loop_f16kv", "short", "loop", "float16"),
]


def shard_spec_and_ctx(spec: dict, ctx_all: torch.Tensor, shard: str, world: int, rank: int):
    """This rank's part of one batch: (spec, context lengths, ids of its sequences)."""
    from flash_attention_factory_b200.sharding import shard_kv_heads, shard_sequences_by_kv_length, shard_sequences_lpt

    spec = dict(spec)
    if world == 1 or shard in ("none", "replicas"):
        return spec, ctx_all, None
    if shard == "heads":
        lo, hi = shard_kv_heads(spec["kv_heads"], world)[rank]
        if (hi - lo) * world != spec["kv_heads"]:
            raise SystemExit("--shard heads needs num_kv_heads divisible by the number of GPUs")
        group = spec["heads"] // spec["kv_heads"]
        spec["kv_heads"], spec["heads"] = hi - lo, (hi - lo) * group  # this rank's slice of both caches
        return spec, ctx_all, None
    if shard == "lpt":
        ids = shard_sequences_lpt(ctx_all.tolist(), world)[rank]
    else:
        lo, hi = shard_sequences_by_kv_length(ctx_all.tolist(), world)[rank]
        ids = list(range(lo, hi))
    return spec, ctx_all[torch.tensor(ids, dtype=torch.long)].clone(), ids


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c5",
                    choices=["c1", "c2", "c3", "c4", "c5", "refperf16", "refperf8", "short", "kvwrite"],
                    help="c1..c5: BASELINE configs of the attention path; refperf16 / refperf8: the shapes the "
                         "reference's perf mode times; short: 4096 sequences of 64..512 tokens; kvwrite: the "
                         "cache-append kernel")
    ap.add_argument("--variant", default=None, choices=["loop", "reduce", "auto"],
                    help="override the entry point the configuration names")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="least duration of the headline's timed region; calls_per_step follows from it")
    ap.add_argument("--no-variants", action="store_true", help="skip the roofline.variants table")
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
    ap.add_argument("--shard", default=None, choices=["contiguous", "lpt", "heads", "replicas"],
                    help="several GPUs: how the batch is divided.  Default: c5 is dealt by sequence, longest "
                         "first to the lightest GPU (lpt); the other configs run one copy per GPU (replicas). "
                         "'contiguous' cuts consecutive sequences with equal KV shares, 'heads' gives every GPU "
                         "num_kv_heads / N heads of all sequences (few very long sequences)")
    ap.add_argument("--cache-copies", type=int, default=None,
                    help="diagnostic: number of KV-cache copies the steps rotate over (1 with a small cache "
                         "measures the kernel fed from L2, not an HBM figure)")
    ap.add_argument("--block-order", default=None, choices=["random", "sequential"],
                    help="physical placement of a sequence's blocks (default: a random permutation)")
    ap.add_argument("--timeline", action="store_true",
                    help="measuring aid: run one call on the -DPA_TIMELINE build of the library "
                         "(python -m flash_attention_factory_b200.build --timeline) and print when the CTAs of "
                         "the attention kernel started, got their first data, finished and left")
    ap.add_argument("--num-seqs", type=int, default=None,
                    help="override the number of sequences (small cases for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if a.timeline:
        os.environ["PA_B200_LIBRARY_VARIANT"] = "timeline"

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
    overridden = any(v is not None for v in (a.num_seqs, a.kv, a.head_size, a.heads, a.kv_heads, a.block_size,
                                              a.block_order, a.cache_copies))
    variant = a.variant or spec["variant"]
    scheme = a.shard or ("lpt" if a.config == "c5" else "replicas")  # how the workload divides over GPUs
    shard = "none" if world == 1 else scheme
    a.strong = scheme in ("lpt", "contiguous", "heads")  # total work fixed as N grows (also said at N = 1)
    seed = CONFIG_SEEDS[a.config]

    if a.impl == "reference":
        if rank != 0:
            return
        run_reference_arm(a, spec, variant, world, shard)
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
    group = Group(dist, device)
    peak, peak_kind = measured_hbm_peak()

    ctx_all = draw_context_lens(spec, seed=seed)
    my_spec, ctx, _ = shard_spec_and_ctx(spec, ctx_all, shard, world, rank)
    w = Workload(my_spec, ctx, device, seed=1000 * seed + rank, variant=variant)

    if a.timeline:
        timeline_report(w, a.steps)
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    m = measure_workload(w, a, group, a.min_seconds, max(0.3, a.min_seconds / 2), with_errors=True,
                         graph=a.cuda_graph, sampler=sampler if rank == 0 else None)
    clocks = m["clocks"]

    import flash_attention_factory_b200 as pkg

    pkg.device_status()

    # ---- read rate of a kernel that only reads, same pools, one launch, this GPU, this run: as a
    # burst (10 launches) and sustained (as many launches as fill 0.3 s, like the timed region)
    read_gbs, bulk_gbs, bulk_sustained, read_bytes = None, None, None, 0
    if rank == 0:
        from flash_attention_factory_b200 import _test_aids

        kp, vp = w.k[0], w.v[0]
        read_bytes = (kp.numel() + vp.numel()) * kp.element_size()
        if read_bytes >= 4 * L2_BYTES:  # several times L2, else the figure is not an HBM figure
            cur = torch.cuda.current_stream(device).cuda_stream
            read_gbs = _test_aids.measure_read_bandwidth(kp.data_ptr(), read_bytes // 2, 10, cur,
                                                         vp.data_ptr(), read_bytes // 2, method=0)
            bulk_gbs = _test_aids.measure_read_bandwidth(kp.data_ptr(), read_bytes // 2, 10, cur,
                                                         vp.data_ptr(), read_bytes // 2, method=1)
            long_run = max(10, min(1000, int(0.3 * 7.0e12 / read_bytes)))
            bulk_sustained = _test_aids.measure_read_bandwidth(kp.data_ptr(), read_bytes // 2, long_run, cur,
                                                               vp.data_ptr(), read_bytes // 2, method=1)
    cpu = cpu_baseline(w) if (rank == 0 and world == 1 and not a.no_cpu_baseline) else None
    kv_bytes_rank0 = w.kv_bytes
    entry_variant = w.entry_variant() or "auto"
    w.free()

    # ---- the other workloads of the record
    variants = {}
    if not a.no_variants and not overridden:
        if world == 1:
            for name, cfg, var, kv in VARIANT_TABLE:
                if (cfg, var, kv) == (a.config, variant, None):
                    continue
                vs = config_spec(cfg)
                if kv is not None:
                    vs["kv"] = kv
                vctx = draw_context_lens(vs, seed=CONFIG_SEEDS[cfg])
                vw = Workload(vs, vctx, device, seed=1000 * CONFIG_SEEDS[cfg], variant=var)
                vm = measure_workload(vw, a, group, 0.25, 0.2, with_errors=True, kernel_reps=10, error_seqs=3)
                row = variant_row(vm, peak)
                if cfg == "c1":  # a few MB of KV: latency-bound, microseconds are the figure
                    row = {k: row[k] for k in ("us_per_call", "kernel_us", "e2e_us_per_call", "errors", "timed_ms")}
                row["entry_point"] = f"launch_kernels_{'fp8_' if vw.fp8 else ''}{var}"
                row["kv"] = vs["kv"]
                variants[name] = row
                vw.free()
        else:
            # config 4 (16 sequences of 32768 tokens, 8 KV heads) divided both ways
            for name, vshard in (("c4_split_by_kv_head", "heads"), ("c4_split_by_sequence", "contiguous")):
                vs = config_spec("c4")
                if vshard == "heads" and vs["kv_heads"] % world != 0:
                    continue
                vctx_all = draw_context_lens(vs, seed=CONFIG_SEEDS["c4"])
                s2, c2, _ = shard_spec_and_ctx(vs, vctx_all, vshard, world, rank)
                vw = Workload(s2, c2, device, seed=4000 + rank, variant="reduce")
                vm = measure_workload(vw, a, group, 0.25, 0.2, with_errors=(rank == 0), kernel_reps=10, error_seqs=2)
                row = variant_row(vm, peak, world)
                row["entry_point"], row["kv"] = "launch_kernels_fp8_reduce", vs["kv"]
                row["per_gpu"] = f"{s2['kv_heads']} KV heads x {int(c2.numel())} sequences"
                variants[name] = row
                vw.free()
        pkg.device_status()

    if rank == 0:
        errors = m["errors"]
        all_ok = bool(errors["within_tol"]) and all(v.get("errors", {}).get("within_tol", True)
                                                    for v in variants.values())
        line = {
            "metric": "decode_attention_kv_GBps", "value": round(m["gbs"], 1), "unit": "GB/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(m["ms_total"] / a.steps, 5), "calls_per_step": m["calls_per_step"],
            "us_per_call": round(m["us_per_call"], 2), "higher_is_better": True,
            "scaling": "strong" if a.strong else "weak", "vs_baseline": None,
            "dtype": "f16 x f16 -> f32 (mma.sync), KV stored as " + spec["kv"], "data": "synthetic",
            "config": dict(describe_config(a, spec, variant, world, ctx_all, shard),
                           calls_per_step=m["calls_per_step"], timed_region_ms=round(m["ms_total"], 1),
                           e2e_calls_per_step=m["e2e_calls_per_step"]),
            "pct_of_8TBps": round(100 * m["gbs"] / (NOMINAL_HBM_GBS * world), 2),
            "roofline": {"bound": "hbm", "kernel": "paged_attention_kernel (" + entry_variant + ")",
                         "achieved": round(m["kernel_gbs"], 1), "peak": peak, "unit": "GB/s",
                         "frac": round(m["kernel_gbs"] / peak, 4), "peak_kind": f"of {peak_kind}",
                         "frac_of_8TBps": round(m["kernel_gbs"] / NOMINAL_HBM_GBS, 4),
                         "algorithmic_bytes_per_launch": kv_bytes_rank0,
                         "read_only_stream_gbs": round(read_gbs, 1) if read_gbs else None,
                         "read_only_bulk_copy_gbs": round(bulk_gbs, 1) if bulk_gbs else None,
                         "read_only_bulk_copy_sustained_gbs": round(bulk_sustained, 1) if bulk_sustained else None,
                         "read_only_stream_bytes": read_bytes if read_gbs else None,
                         "frac_of_read_only_stream": round(m["kernel_gbs"] / max(read_gbs, bulk_gbs), 4) if read_gbs else None,
                         "frac_of_read_only_stream_sustained": round(m["gbs"] / bulk_sustained, 4) if bulk_sustained else None,
                         "kernel_us": round(m["kernel_us"], 2),
                         "merge_kernel_us": round(m["merge_us"], 2) if m["merge_us"] else None,
                         "traffic": traffic_bytes(a.config, entry_variant, kv_bytes_rank0) if not overridden else None,
                         "errors": dict({k: (round(v, 6) if isinstance(v, float) else v) for k, v in errors.items()},
                                        all_workloads_within_tol=all_ok),
                         "variants": variants},
            "errors": {"max_abs": round(errors["max_abs"], 6), "max_rel": round(errors["max_rel"], 6),
                       "within_tol": all_ok, "checked_seqs": errors["checked_seqs"]},
            "e2e": {"value": round(m["e2e_gbs"], 1), "unit": "GB/s",
                    "h2d_bytes_per_step": m["e2e_plan"]["h2d_bytes"] * m["e2e_calls_per_step"],
                    "d2h_bytes_per_step": m["e2e_plan"]["d2h_bytes"] * m["e2e_calls_per_step"],
                    "h2d_bytes_per_call": m["e2e_plan"]["h2d_bytes"], "d2h_bytes_per_call": m["e2e_plan"]["d2h_bytes"],
                    "us_per_call": round(m["e2e_us_per_call"], 2), "sub_batches": m["e2e_plan"]["sub_batches"],
                    "api": "pa_decode_step_host_batch (host_io.DecodeBatchIO)"},
            "gpu_launches": m["launches"],
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one attention-kernel launch over
# its algorithmic bytes, from the ncu captures of smaller cases of the same kernels summarised
# under profiles/ (traffic grows in proportion to the KV bytes: every sequence streams its own
# KV once); None until a capture exists for the workload
TRAFFIC_RATIO: dict = {
    # profiles/paged_attention_kernel_split_e5m2_c5_small.md: (1046.30 + 7.10) MB for 1042.26 MB
    ("c5", "reduce"): 1.01072, ("c5", "auto"): 1.01072,
    # profiles/paged_attention_kernel_split_e4m3_c4_small.md: (537.14 + 5.04) MB for 536.87 MB
    ("c4", "reduce"): 1.00990,
    # profiles/paged_attention_kernel_loop_e4m3_c4_small.md: (537.14 + 3.48) MB for 536.87 MB
    ("c4", "loop"): 1.00698,
    # profiles/paged_attention_kernel_loop_e5m2_c3_small.md: (514.74 + 3.11) MB for 513.46 MB
    ("c3", "loop"): 1.00854,
    # profiles/paged_attention_kernel_fp16_c2_small.md: split (1073.97 + 3.24) MB, loop (1074.05 + 3.51) MB for 1073.74 MB
    ("c2", "reduce"): 1.00323, ("c2", "loop"): 1.00355,
    # profiles/paged_attention_kernel_loop_e5m2_refperf8.md: (101.10 + 2.96) MB for 98.30 MB (block tails)
    ("refperf8", "loop"): 1.05852,
}


def traffic_bytes(config: str, variant: str, kv_bytes: int):
    ratio = TRAFFIC_RATIO.get((config, variant))
    return int(round(ratio * kv_bytes)) if ratio else None


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


def run_reference_arm(a, spec: dict, variant: str, world: int, shard: str) -> None:
    """`--impl reference`: the reference's CPU algorithm (oracle port) on the host cores.

    The reference's GPU kernels are Intel SYCL/ESIMD and cannot be built for this machine; its
    CPU implementation of the path is the torch code of its tests, restated in oracle/.  Every
    step runs the oracle on a bounded sample of the configured workload."""
    ctx = draw_context_lens(spec, seed=CONFIG_SEEDS[a.config])
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
        sinks = (torch.randn(h, generator=g) * 2 + 3).to(torch.float16) if spec.get("sinks") else None
        return dict(query=q, key_cache=k, value_cache=v, block_tables=bt, context_lens=c,
                    sm_scale=1.0 / math.sqrt(d), fp8_scale=scale, sinks=sinks)

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
        "higher_is_better": True, "scaling": "strong" if a.strong else "weak",
        "vs_baseline": None, "dtype": "f32 (CPU)",
        "data": "synthetic",
        "config": describe_config(a, spec, variant, world, ctx, shard),
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


if __name__ == "__main__":
    main()
