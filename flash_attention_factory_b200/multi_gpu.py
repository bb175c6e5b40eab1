"""One decode batch on several GPUs of one process (`pa_multi_gpu_run`).

No counterpart in the reference, which is single-device (launch_kernels_loop.h:32-34).  Every
(sequence, KV head) of the path is independent, so a batch shards with no exchange step: by
sequence (consecutive ranges with equal KV shares, or longest-first to the lightest GPU) or by
KV head (few very long sequences).  Each shard owns its KV pool, tables, queries and outputs on
its GPU; the library runs the shards from one host thread and stream each, behind a common
start barrier, and reports the slowest shard.  The only cross-GPU step is the optional gather
of the outputs afterwards.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _cabi
from .sharding import shard_kv_heads


def plan_shards(context_lens: Sequence[int], num_kv_heads: int, parts: int, scheme: str):
    """What each shard holds: lists of sequence ids ("contiguous", "lpt") or [lo, hi) KV-head
    ranges ("heads").  The sequence schemes are computed by the library
    (pa_split_by_kv_length / pa_split_lpt), so every caller, in any language, gets the same cut."""
    if scheme == "heads":
        return shard_kv_heads(num_kv_heads, parts)
    if scheme == "lpt":
        return _cabi.split_lpt(context_lens, parts)
    if scheme == "contiguous":
        return [list(range(lo, hi)) for lo, hi in _cabi.split_by_kv_length(context_lens, parts)]
    raise ValueError(f"unknown sharding scheme {scheme!r}")


class ShardedDecode:
    """The shards of one batch and the call that runs them together."""

    def __init__(self, scheme: str):
        self.scheme = scheme
        self.devices: List[int] = []
        self.entries: List[str] = []
        self.params: List[_cabi.PaParams] = []
        self.keep = []  # the tensors behind the pointers
        self.assignment = []

    def add_shard(self, device, entry: str, params: _cabi.PaParams, assignment, keep=()) -> None:
        """`params` is the shard's argument block (all tensors on `device`), e.g. from
        `lib.<module>.params(...)`; `assignment` what `plan_shards` gave this shard."""
        self.devices.append(torch.device(device).index or 0)
        self.entries.append(entry)
        copy = _cabi.PaParams()
        ctypes.memmove(ctypes.byref(copy), ctypes.byref(params), ctypes.sizeof(_cabi.PaParams))
        self.params.append(copy)
        self.keep.append(keep)
        self.assignment.append(assignment)

    def _shard_array(self):
        arr = (_cabi.PaDeviceShard * len(self.params))()
        for i, p in enumerate(self.params):
            arr[i].device = self.devices[i]
            arr[i].entry = _cabi.ENTRY_IDS[self.entries[i]]
            ctypes.memmove(ctypes.byref(arr[i].params), ctypes.byref(p), ctypes.sizeof(_cabi.PaParams))
        return arr

    def run(self, calls: int = 1, warmup: int = 0, launch=None, host_only: bool = False):
        """Runs all shards at the same time; returns (microseconds per call of the slowest
        shard, list of microseconds per call of every shard).  `launch` (a Python callable
        `(entry, params_pointer, stream, user) -> status`) stands in for the library's entry
        points in tests of the driver itself."""
        opt = _cabi.PaMultiGpuOptions()
        opt.calls, opt.warmup = calls, warmup
        opt.flags = _cabi.MULTI_GPU_HOST_ONLY if host_only else 0
        callback = _cabi.SHARD_LAUNCH_FN(launch) if launch is not None else ctypes.cast(None, _cabi.SHARD_LAUNCH_FN)
        opt.launch = callback
        worst = ctypes.c_float(0.0)
        each = (ctypes.c_float * len(self.params))()
        arr = self._shard_array()
        _cabi.check(_cabi.load_library().pa_multi_gpu_run(arr, len(self.params), ctypes.byref(opt),
                                                          ctypes.byref(worst), each))
        return float(worst.value), [float(x) for x in each]

    def gather(self, dst: torch.Tensor) -> torch.Tensor:
        """Collects the shards' outputs into `dst` with peer copies: [S, H, D] in the batch's
        own sequence order (by-sequence schemes) or with the heads side by side ("heads")."""
        by_heads = self.scheme == "heads"
        mode = _cabi.GATHER_BY_KV_HEAD if by_heads else _cabi.GATHER_BY_SEQUENCE
        staging = dst if (by_heads or self.scheme == "contiguous") else torch.empty_like(dst)
        _cabi.check(_cabi.load_library().pa_multi_gpu_gather_out(
            self._shard_array(), len(self.params), mode, ctypes.c_void_p(staging.data_ptr()),
            dst.device.index or 0, dst.size(1)))
        if staging is not dst:
            # rows arrived shard after shard: put them back into the batch's order
            order = torch.tensor([i for ids in self.assignment for i in ids], dtype=torch.long, device=dst.device)
            dst[order] = staging
        return dst


def shard_reference_batch(case: dict, devices: Sequence, scheme: str, variant: str,
                          max_num_partitions: Optional[int] = None) -> ShardedDecode:
    """Builds the shards of a batch given as CPU tensors in the reference's layouts (query,
    key_cache, value_cache, block_tables, context_lens, sm_scale, optional sinks / fp8_scale):
    by sequence, every shard gets its sequences' rows and a compacted pool of the blocks they
    use (ids renumbered); by KV head, every shard gets all sequences and its slice of the heads.
    A convenience for tests and benchmarks; a serving system builds its shards where the data is."""
    from . import lib

    ctx = [int(c) for c in case["context_lens"].tolist()]
    hk = case["key_cache"].size(2)
    h = case["query"].size(1)
    group = h // hk
    d = case["query"].size(2)
    bs = case["key_cache"].size(1)
    fp8 = case["key_cache"].dtype != torch.float16
    mod = getattr(lib, f"paged_attention_{'fp8_' if fp8 else ''}{variant}")
    psize = _cabi.partition_size(d)
    plan = plan_shards(ctx, hk, len(devices), scheme)
    job = ShardedDecode(scheme)
    for dev, part in zip(devices, plan):
        dev = torch.device(dev)
        if scheme == "heads":
            lo, hi = part
            ids = list(range(len(ctx)))
            q = case["query"][:, lo * group:hi * group, :].contiguous()
            k = case["key_cache"][:, :, lo:hi, :].contiguous()
            v = case["value_cache"][:, :, lo:hi, :].contiguous()
            bt = case["block_tables"]
            sinks = case["sinks"][lo * group:hi * group].contiguous() if case.get("sinks") is not None else None
        else:
            ids = list(part)
            sel = torch.tensor(ids, dtype=torch.long)
            q = case["query"][sel].contiguous()
            counts = [(ctx[i] + bs - 1) // bs for i in ids]
            used = torch.cat([case["block_tables"][i, :n] for i, n in zip(ids, counts)]).long() if ids else \
                torch.zeros(0, dtype=torch.long)
            k = case["key_cache"][used] if used.numel() else case["key_cache"][:1]
            v = case["value_cache"][used] if used.numel() else case["value_cache"][:1]
            bt = torch.zeros(max(1, len(ids)), case["block_tables"].size(1), dtype=torch.int32)
            pos = 0
            for r, n in enumerate(counts):
                bt[r, :n] = torch.arange(pos, pos + n, dtype=torch.int32)
                pos += n
            sinks = case.get("sinks")
        s_i = len(ids)
        if s_i == 0:
            continue
        cl = torch.tensor([ctx[i] for i in ids], dtype=torch.int32)
        npart = max_num_partitions or max(1, (max(ctx) + psize - 1) // psize)
        hq = q.size(1)
        t = dict(q=q.to(dev), k=k.to(dev), v=v.to(dev), bt=bt.to(dev), cl=cl.to(dev),
                 ml=torch.zeros(s_i, hq, npart, dtype=torch.float32, device=dev),
                 es=torch.zeros(s_i, hq, npart, dtype=torch.float32, device=dev),
                 tmp=torch.zeros(s_i, hq, npart, d, dtype=torch.float16, device=dev),
                 out=torch.zeros(s_i, hq, d, dtype=torch.float16, device=dev),
                 alibi=torch.ones(hq, dtype=torch.float32, device=dev),
                 sinks=sinks.to(dev) if sinks is not None else None)
        args = [t["ml"], t["es"], t["tmp"], t["out"], None, t["q"], t["k"], t["v"], t["bt"], t["cl"], group,
                case["sm_scale"]]
        if fp8:
            args.append(case.get("fp8_scale", 1.0))
        args += [bs, max(ctx), t["alibi"], t["sinks"], -1.0]
        job.add_shard(dev, mod.ENTRY, mod.params(*args), part, keep=t)
    return job
