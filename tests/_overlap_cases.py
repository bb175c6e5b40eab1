"""Cases of tests/test_overlapping_launches_gpu.py, runnable as a script.

`python tests/_overlap_cases.py out.pt` runs pairs of split-context launches that belong to
DIFFERENT kernel instantiations of ONE translation unit, first each alone, then both at once on
two streams with nothing ordering them, several times, and records whether every concurrent run
reproduced the solitary run bit for bit (output and all three scratch tensors).  The parent
process sets PA_WIDE_CTA=1, so an FP8 launch with 8 KV heads takes the 8-warp CTA while one with
4 KV heads takes the default shape; the fp16 pair differs in head size.  Launches of one unit
share one table of work counters: if two launches in flight ever held the same row, each would
skip work items the other drew.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from _util import make_case  # noqa: E402

POISON = -7.0
REPEATS = 6

# name -> (kv, head_size, num_heads, num_kv_heads, context_lens)
PROBLEMS = {
    # FP8 unit: wide CTA (8 KV heads) against the default shape (4 KV heads)
    "fp8_wide": ("float8_e5m2", 128, 32, 8, [5000, 4097, 3000, 5120, 700, 2049, 4600, 1, 3333, 5119]),
    "fp8_default": ("float8_e5m2", 128, 16, 4, [2500 + 97 * i for i in range(24)]),
    # fp16 unit: head size 128 against head size 64
    "f16_d128": ("float16", 128, 8, 4, [1800 + 61 * i for i in range(16)]),
    "f16_d64": ("float16", 64, 16, 4, [1500 + 53 * i for i in range(20)]),
}
PAIRS = [("fp8_wide", "fp8_default"), ("f16_d128", "f16_d64")]


def build(name):
    kv, d, h, hk, ctx = PROBLEMS[name]
    return make_case(seed=500 + list(PROBLEMS).index(name), num_seqs=len(ctx), num_heads=h, num_kv_heads=hk,
                     head_size=d, block_size=16, context_lens=ctx, kv_dtype=kv)


class Launch:
    """Device tensors and the checked argument block of one problem."""

    def __init__(self, name, dev):
        from flash_attention_factory_b200 import _cabi
        from flash_attention_factory_b200 import lib

        c = build(name)
        self.fp8 = c["kv_dtype"] != "float16"
        self.mod = lib.paged_attention_fp8_reduce if self.fp8 else lib.paged_attention_reduce
        self.dev = dev
        q, k, v = c["query"].to(dev), c["key_cache"].to(dev), c["value_cache"].to(dev)
        bt, cl = c["block_tables"].to(dev), c["context_lens"].to(dev)
        s, h, d = q.shape
        psize = _cabi.partition_size(d)
        npart = (int(c["context_lens"].max()) + psize - 1) // psize
        self.ml = torch.empty((s, h, npart), dtype=torch.float32, device=dev)
        self.es = torch.empty_like(self.ml)
        self.tmp = torch.empty((s, h, npart, d), dtype=torch.float16, device=dev)
        self.out = torch.empty((s, h, d), dtype=torch.float16, device=dev)
        self.keep = (q, k, v, bt, cl)
        args = [self.ml, self.es, self.tmp, self.out, torch.zeros(1, device=dev), q, k, v, bt, cl, h // k.size(2),
                c["sm_scale"]]
        if self.fp8:
            args.append(1.0)
        args += [16, int(c["context_lens"].max()), torch.ones(h, device=dev), None, -1.0]
        self.params = self.mod.params(*args)

    def poison(self):
        for t in (self.ml, self.es, self.tmp, self.out):
            t.fill_(POISON)

    def enqueue(self):
        from flash_attention_factory_b200.lib import _shim

        _shim.enqueue_entry(self.mod.ENTRY, self.params, self.dev)

    def snapshot(self):
        return [t.clone() for t in (self.out, self.ml, self.es, self.tmp)]


def main(out_path):
    dev = torch.device("cuda:0")
    import flash_attention_factory_b200 as pkg

    report = {"serial_out": {}, "mismatches": []}
    streams = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    for pair in PAIRS:
        launches = [Launch(n, dev) for n in pair]
        serial = []
        for ln in launches:  # each alone (twice: the first call also loads the kernel image)
            for _ in range(2):
                ln.poison()
                ln.enqueue()
                torch.cuda.synchronize(dev)
            serial.append(ln.snapshot())
            report["serial_out"][pair[launches.index(ln)]] = ln.out.cpu()
        for rep in range(REPEATS):
            for ln in launches:
                ln.poison()
            torch.cuda.synchronize(dev)
            order = (0, 1) if rep % 2 == 0 else (1, 0)  # who is enqueued first alternates
            for idx in order:
                with torch.cuda.stream(streams[idx]):
                    launches[idx].enqueue()
            torch.cuda.synchronize(dev)
            for idx, ln in enumerate(launches):
                for what, got, want in zip(("out", "max_logits", "exp_sums", "tmp_out"), ln.snapshot(), serial[idx]):
                    if not torch.equal(got, want):
                        report["mismatches"].append(f"{pair[idx]} repeat {rep}: {what} differs from the solitary run")
    pkg.device_status()
    torch.save(report, out_path)


if __name__ == "__main__":
    main(sys.argv[1])
