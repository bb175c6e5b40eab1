"""Cases of tests/test_debug_bounds_gpu.py, runnable as a script.

`PA_B200_LIBRARY_VARIANT=bounds python tests/_bounds_cases.py out.pt` loads the range-checked
build of the library (-DPA_DEBUG_BOUNDS) and runs, through the four entry points:

* well-formed inputs: no finding, results within tolerance of the oracle;
* a block id beyond the cache: recorded with its value, the limit and the sequence; the access
  uses block 0 instead, so the result is the oracle's with that table entry set to 0;
* a context length beyond the block-table row: recorded, cut to the row, result of the honest
  length.

None of the cases can fault: the product build zero-fills a block id beyond the cache through
the tensor-map bounds and cuts the context length; the range-checked build reports the same
values before making them safe.
"""
import ctypes
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from _util import ATOL, RTOL, make_case, run_entry  # noqa: E402
from oracle import paged_attention_oracle as oracle  # noqa: E402

KIND_TABLE_INDEX, KIND_BLOCK_ID, KIND_CONTEXT_LENGTH = 1, 2, 3
UNITS = {"loop": ("loop", "float16"), "reduce": ("reduce", "float16"),
         "fp8_loop": ("loop", "float8_e5m2"), "fp8_reduce": ("reduce", "float8_e5m2")}
BLOCK = 16
LIMIT_BLOCKS = 70


def bounds_report(unit: str) -> list:
    """Reads and clears the range-check report of one launcher's translation unit."""
    from flash_attention_factory_b200 import _cabi

    fn = getattr(_cabi.load_library(), f"pa_debug_bounds_{unit}")
    fn.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    fn.restype = ctypes.c_int
    buf = (ctypes.c_uint32 * 8)()
    rc = fn(buf)
    if rc != 0:
        raise RuntimeError(f"pa_debug_bounds_{unit} returned {rc}")
    return list(buf)


def close(actual, expected) -> bool:
    return bool(torch.allclose(actual.float().cpu(), expected.float().cpu(), atol=ATOL, rtol=RTOL))


def main(out_path: str) -> None:
    dev = torch.device("cuda:0")
    limit = BLOCK * LIMIT_BLOCKS
    report = {"clean": {}, "block_id": {}, "context": {}}
    for unit, (variant, kv) in UNITS.items():
        c = make_case(seed=91, num_seqs=4, num_heads=8, num_kv_heads=2, head_size=128, block_size=BLOCK,
                      context_lens=[limit - 3, limit, 200, limit - BLOCK], kv_dtype=kv)
        num_blocks = c["key_cache"].shape[0]
        want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                          c["context_lens"], sm_scale=c["sm_scale"])
        bounds_report(unit)  # clear
        res = run_entry(variant, c, dev)
        report["clean"][unit] = {"report": bounds_report(unit), "close": close(res["out"], want)}

        bad = dict(c)
        bad["block_tables"] = c["block_tables"].clone()
        bad["block_tables"][1, 2] = num_blocks + 7
        zeroed = c["block_tables"].clone()
        zeroed[1, 2] = 0
        want_zeroed = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], zeroed,
                                                 c["context_lens"], sm_scale=c["sm_scale"])
        res = run_entry(variant, bad, dev)
        report["block_id"][unit] = {"report": bounds_report(unit), "close": close(res["out"], want_zeroed),
                                    "num_blocks": num_blocks}

        lying = dict(c)
        lying["context_lens"] = torch.tensor([limit - 3, limit + 5000, 200, limit - BLOCK], dtype=torch.int32)
        res = run_entry(variant, lying, dev)
        report["context"][unit] = {"report": bounds_report(unit), "close": close(res["out"], want),
                                   "limit": limit}
    torch.save(report, out_path)


if __name__ == "__main__":
    main(sys.argv[1])
