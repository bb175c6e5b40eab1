"""Split-context launches of different kernel instantiations that run at the same time.

The library's contract allows calls on different streams (with different buffers) to overlap.  The
split kernel draws its work items from a table of counters of which every launch must hold a
row of its own; the table is shared by all instantiations of a translation unit (wide and
default CTA shape, e5m2 and e4m3, head 128 and 64).  A child process (fresh counter state,
PA_WIDE_CTA=1) runs such pairs concurrently on two streams and compares output and scratch
with each launch run alone, bit for bit; this process checks the solitary outputs against the
oracle.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import _overlap_cases as cases
from _util import assert_close
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def test_concurrent_split_launches_of_one_unit_do_not_share_counters(cuda_device, tmp_path):
    out_file = tmp_path / "overlap.pt"
    env = dict(os.environ, PA_WIDE_CTA="1")
    res = subprocess.run([sys.executable, str(Path(cases.__file__).resolve()), str(out_file)], env=env,
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout + res.stderr
    report = torch.load(out_file)
    assert report["mismatches"] == [], "\n".join(report["mismatches"])
    for name in cases.PROBLEMS:
        c = cases.build(name)
        sample = [0, len(c["context_lens"]) // 2, len(c["context_lens"]) - 1]
        want = oracle.paged_attention_ref(c["query"][sample], c["key_cache"], c["value_cache"],
                                          c["block_tables"][sample], c["context_lens"][sample],
                                          sm_scale=c["sm_scale"])
        assert_close(report["serial_out"][name][sample], want, what=name)
