"""The 8-warp ("wide") CTA of the FP8 split variant: same bits as the default shape, right answers.

The launcher picks the wide shape only for launches with at least two rounds of work, so the
cases here would all run in the default shape.  A child process with PA_WIDE_CTA=1 forces the
wide shape for them (sinks, ragged tails, block sizes, head size 64, per-head scales, score
modifiers, sequence subsets); this process runs the same cases in the default shape.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import _wide_cta_cases as cases
from _util import assert_close
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def test_wide_cta_gives_the_default_shapes_bits_and_the_oracles_answer(cuda_device, tmp_path):
    assert os.environ.get("PA_WIDE_CTA") in (None, "", "0"), "this process must run the default shape"
    out_file = tmp_path / "wide.pt"
    env = dict(os.environ, PA_WIDE_CTA="1")
    script = Path(cases.__file__).resolve()
    res = subprocess.run([sys.executable, str(script), str(out_file)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    wide = torch.load(out_file)
    for name in cases.CASES:
        default = cases.run_case(name, cuda_device)
        assert torch.equal(wide[name], default), f"{name}: the wide CTA gives other bits than the default shape"
        c = cases.build(name)
        want = oracle.paged_attention_ref(
            c["query"], c["key_cache"], c["value_cache"], c["block_tables"], c["context_lens"],
            sm_scale=c["sm_scale"], sinks=c["sinks"], fp8_scale=c["fp8_scale"], k_scales=c["k_scales"],
            v_scales=c["v_scales"], softcap=c["softcap"], alibi_slopes=c["alibi"],
            k_block_scales=c["k_block_scales"], v_block_scales=c["v_block_scales"])
        got = wide[name]
        if c["subset"] is not None:
            rest = [i for i in range(got.size(0)) if i not in c["subset"]]
            assert (got[rest] == -7.0).all(), "sequences outside the subset were written"
            got, want = got[c["subset"]], want[c["subset"]]
        scaled = c["v_scales"] is not None or c["v_block_scales"] is not None
        assert_close(got, want, atol=3e-3 if scaled else 1e-3, what=name)
