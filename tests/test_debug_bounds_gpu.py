"""The range-checked build (-DPA_DEBUG_BOUNDS) names the first index it finds out of range.

The product build makes every index that a malformed block table or context length can move safe
without saying so (a block id beyond the cache reads zeros through the tensor-map bounds, a
context length beyond the block-table row is cut).  The range-checked build of the same sources
records kind, value, limit, sequence and token of the first such value per translation unit;
a child process loads it (PA_B200_LIBRARY_VARIANT=bounds) and runs well-formed and malformed
inputs through the four entry points.  The reference trusts both tensors
(paged_attention_loop/launch_kernels_loop.h:114-115,170-172 check sizes only).
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import _bounds_cases as cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def report(cuda_device, tmp_path_factory):
    from flash_attention_factory_b200 import _cabi

    variant = Path(_cabi.library_path()).with_name("libpaged_attention_b200_bounds.so")
    assert variant.exists(), ("the range-checked build is missing: run "
                              "`python -m flash_attention_factory_b200.build --bounds`")
    out_file = tmp_path_factory.mktemp("bounds") / "bounds.pt"
    env = dict(os.environ, PA_B200_LIBRARY_VARIANT="bounds")
    res = subprocess.run([sys.executable, str(Path(cases.__file__).resolve()), str(out_file)], env=env,
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout + res.stderr
    return torch.load(out_file)


@pytest.mark.parametrize("unit", list(cases.UNITS))
def test_well_formed_inputs_leave_no_finding(report, unit):
    r = report["clean"][unit]
    assert r["report"][0] == 0, r["report"]
    assert r["close"]


@pytest.mark.parametrize("unit", list(cases.UNITS))
def test_block_id_beyond_the_cache_is_named_and_replaced_by_block_0(report, unit):
    r = report["block_id"][unit]
    count, kind, index, limit, seq, tok = r["report"][:6]
    assert count >= 1
    assert (kind, index, limit, seq) == (cases.KIND_BLOCK_ID, r["num_blocks"] + 7, r["num_blocks"], 1)
    assert 2 * cases.BLOCK <= tok < 3 * cases.BLOCK  # the token range of table column 2
    assert r["close"]


@pytest.mark.parametrize("unit", list(cases.UNITS))
def test_context_length_beyond_the_row_is_named_and_cut(report, unit):
    r = report["context"][unit]
    count, kind, index, limit, seq, _ = r["report"][:6]
    assert count >= 1
    assert (kind, index, limit, seq) == (cases.KIND_CONTEXT_LENGTH, r["limit"] + 5000, r["limit"] + 1, 1)
    assert r["close"]
