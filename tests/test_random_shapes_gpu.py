"""Seeded random shapes through all four operators against the oracle."""
import random

import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu


def _random_case(seed):
    rng = random.Random(seed)
    d = rng.choice([64, 128])
    bs = rng.choice([16, 32, 64, 128])
    hk = rng.choice([1, 2, 3, 4, 6, 8, 16])
    group = rng.randint(1, 8)
    kv = rng.choice(["float16", "float8_e5m2", "float8_e4m3fn"])
    s = rng.randint(1, 6)
    psize = 512 if d == 128 else 256
    ctx = []
    for _ in range(s):
        kind = rng.random()
        if kind < 0.2:
            ctx.append(rng.choice([0, 1, bs - 1, bs, bs + 1]))
        elif kind < 0.5:
            ctx.append(rng.choice([psize - 1, psize, psize + 1, 2 * psize, 2 * psize + 17]))
        else:
            ctx.append(rng.randint(1, 3000))
    sinks = rng.random() < 0.5
    scale = rng.choice([1.0, 0.5, 0.37]) if kv != "float16" else 1.0
    return dict(seed=seed, num_seqs=s, num_heads=hk * group, num_kv_heads=hk, head_size=d, block_size=bs,
                context_lens=ctx, kv_dtype=kv, sinks=sinks, fp8_scale=scale)


@pytest.mark.parametrize("seed", range(1000, 1024))
def test_random_shape(cuda_device, seed):
    spec = _random_case(seed)
    c = make_case(**spec)
    want = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                      c["context_lens"], sm_scale=c["sm_scale"], sinks=c["sinks"],
                                      fp8_scale=c["fp8_scale"])
    for variant in ("loop", "reduce"):
        got = run_entry(variant, c, cuda_device)["out"]
        assert_close(got, want, what=f"{variant} {spec}")
    import flash_attention_factory_b200 as pkg

    pkg.device_status()
