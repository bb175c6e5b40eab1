"""Replay of the reference's own parametrisation (test_paged.py:211-256,
test_paged_fp8cache.py) on all four entry points: block 64, head 128/64, the nine
(heads, kv heads) pairs, sinks on/off, full / ragged lengths, seed 0 — with both acceptance
criteria: BASELINE's atol 1e-3 / rtol 1e-2 and the reference's 3x-the-fp16-error bound."""
import pytest
import torch

from _util import assert_close, make_case, run_entry
from oracle import paged_attention_oracle as oracle

pytestmark = pytest.mark.gpu

HEADS = [(8, 1), (16, 2), (10, 2), (14, 2), (12, 2), (8, 2), (6, 2), (4, 2), (2, 2)]
SEQLENS = [128, 339, 1024, 800, 256, 799, 2048]


def _lengths(seqlen, batch, varlen, seed):
    if not varlen:
        return [seqlen] * batch
    g = torch.Generator().manual_seed(seed)
    # generate_random_padding_mask(mode="random"): uniform in [max(1, S - 20), S] (test_paged.py:201-203)
    return torch.randint(max(1, seqlen - 20), seqlen + 1, (batch,), generator=g).tolist()


@pytest.mark.parametrize("heads", HEADS, ids=lambda h: f"h{h[0]}k{h[1]}")
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("sinks", [True, False], ids=["sink", "nosink"])
@pytest.mark.parametrize("varlen", [False, True], ids=["full", "varlen"])
@pytest.mark.parametrize("kv", ["float16", "float8_e5m2"])
def test_reference_parametrisation(cuda_device, heads, d, sinks, varlen, kv):
    h, hk = heads
    # two sequence lengths of the reference list per case, rotating through it
    pick = (HEADS.index(heads) + (d == 64) + 2 * sinks + 3 * varlen) % len(SEQLENS)
    for seqlen in (SEQLENS[pick], SEQLENS[(pick + 3) % len(SEQLENS)]):
        batch = 2 if seqlen != 2048 else 1
        ctx = _lengths(seqlen, batch, varlen, seed=seqlen)
        c = make_case(seed=0, num_seqs=batch, num_heads=h, num_kv_heads=hk, head_size=d, block_size=64,
                      context_lens=ctx, kv_dtype=kv)
        if sinks:
            c["sinks"] = torch.ones(h, dtype=torch.float16) * 10  # test_paged.py:414-417
        ref = oracle.paged_attention_ref(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                         c["context_lens"], sm_scale=None, sinks=c["sinks"])
        pt = oracle.paged_attention_ref_fp16(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                             c["context_lens"], sinks=c["sinks"])
        bound = 3 * (pt.float() - ref.float()).abs().max().item() + 1e-5
        for variant in ("loop", "reduce"):
            out = run_entry(variant, c, cuda_device)["out"]
            assert_close(out, ref, what=f"{heads}/{d}/{seqlen}/{variant}")
            err = (out.float() - ref.float()).abs().max().item()
            assert err <= bound, f"reference criterion {err} > {bound} ({heads}, d={d}, S={seqlen}, {variant})"
