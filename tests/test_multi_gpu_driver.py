"""Host logic of the multi-GPU driver (pa_multi_gpu_run): threads, start barrier, aggregation of
times and failures.  Runs without a GPU: PA_MULTI_GPU_HOST_ONLY makes the driver skip every CUDA
call, and a Python callable stands in for the per-shard launcher."""
import threading
import time

import pytest

from flash_attention_factory_b200 import _cabi, build
from flash_attention_factory_b200.multi_gpu import ShardedDecode, plan_shards
from flash_attention_factory_b200.sharding import shard_sequences_by_kv_length, shard_sequences_lpt


@pytest.fixture(scope="module", autouse=True)
def _library():
    build.build()
    return _cabi.load_library()


def _job(num_shards):
    job = ShardedDecode("contiguous")
    for i in range(num_shards):
        p = _cabi.PaParams()
        p.num_seqs = 100 + i  # lets the fake launcher tell the shards apart
        job.add_shard(f"cuda:{i}", "launch_kernels_fp8_reduce", p, [i])
    return job


def test_every_shard_runs_its_calls_on_its_own_thread_after_a_common_start():
    job = _job(4)
    calls, threads, first_call = {}, {}, {}
    lock = threading.Lock()

    def fake(entry, params, stream, user):
        sid = params.contents.num_seqs - 100
        with lock:
            calls[sid] = calls.get(sid, 0) + 1
            threads.setdefault(sid, set()).add(threading.get_ident())
            first_call.setdefault(sid, time.perf_counter())
        assert entry == _cabi.ENTRY_IDS["launch_kernels_fp8_reduce"]
        time.sleep(0.002 * (sid + 1))  # shard 3 is the slowest
        return _cabi.PA_OK

    worst, each = job.run(calls=5, warmup=2, launch=fake, host_only=True)
    assert calls == {0: 7, 1: 7, 2: 7, 3: 7}
    assert all(len(t) == 1 for t in threads.values())  # one thread per shard ...
    assert len({next(iter(t)) for t in threads.values()}) == 4  # ... and four different ones
    assert worst == pytest.approx(max(each)) and each[3] == max(each)  # max over shards
    assert 1500.0 < each[0] < each[1] < each[2] < each[3] < 30000.0  # microseconds per call


def test_a_failing_shard_is_reported_and_does_not_block_the_others():
    job = _job(4)
    done = {}
    lock = threading.Lock()

    def fake(entry, params, stream, user):
        sid = params.contents.num_seqs - 100
        with lock:
            done[sid] = done.get(sid, 0) + 1
            n = done[sid]
        if sid == 2 and n == 2:
            return _cabi.PA_ERR_CUDA  # second call of shard 2 fails
        return _cabi.PA_OK

    t0 = time.perf_counter()
    with pytest.raises(RuntimeError, match=r"shard 2 \(device 2\)"):
        job.run(calls=3, warmup=1, launch=fake, host_only=True)
    assert time.perf_counter() - t0 < 5.0  # nobody waited for the failed shard
    assert done[0] == done[1] == done[3] == 4  # the healthy shards finished all their calls
    assert done[2] == 2  # the failed one stopped at its failure

    def always_fails(entry, params, stream, user):
        return _cabi.PA_ERR_BAD_ARG

    with pytest.raises(RuntimeError) as info:
        job.run(calls=1, launch=always_fails, host_only=True)
    assert all(f"shard {i}" in str(info.value) for i in range(4))  # every failing shard is named


def test_bad_arguments_are_refused():
    import ctypes

    lib = _cabi.load_library()
    opt = _cabi.PaMultiGpuOptions()
    shard = (_cabi.PaDeviceShard * 1)()
    assert lib.pa_multi_gpu_run(shard, 1, ctypes.byref(opt), None, None) == _cabi.PA_ERR_BAD_ARG  # calls == 0
    opt.calls = 1
    assert lib.pa_multi_gpu_run(None, 1, ctypes.byref(opt), None, None) == _cabi.PA_ERR_BAD_ARG
    assert lib.pa_multi_gpu_run(shard, 0, ctypes.byref(opt), None, None) == _cabi.PA_ERR_BAD_ARG


def test_library_sharding_schemes_agree_with_the_python_helpers():
    import random

    rng = random.Random(3)
    for _ in range(20):
        lens = [max(1, min(32768, int(rng.lognormvariate(7.5, 1.0)))) for _ in range(rng.randint(1, 400))]
        for parts in (1, 2, 4, 8):
            assert plan_shards(lens, 8, parts, "lpt") == shard_sequences_lpt(lens, parts)
            assert plan_shards(lens, 8, parts, "contiguous") == [
                list(range(lo, hi)) for lo, hi in shard_sequences_by_kv_length(lens, parts)]
    assert plan_shards([5, 5, 5], 8, 2, "lpt") == [[0, 2], [1]]
    assert plan_shards([1, 2, 3], 8, 4, "heads") == [(0, 2), (2, 4), (4, 6), (6, 8)]
