"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header
declares, reports the policy, and rejects bad arguments before touching a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

import flash_attention_factory_b200 as pkg
from flash_attention_factory_b200 import _cabi

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from flash_attention_factory_b200 import build

    build.build()
    return pkg.load_library()


def declared_symbols(header_name):
    text = (ROOT / "include" / header_name).read_text()
    return sorted(set(re.findall(r"PA_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from flash_attention_factory_b200 import _test_aids

    # every header under include/ belongs to one of the two libraries
    assert sorted(h.name for h in (ROOT / "include").glob("*.h")) == [
        "paged_attention_b200.h", "paged_attention_b200_test_aids.h"]
    names = declared_symbols("paged_attention_b200.h")
    assert set(_cabi.EXPORTED_SYMBOLS) == set(names)
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    aid_names = declared_symbols("paged_attention_b200_test_aids.h")
    assert set(_test_aids.EXPORTED_SYMBOLS) == set(aid_names)
    aids = _test_aids.load_library()
    for name in aid_names:
        assert hasattr(aids, name), f"{name} declared in the aid header but not exported"
    # the product library carries no test aid, and allocates nothing: it imports no allocator
    for name in aid_names + ["pa_selftest_wait_timeout", "pa_measure_read_bandwidth"]:
        assert not hasattr(lib, name), f"{name} must not be exported by the product library"


def test_public_header_is_plain_c(tmp_path):
    """include/paged_attention_b200.h compiles as C99 and the struct layout matches ctypes."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler on this machine")
    src = tmp_path / "abi_check.c"
    src.write_text(
        '#include <stddef.h>\n#include <stdio.h>\n#include "paged_attention_b200.h"\n'
        '#include "paged_attention_b200_test_aids.h"\n'
        "int main(void) {\n"
        "  pa_params p = {0};\n  pa_host_step io = {0};\n  pa_cache_write_params c = {0};\n"
        "  (void)io; (void)c; p.kv_dtype = PA_KV_FP8_E4M3;\n"
        '  printf("%zu %zu %zu %zu %zu\\n", sizeof(pa_params), offsetof(pa_params, num_blocks),\n'
        "         offsetof(pa_params, sm_scale), sizeof(pa_host_step), sizeof(pa_cache_write_params));\n"
        "  return p.kv_dtype == 2 ? 0 : 1;\n}\n")
    exe = tmp_path / "abi_check"
    subprocess.run([gcc, "-std=c99", "-pedantic", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)],
                   check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(x) for x in out] == [
        ctypes.sizeof(_cabi.PaParams), _cabi.PaParams.num_blocks.offset, _cabi.PaParams.sm_scale.offset,
        ctypes.sizeof(_cabi.PaHostStep), ctypes.sizeof(_cabi.PaCacheWriteParams)]


def test_params_struct_matches_header_layout():
    # 10 pointers, 10 uint32, uint64, 2 floats, 2 int32 with natural alignment
    assert ctypes.sizeof(_cabi.PaParams) == 10 * 8 + 10 * 4 + 8 + 2 * 4 + 2 * 4 + 2 * 8 + 8 + 2 * 4 + 8 + 8 + 2 * 8
    assert _cabi.PaParams.num_blocks.offset == 120
    assert _cabi.PaParams.sm_scale.offset == 128


@pytest.mark.parametrize("head,block", [(128, 16), (128, 64), (64, 16), (64, 64), (128, 32), (64, 128)])
def test_policy_knobs(lib, head, block):
    info = pkg.query_policy(head, block, 4)
    # the observable constants of the reference policy (paged_attention_policy_v2.hpp:6-7,28,35-36,50,58)
    assert info.partition_size == (512 if head == 128 else 256)
    assert info.stages == 3 and info.head_size_stride == 16 and info.partition_stride == 8
    assert info.max_partitions_per_sg == (4 if head == 128 else 16)
    assert info.partition_size % info.tokens_per_stage == 0
    assert info.threads_per_cta == 32 * (info.consumer_warps + 1)
    assert pkg.partition_size(head) == info.partition_size


def test_unsupported_shapes_use_the_reference_messages(lib):
    # launch_kernels_loop.h:114-115,170-172
    with pytest.raises(RuntimeError, match="Unsupported head size or block size"):
        pkg.query_policy(96, 64, 1)
    with pytest.raises(RuntimeError, match="Unsupported head size or block size"):
        pkg.query_policy(128, 48, 1)
    with pytest.raises(RuntimeError, match="Unsupported number of queries per token"):
        pkg.query_policy(128, 64, 9)
    assert pkg.partition_size(96) == 0


def _params(**kw):
    p = _cabi.PaParams()
    base = dict(out=0x1000, max_logits=0x2000, exp_sums=0x3000, tmp_out=0x4000, query=0x5000,
                key_cache=0x6000, value_cache=0x7000, block_tables=0x8000, context_lens=0x9000,
                num_seqs=2, num_heads=8, head_size=128, num_kv_heads=2, max_num_partitions=1,
                max_blocks_per_seq=4, block_size=16, num_queries_per_tokens=4, num_blocks=8,
                sm_scale=0.1, fp8_scale=1.0, kv_dtype=_cabi.KV_F16)
    base.update(kw)
    for k, v in base.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("entry,fp8", [("launch_kernels_loop", False), ("launch_kernels_reduce", False),
                                       ("launch_kernels_fp8_loop", True), ("launch_kernels_fp8_reduce", True)])
def test_launchers_validate_before_any_device_work(lib, entry, fp8):
    """Every rejection below happens on the host; nothing is launched."""
    fn = getattr(lib, entry)
    kv = _cabi.KV_FP8_E5M2 if fp8 else _cabi.KV_F16

    def call(**kw):
        kw.setdefault("kv_dtype", kv)
        p = _params(**kw)
        return fn(ctypes.byref(p), None, None), lib.pa_last_error().decode()

    rc, msg = call(head_size=96)
    assert rc == _cabi.PA_ERR_UNSUPPORTED and msg == "Unsupported head size or block size"
    rc, msg = call(block_size=24)
    assert rc == _cabi.PA_ERR_UNSUPPORTED and msg == "Unsupported head size or block size"
    rc, msg = call(num_queries_per_tokens=9, num_heads=18)
    assert rc == _cabi.PA_ERR_UNSUPPORTED and msg == "Unsupported number of queries per token"
    rc, msg = call(num_queries_per_tokens=0)
    assert rc == _cabi.PA_ERR_UNSUPPORTED
    rc, msg = call(kv_dtype=_cabi.KV_F16 if fp8 else _cabi.KV_FP8_E4M3)
    assert rc == _cabi.PA_ERR_BAD_ARG and "kv_dtype" in msg
    rc, msg = call(query=0)
    assert rc == _cabi.PA_ERR_BAD_ARG and "null" in msg
    rc, msg = call(num_heads=7)
    assert rc == _cabi.PA_ERR_BAD_ARG and "num_heads" in msg
    rc, msg = call(key_cache=0x6008)
    assert rc == _cabi.PA_ERR_BAD_ARG and "aligned" in msg
    rc, msg = call(num_blocks=0)
    assert rc == _cabi.PA_ERR_BAD_ARG
    if entry.endswith("reduce"):
        rc, msg = call(max_logits=0)
        assert rc == _cabi.PA_ERR_BAD_ARG and "max_logits" in msg
        rc, msg = call(max_num_partitions=0)
        assert rc == _cabi.PA_ERR_BAD_ARG
    # an empty batch is a successful no-op
    rc, _ = call(num_seqs=0)
    assert rc == _cabi.PA_OK
    assert fn(None, None, None) == _cabi.PA_ERR_BAD_ARG


def test_lib_modules_mirror_the_reference_surface():
    import inspect

    from flash_attention_factory_b200 import lib as shim

    # 17 positional arguments for fp16, 18 for FP8 (paged_attention_loop.cpp:21-38,
    # paged_attention_fp8_loop.cpp:21-39)
    for name, n in (("paged_attention_loop", 17), ("paged_attention_reduce", 17),
                    ("paged_attention_fp8_loop", 18), ("paged_attention_fp8_reduce", 18)):
        sig = inspect.signature(getattr(shim, name).run)
        assert len(sig.parameters) == n
        params = list(sig.parameters)
        assert params[:5] == ["max_logits", "exp_sums", "tem_output", "output", "debug_output"]
        if n == 18:
            assert params[12] == "fp8_scale"


def test_no_cpu_fallback():
    """CPU tensors are refused: the operators never compute on the host."""
    import torch

    from flash_attention_factory_b200 import lib as shim

    s, h, d = 1, 2, 128
    f32 = torch.zeros(s, h, 1)
    with pytest.raises(RuntimeError, match="CUDA"):
        shim.paged_attention_loop.run(
            f32, f32.clone(), torch.zeros(s, h, 1, d).half(), torch.zeros(s, h, d).half(),
            torch.zeros(s, h, d), torch.zeros(s, h, d).half(), torch.zeros(1, 16, 1, d).half(),
            torch.zeros(1, 16, 1, d).half(), torch.zeros(s, 1, dtype=torch.int32),
            torch.ones(s, dtype=torch.int32), 2, 0.1, 16, 1, torch.ones(h), None, -1.0)


def test_cache_write_validates_on_the_host(lib):
    def call(**kw):
        p = _cabi.PaCacheWriteParams()
        base = dict(key=0x1000, value=0x2000, key_cache=0x3000, value_cache=0x4000, slot_mapping=0x5000,
                    num_tokens=3, num_kv_heads=2, head_size=128, block_size=16, num_blocks=4,
                    fp8_scale=1.0, kv_dtype=_cabi.KV_FP8_E4M3)
        base.update(kw)
        for k, v in base.items():
            setattr(p, k, v)
        return lib.pa_reshape_and_cache(ctypes.byref(p), None), lib.pa_last_error().decode()

    assert call(num_tokens=0)[0] == _cabi.PA_OK
    assert call(kv_dtype=7)[0] == _cabi.PA_ERR_BAD_ARG
    assert call(key=0)[0] == _cabi.PA_ERR_BAD_ARG
    assert call(head_size=3)[0] == _cabi.PA_ERR_BAD_ARG
    assert call(fp8_scale=0.0)[0] == _cabi.PA_ERR_BAD_ARG
    assert call(key_cache=0x3004)[0] == _cabi.PA_ERR_BAD_ARG
    assert lib.pa_reshape_and_cache(None, None) == _cabi.PA_ERR_BAD_ARG
    # scale arrays: K and V together, one kind at most, FP8 caches only
    rc, msg = call(k_scale_per_head=0x6000)
    assert rc == _cabi.PA_ERR_BAD_ARG and "together" in msg
    rc, msg = call(v_scale_per_block=0x6000)
    assert rc == _cabi.PA_ERR_BAD_ARG and "together" in msg
    rc, msg = call(k_scale_per_head=0x6000, v_scale_per_head=0x7000, k_scale_per_block=0x8000,
                   v_scale_per_block=0x9000)
    assert rc == _cabi.PA_ERR_BAD_ARG and "exclude" in msg
    rc, msg = call(k_scale_per_block=0x8000, v_scale_per_block=0x9000, kv_dtype=_cabi.KV_F16)
    assert rc == _cabi.PA_ERR_BAD_ARG and "FP8" in msg


def test_static_scratch_refusals_need_no_gpu(lib):
    """The no-allocation entry point decides both refusals on the host, before any CUDA call."""
    p = _cabi.PaParams()
    p.num_seqs, p.num_heads, p.head_size, p.num_kv_heads, p.max_num_partitions = 2, 8, 128, 2, 4
    p.max_blocks_per_seq, p.block_size, p.num_queries_per_tokens = 128, 16, 4
    p.num_blocks, p.sm_scale, p.kv_dtype = 1 << 12, 0.1, _cabi.KV_F16
    p.seq_indices = 0x1000  # never dereferenced
    assert lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), None) == _cabi.PA_ERR_BAD_ARG
    assert "seq_indices" in lib.pa_last_error().decode()
    p.seq_indices = None
    p.num_seqs, p.num_heads, p.num_kv_heads, p.num_queries_per_tokens, p.max_num_partitions = 3259, 3, 3, 1, 13
    assert lib.launch_kernels_reduce_static_scratch(ctypes.byref(p), None) == _cabi.PA_ERR_BAD_ARG
    assert "static scratch too small" in lib.pa_last_error().decode()
