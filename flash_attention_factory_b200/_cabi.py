"""ctypes binding of libpaged_attention_b200.so (include/paged_attention_b200.h).

This is the only place that touches the shared library; the ``lib`` modules and
the tests go through it.  The library is loaded from this package directory and
nowhere else, and a missing library is an error (no fallback path exists).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

KV_F16 = 0
KV_FP8_E5M2 = 1
KV_FP8_E4M3 = 2

PA_OK = 0
PA_ERR_UNSUPPORTED = 1
PA_ERR_BAD_ARG = 2
PA_ERR_CUDA = 3
PA_ERR_TIMEOUT = 4

STATIC_SCRATCH_BYTES = 32 * 1024 * 1024  # PA_STATIC_SCRATCH_BYTES

_LIB_NAME = "libpaged_attention_b200.so"
_lib = None

EXPORTED_SYMBOLS = (
    "launch_kernels_loop",
    "launch_kernels_reduce",
    "launch_kernels_fp8_loop",
    "launch_kernels_fp8_reduce",
    "launch_kernels_reduce_static_scratch",
    "pa_reshape_and_cache",
    "pa_query_policy",
    "pa_partition_size",
    "pa_last_error",
    "pa_device_status",
    "pa_decode_step_host",
    "pa_decode_step_host_batch",
    "pa_split_by_kv_length",
    "pa_host_batch_plan",
    "pa_split_lpt",
    "pa_multi_gpu_run",
    "pa_multi_gpu_gather_out",
    "pa_version",
)


class PaParams(ctypes.Structure):
    """struct pa_params of include/paged_attention_b200.h (field order matters)."""

    _fields_ = [
        ("out", ctypes.c_void_p),
        ("max_logits", ctypes.c_void_p),
        ("exp_sums", ctypes.c_void_p),
        ("tmp_out", ctypes.c_void_p),
        ("query", ctypes.c_void_p),
        ("key_cache", ctypes.c_void_p),
        ("value_cache", ctypes.c_void_p),
        ("sinks", ctypes.c_void_p),
        ("block_tables", ctypes.c_void_p),
        ("context_lens", ctypes.c_void_p),
        ("num_seqs", ctypes.c_uint32),
        ("num_heads", ctypes.c_uint32),
        ("head_size", ctypes.c_uint32),
        ("num_kv_heads", ctypes.c_uint32),
        ("max_num_partitions", ctypes.c_uint32),
        ("max_blocks_per_seq", ctypes.c_uint32),
        ("block_size", ctypes.c_uint32),
        ("num_queries_per_tokens", ctypes.c_uint32),
        ("max_context_len", ctypes.c_uint32),
        ("reserved0", ctypes.c_uint32),
        ("num_blocks", ctypes.c_uint64),
        ("sm_scale", ctypes.c_float),
        ("fp8_scale", ctypes.c_float),
        ("kv_dtype", ctypes.c_int32),
        ("reserved1", ctypes.c_int32),
        ("k_scale_per_head", ctypes.c_void_p),
        ("v_scale_per_head", ctypes.c_void_p),
        ("alibi_slopes", ctypes.c_void_p),
        ("softcap", ctypes.c_float),
        ("reserved2", ctypes.c_float),
        ("seq_indices", ctypes.c_void_p),
        ("block_table_offsets", ctypes.c_void_p),
        ("k_scale_per_block", ctypes.c_void_p),
        ("v_scale_per_block", ctypes.c_void_p),
    ]


class PaPolicyInfo(ctypes.Structure):
    """struct pa_policy_info of include/paged_attention_b200.h."""

    _fields_ = [
        ("partition_size", ctypes.c_uint32),
        ("stages", ctypes.c_uint32),
        ("head_size_stride", ctypes.c_uint32),
        ("partition_stride", ctypes.c_uint32),
        ("max_partitions_per_sg", ctypes.c_uint32),
        ("tokens_per_stage", ctypes.c_uint32),
        ("ring_stages", ctypes.c_uint32),
        ("ring_stages_fp8", ctypes.c_uint32),
        ("consumer_warps", ctypes.c_uint32),
        ("threads_per_cta", ctypes.c_uint32),
    ]


class PaCacheWriteParams(ctypes.Structure):
    """struct pa_cache_write_params of include/paged_attention_b200.h."""

    _fields_ = [
        ("key", ctypes.c_void_p),
        ("value", ctypes.c_void_p),
        ("key_cache", ctypes.c_void_p),
        ("value_cache", ctypes.c_void_p),
        ("slot_mapping", ctypes.c_void_p),
        ("num_tokens", ctypes.c_uint32),
        ("num_kv_heads", ctypes.c_uint32),
        ("head_size", ctypes.c_uint32),
        ("block_size", ctypes.c_uint32),
        ("num_blocks", ctypes.c_uint64),
        ("fp8_scale", ctypes.c_float),
        ("kv_dtype", ctypes.c_int32),
        ("k_scale_per_head", ctypes.c_void_p),
        ("v_scale_per_head", ctypes.c_void_p),
        ("k_scale_per_block", ctypes.c_void_p),
        ("v_scale_per_block", ctypes.c_void_p),
    ]


class PaHostStep(ctypes.Structure):
    """struct pa_host_step of include/paged_attention_b200.h."""

    _fields_ = [
        ("host_in", ctypes.c_void_p),
        ("dev_in", ctypes.c_void_p),
        ("in_bytes", ctypes.c_uint64),
        ("host_out", ctypes.c_void_p),
        ("out_bytes", ctypes.c_uint64),
    ]


class PaHostBatch(ctypes.Structure):
    """struct pa_host_batch of include/paged_attention_b200.h."""

    _fields_ = [
        ("host_query", ctypes.c_void_p),
        ("host_block_tables", ctypes.c_void_p),
        ("host_block_table_offsets", ctypes.c_void_p),
        ("host_context_lens", ctypes.c_void_p),
        ("host_out", ctypes.c_void_p),
        ("sub_batches", ctypes.c_uint32),
        ("flags", ctypes.c_uint32),
        ("host_staging", ctypes.c_void_p),
        ("dev_staging", ctypes.c_void_p),
        ("staging_bytes", ctypes.c_uint64),
    ]


STEP_LAST_OUT_DIRECT = 1


class PaDeviceShard(ctypes.Structure):
    """struct pa_device_shard of include/paged_attention_b200.h."""

    _fields_ = [("device", ctypes.c_int32), ("entry", ctypes.c_int32), ("params", PaParams)]


SHARD_LAUNCH_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int32, ctypes.POINTER(PaParams), ctypes.c_void_p,
                                   ctypes.c_void_p)


class PaMultiGpuOptions(ctypes.Structure):
    """struct pa_multi_gpu_options of include/paged_attention_b200.h."""

    _fields_ = [
        ("calls", ctypes.c_uint32),
        ("warmup", ctypes.c_uint32),
        ("flags", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32),
        ("launch", SHARD_LAUNCH_FN),
        ("user", ctypes.c_void_p),
    ]


MULTI_GPU_HOST_ONLY = 1
GATHER_BY_SEQUENCE, GATHER_BY_KV_HEAD = 0, 1

ENTRY_IDS = {"launch_kernels_loop": 0, "launch_kernels_reduce": 1, "launch_kernels_fp8_loop": 2,
             "launch_kernels_fp8_reduce": 3}


def library_path() -> Path:
    """The product library, or (PA_B200_LIBRARY_VARIANT=<name>) a differently compiled build of it
    from this same directory, e.g. the one with per-CTA time stamps."""
    import os

    variant = os.environ.get("PA_B200_LIBRARY_VARIANT", "")
    if variant and variant.isalnum():
        return Path(__file__).resolve().parent / f"libpaged_attention_b200_{variant}.so"
    return Path(__file__).resolve().parent / _LIB_NAME


def load_library() -> ctypes.CDLL:
    """Loads the shared library (once) and declares the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m flash_attention_factory_b200.build` "
            "(there is no CPU or PyTorch fallback)"
        )
    lib = ctypes.CDLL(str(path))
    launcher_args = [ctypes.POINTER(PaParams), ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    for name in ("launch_kernels_loop", "launch_kernels_reduce", "launch_kernels_fp8_loop",
                 "launch_kernels_fp8_reduce"):
        fn = getattr(lib, name)
        fn.argtypes = launcher_args
        fn.restype = ctypes.c_int
    lib.launch_kernels_reduce_static_scratch.argtypes = [ctypes.POINTER(PaParams), ctypes.c_void_p]
    lib.launch_kernels_reduce_static_scratch.restype = ctypes.c_int
    lib.pa_reshape_and_cache.argtypes = [ctypes.POINTER(PaCacheWriteParams), ctypes.c_void_p]
    lib.pa_reshape_and_cache.restype = ctypes.c_int
    lib.pa_query_policy.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                    ctypes.POINTER(PaPolicyInfo)]
    lib.pa_query_policy.restype = ctypes.c_int
    lib.pa_partition_size.argtypes = [ctypes.c_uint32]
    lib.pa_partition_size.restype = ctypes.c_uint32
    lib.pa_last_error.argtypes = []
    lib.pa_last_error.restype = ctypes.c_char_p
    lib.pa_device_status.argtypes = []
    lib.pa_device_status.restype = ctypes.c_int
    lib.pa_decode_step_host.argtypes = [ctypes.c_int32, ctypes.POINTER(PaParams), ctypes.POINTER(PaHostStep),
                                        ctypes.c_void_p, ctypes.c_int32]
    lib.pa_decode_step_host.restype = ctypes.c_int
    lib.pa_decode_step_host_batch.argtypes = [ctypes.c_int32, ctypes.POINTER(PaParams), ctypes.POINTER(PaHostBatch),
                                              ctypes.c_void_p, ctypes.c_int32]
    lib.pa_decode_step_host_batch.restype = ctypes.c_int
    lib.pa_host_batch_plan.argtypes = [ctypes.POINTER(PaParams), ctypes.POINTER(PaHostBatch),
                                       ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint64),
                                       ctypes.POINTER(ctypes.c_uint64)]
    lib.pa_host_batch_plan.restype = ctypes.c_int
    lib.pa_split_lpt.argtypes = [ctypes.POINTER(ctypes.c_uint32), ctypes.c_uint32, ctypes.c_uint32,
                                 ctypes.POINTER(ctypes.c_uint32)]
    lib.pa_split_lpt.restype = ctypes.c_int
    lib.pa_multi_gpu_run.argtypes = [ctypes.POINTER(PaDeviceShard), ctypes.c_uint32, ctypes.POINTER(PaMultiGpuOptions),
                                     ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]
    lib.pa_multi_gpu_run.restype = ctypes.c_int
    lib.pa_multi_gpu_gather_out.argtypes = [ctypes.POINTER(PaDeviceShard), ctypes.c_uint32, ctypes.c_int32,
                                            ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32]
    lib.pa_multi_gpu_gather_out.restype = ctypes.c_int
    lib.pa_split_by_kv_length.argtypes = [ctypes.POINTER(ctypes.c_uint32), ctypes.c_uint32, ctypes.c_uint32,
                                          ctypes.POINTER(ctypes.c_uint32)]
    lib.pa_split_by_kv_length.restype = ctypes.c_int
    lib.pa_version.argtypes = []
    lib.pa_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def last_error() -> str:
    return load_library().pa_last_error().decode()


def check(rc: int) -> None:
    """Turns a pa_status into the exception the reference would have thrown.

    The reference throws std::runtime_error, which pybind11 surfaces as
    RuntimeError (paged_attention_loop/launch_kernels_loop.h:114-115,170-172).
    """
    if rc != PA_OK:
        raise RuntimeError(last_error())


def query_policy(head_size: int, block_size: int, group: int) -> PaPolicyInfo:
    info = PaPolicyInfo()
    check(load_library().pa_query_policy(head_size, block_size, group, ctypes.byref(info)))
    return info


def partition_size(head_size: int) -> int:
    return int(load_library().pa_partition_size(head_size))


def device_status() -> None:
    """Synchronises the current device and raises if a kernel gave up a bounded wait."""
    check(load_library().pa_device_status())


def split_by_kv_length(context_lens, parts: int) -> list[tuple[int, int]]:
    """[lo, hi) ranges of consecutive sequences with equal shares of the KV tokens (pa_split_by_kv_length)."""
    lens = [int(c) for c in context_lens]
    arr = (ctypes.c_uint32 * max(1, len(lens)))(*lens)
    bounds = (ctypes.c_uint32 * (parts + 1))()
    check(load_library().pa_split_by_kv_length(arr, len(lens), parts, bounds))
    return [(int(bounds[r]), int(bounds[r + 1])) for r in range(parts)]


def split_lpt(context_lens, parts: int) -> list[list[int]]:
    """Sequence ids per part, longest first to the lightest part (pa_split_lpt); ids ascending."""
    lens = [int(c) for c in context_lens]
    arr = (ctypes.c_uint32 * max(1, len(lens)))(*lens)
    part_of = (ctypes.c_uint32 * max(1, len(lens)))()
    check(load_library().pa_split_lpt(arr, len(lens), parts, part_of))
    shards = [[] for _ in range(parts)]
    for i in range(len(lens)):
        shards[int(part_of[i])].append(i)
    return shards


def launch(entry: str, params: PaParams, stream: int, timed: bool) -> list[float]:
    """Calls one launcher.  ``timed`` selects the blocking form that returns microseconds."""
    lib = load_library()
    fn = getattr(lib, entry)
    n_times = 2 if entry.endswith("reduce") else 1
    if timed:
        buf = (ctypes.c_float * 2)()
        check(fn(ctypes.byref(params), ctypes.c_void_p(stream), buf))
        return [float(buf[i]) for i in range(n_times)]
    check(fn(ctypes.byref(params), ctypes.c_void_p(stream), None))
    return []
