"""B200-native paged-attention decode library.

A from-scratch sm_100a implementation of the four operators of
baodii/flash_attention_factory (loop / reduce x fp16 / FP8 KV cache) behind a
C ABI (``include/paged_attention_b200.h``).  ``flash_attention_factory_b200.lib``
mirrors the reference's ``lib`` package: four modules, each with ``run(...)``
taking the reference's positional arguments.

There is no CPU fallback: every operator raises if the CUDA library is missing
or no CUDA device is present.
"""
from ._cabi import (  # noqa: F401
    KV_F16,
    KV_FP8_E4M3,
    KV_FP8_E5M2,
    PaParams,
    PaPolicyInfo,
    device_status,
    library_path,
    load_library,
    partition_size,
    query_policy,
)

__version__ = "0.1"
