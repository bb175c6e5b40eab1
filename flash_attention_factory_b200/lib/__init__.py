"""Mirror of the reference's ``lib`` package (generated there by CMakeLists.txt:74-81).

``from flash_attention_factory_b200.lib import paged_attention_loop`` replaces the
reference's ``from lib import paged_attention_loop``; each module exposes ``run``.
"""
from . import (  # noqa: F401
    paged_attention_fp8_loop,
    paged_attention_fp8_reduce,
    paged_attention_loop,
    paged_attention_reduce,
)

__all__ = [
    "paged_attention_loop",
    "paged_attention_reduce",
    "paged_attention_fp8_loop",
    "paged_attention_fp8_reduce",
]
