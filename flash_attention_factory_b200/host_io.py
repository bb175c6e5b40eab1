"""Host <-> device plumbing of one decode step: one packed upload, one download.

A decode step's host-side inputs are small (query, block tables, context lengths) and its
result is one [S, H, D] fp16 tensor.  Copying them as three separate tensors costs three
transfer latencies; `DecodeStepIO` keeps them in one pinned staging buffer with a device
mirror, so a step is one H2D copy, the kernel launches, one D2H copy and a stream wait.
The KV cache is not part of it: it is state that stays on the device.

`bind()` returns a `BoundStep` whose `run()` does the whole step as one call into the library (`pa_decode_step_host`):
the argument block is built once, so a step costs one ctypes call instead of tensor checks
and three torch calls.  With `direct_out=True` the kernels write the result straight into the
pinned host buffer (pinned memory is device-visible under unified addressing), which removes
the download copy from the critical path.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class DecodeStepIO:
    """Pinned host staging and device mirror for (query, block_tables, context_lens) plus a
    pinned host buffer for the output.  The host-side views are what the caller fills in."""

    def __init__(self, num_seqs: int, num_heads: int, head_size: int, max_blocks_per_seq: int, device):
        self.device = torch.device(device)
        q_bytes = num_seqs * num_heads * head_size * 2
        bt_bytes = num_seqs * max_blocks_per_seq * 4
        cl_bytes = num_seqs * 4
        off_bt = _round_up(q_bytes, 256)
        off_cl = off_bt + _round_up(bt_bytes, 256)
        total = off_cl + _round_up(cl_bytes, 256)
        self.host = torch.empty(total, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(total, dtype=torch.uint8, device=self.device)

        def views(buf):
            q = buf[:q_bytes].view(torch.float16).view(num_seqs, num_heads, head_size)
            bt = buf[off_bt:off_bt + bt_bytes].view(torch.int32).view(num_seqs, max_blocks_per_seq)
            cl = buf[off_cl:off_cl + cl_bytes].view(torch.int32)
            return q, bt, cl

        self.query_host, self.block_tables_host, self.context_lens_host = views(self.host)
        self.query, self.block_tables, self.context_lens = views(self.dev)
        self.out = torch.zeros(num_seqs, num_heads, head_size, dtype=torch.float16, device=self.device)
        self.out_host = torch.empty(num_seqs, num_heads, head_size, dtype=torch.float16).pin_memory()
        self.h2d_bytes = total
        self.d2h_bytes = self.out_host.numel() * 2

    def upload(self) -> None:
        """One asynchronous H2D copy of the whole staging buffer on the current stream."""
        self.dev.copy_(self.host, non_blocking=True)

    def download(self) -> torch.Tensor:
        """D2H copy of `out` on the current stream, then waits for the stream; returns the host tensor."""
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self.out_host

    def bind(self, entry: str, params: "_cabi.PaParams", direct_out: bool = False) -> "BoundStep":
        """Fixes the entry point and its argument block; `BoundStep.run()` then is one step.

        `params` is what `lib.<module>.params(...)` returned for tensors that include this
        object's `query`, `block_tables`, `context_lens` and `out`; it is copied, and with
        `direct_out` its `out` pointer is redirected to the pinned host buffer."""
        return BoundStep(self, entry, params, direct_out)


class BoundStep:
    """One decode step on fixed tensors as a single library call (`pa_decode_step_host`)."""

    def __init__(self, io: DecodeStepIO, entry: str, params: "_cabi.PaParams", direct_out: bool):
        self.io = io
        self.entry = _cabi.ENTRY_IDS[entry]
        self.params = _cabi.PaParams()
        ctypes.memmove(ctypes.byref(self.params), ctypes.byref(params), ctypes.sizeof(_cabi.PaParams))
        self.host_step = _cabi.PaHostStep()
        self.host_step.host_in = io.host.data_ptr()
        self.host_step.dev_in = io.dev.data_ptr()
        self.host_step.in_bytes = io.h2d_bytes
        if direct_out:
            self.params.out = io.out_host.data_ptr()
            self.host_step.host_out = None
            self.host_step.out_bytes = 0
        else:
            self.host_step.host_out = io.out_host.data_ptr()
            self.host_step.out_bytes = io.d2h_bytes
        self._fn = _cabi.load_library().pa_decode_step_host
        self._device_index = io.device.index if io.device.index is not None else torch.cuda.current_device()

    def run(self, synchronize: bool = True) -> torch.Tensor:
        """Upload, launch, download (and wait) on the current stream; returns the host result."""
        # the library reads the current device (SM count, kernel attributes, cached tables)
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self.io.device):
                return self.run(synchronize)
        stream = torch.cuda.current_stream(self.io.device).cuda_stream
        rc = self._fn(self.entry, ctypes.byref(self.params), ctypes.byref(self.host_step),
                      ctypes.c_void_p(stream), 1 if synchronize else 0)
        if rc != _cabi.PA_OK:
            _cabi.check(rc)
        return self.io.out_host
