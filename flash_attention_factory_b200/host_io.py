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


def pack_block_tables(block_tables: torch.Tensor, context_lens, block_size: int):
    """Dense [S, MB] tables -> (ids, offsets): the entries in use, row after row, and the
    S + 1 row offsets (`pa_params.block_table_offsets`).  Host-side helper."""
    lens = [int(c) for c in (context_lens.tolist() if torch.is_tensor(context_lens) else context_lens)]
    counts = [(c + block_size - 1) // block_size for c in lens]
    offsets = torch.zeros(len(lens) + 1, dtype=torch.int32)
    offsets[1:] = torch.tensor(counts, dtype=torch.int64).cumsum(0).to(torch.int32)
    ids = torch.cat([block_tables[i, :n] for i, n in enumerate(counts)]) if lens else block_tables.new_zeros(0)
    return ids.to(torch.int32).contiguous(), offsets


class DecodeBatchIO:
    """Host and device buffers of a pipelined decode step (`pa_decode_step_host_batch`).

    Pinned host tensors the caller fills (`query_host`, `context_lens_host`, and either the dense
    `block_tables_host` [S, MB] or, with `packed_capacity`, the packed `block_ids_host` /
    `block_offsets_host` pair), their device mirrors, and the pinned `out_host`.  `bind()` fixes
    the entry point and argument block; `BoundBatchStep.run()` is one step: the library cuts the
    batch into sub-batches and overlaps uploads, kernels and downloads."""

    def __init__(self, num_seqs: int, num_heads: int, head_size: int, max_blocks_per_seq: int, device,
                 packed_capacity: int = 0):
        self.device = torch.device(device)
        s = num_seqs
        self.packed = packed_capacity > 0
        # one pinned staging block and its device mirror with the same layout:
        # [query | context_lens | offsets (packed) | block ids or dense tables]
        q_bytes = s * num_heads * head_size * 2
        off_cl = _round_up(q_bytes, 256)
        off_offsets = off_cl + _round_up(4 * s, 256)
        off_tables = off_offsets + (_round_up(4 * (s + 1), 256) if self.packed else 0)
        table_entries = packed_capacity if self.packed else s * max_blocks_per_seq
        total = off_tables + _round_up(4 * table_entries, 256)
        self.host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.uint8, device=self.device)

        def views(buf):
            q = buf[:q_bytes].view(torch.float16).view(s, num_heads, head_size)
            cl = buf[off_cl:off_cl + 4 * s].view(torch.int32)
            offsets = buf[off_offsets:off_offsets + 4 * (s + 1)].view(torch.int32) if self.packed else None
            tables = buf[off_tables:off_tables + 4 * table_entries].view(torch.int32)
            return q, cl, offsets, tables

        self.query_host, self.context_lens_host, offsets_host, tables_host = views(self.host)
        self.query, self.context_lens, offsets_dev, tables_dev = views(self.dev)
        if self.packed:
            self.block_ids_host, self.block_offsets_host = tables_host, offsets_host
            self.block_ids, self.block_offsets = tables_dev, offsets_dev
            # what the entry points take as `block_tables`: a [1, capacity] view of the id list
            self.block_tables = self.block_ids.view(1, -1)
        else:
            self.block_tables_host = tables_host.view(s, max_blocks_per_seq)
            self.block_tables = tables_dev.view(s, max_blocks_per_seq)
        self.out_host = torch.empty(s, num_heads, head_size, dtype=torch.float16).pin_memory()
        self.out = torch.zeros(s, num_heads, head_size, dtype=torch.float16, device=self.device)

    def set_block_tables(self, block_tables: torch.Tensor, context_lens, block_size: int) -> None:
        """Fills the host-side tables from a dense [S, MB] tensor (packing them if this object is packed)."""
        if not self.packed:
            self.block_tables_host.copy_(block_tables)
            return
        ids, offsets = pack_block_tables(block_tables, context_lens, block_size)
        if ids.numel() > self.block_ids_host.numel():
            raise RuntimeError("packed block tables exceed the capacity this DecodeBatchIO was built with")
        self.block_ids_host[:ids.numel()].copy_(ids)
        self.block_offsets_host.copy_(offsets)

    def bind(self, entry: str, params: "_cabi.PaParams", sub_batches: int = 0,
             last_out_direct: bool = True) -> "BoundBatchStep":
        """`params` is the argument block for this object's device tensors (`query`,
        `block_tables`, `context_lens`, `out`); with packed tables its `block_table_offsets` is
        set here."""
        return BoundBatchStep(self, entry, params, sub_batches, last_out_direct)


class BoundBatchStep:
    """One pipelined decode step on fixed tensors as a single library call."""

    def __init__(self, io: DecodeBatchIO, entry: str, params: "_cabi.PaParams", sub_batches: int,
                 last_out_direct: bool):
        self.io = io
        self.entry = _cabi.ENTRY_IDS[entry]
        self.params = _cabi.PaParams()
        ctypes.memmove(ctypes.byref(self.params), ctypes.byref(params), ctypes.sizeof(_cabi.PaParams))
        self.batch = _cabi.PaHostBatch()
        self.batch.host_query = io.query_host.data_ptr()
        self.batch.host_context_lens = io.context_lens_host.data_ptr()
        self.batch.host_out = io.out_host.data_ptr()
        if io.packed:
            self.params.block_tables = io.block_ids.data_ptr()
            self.params.block_table_offsets = io.block_offsets.data_ptr()
            self.batch.host_block_tables = io.block_ids_host.data_ptr()
            self.batch.host_block_table_offsets = io.block_offsets_host.data_ptr()
        else:
            self.batch.host_block_tables = io.block_tables_host.data_ptr()
        self.batch.sub_batches = sub_batches
        self.batch.flags = _cabi.STEP_LAST_OUT_DIRECT if last_out_direct else 0
        self.batch.host_staging = io.host.data_ptr()
        self.batch.dev_staging = io.dev.data_ptr()
        self.batch.staging_bytes = io.host.numel()
        self._fn = _cabi.load_library().pa_decode_step_host_batch
        self._device_index = io.device.index if io.device.index is not None else torch.cuda.current_device()

    def plan(self) -> dict:
        """Sub-batch count and bytes moved per step with the host buffers as they are filled now."""
        n, up, down = ctypes.c_uint32(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
        _cabi.check(_cabi.load_library().pa_host_batch_plan(ctypes.byref(self.params), ctypes.byref(self.batch),
                                                            ctypes.byref(n), ctypes.byref(up), ctypes.byref(down)))
        return {"sub_batches": int(n.value), "h2d_bytes": int(up.value), "d2h_bytes": int(down.value)}

    def run(self, synchronize: bool = True) -> torch.Tensor:
        """Uploads, launches and downloads on the current stream (and the library's two copy
        streams); returns the host result, complete if `synchronize`."""
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self.io.device):
                return self.run(synchronize)
        stream = torch.cuda.current_stream(self.io.device).cuda_stream
        rc = self._fn(self.entry, ctypes.byref(self.params), ctypes.byref(self.batch),
                      ctypes.c_void_p(stream), 1 if synchronize else 0)
        if rc != _cabi.PA_OK:
            _cabi.check(rc)
        return self.io.out_host
