"""Host <-> device plumbing of one decode step: one packed upload, one download.

A decode step's host-side inputs are small (query, block tables, context lengths) and its
result is one [S, H, D] fp16 tensor.  Copying them as three separate tensors costs three
transfer latencies; `DecodeStepIO` keeps them in one pinned staging buffer with a device
mirror, so a step is one H2D copy, the kernel launches, one D2H copy and a stream wait.
The KV cache is not part of it: it is state that stays on the device.
"""
from __future__ import annotations

import torch


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
