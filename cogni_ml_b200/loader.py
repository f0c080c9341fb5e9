"""Streaming upload of raw GGUF tensors to (row-sharded) device buffers.

The reference uploads each tensor with one synchronous cuMemcpyHtoD from pageable memory
(src/ml/cuda/qwen_recurrent_layer_runner.cr:570-587); its tensors are slices of the GGUF mmap
(src/ml/gguf/reader.cr:183-215) whose lifetime Qwen35Weights owns
(src/ml/gguf/qwen35_weights.cr:80-90, 147-160).  Here the bytes go through a small ring of pinned
staging buffers: while one chunk is on its way to the device over a copy stream, the CPU fills the
next buffer from the mmap, so page faults and the host copy overlap the PCIe transfer.  Nothing
is repacked; a rank uploads only the contiguous byte range of its rows.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .quant_matmul import DeviceQuantWeight, QuantWeight, row_bytes
from .sharded import shard_rows


def plan_chunks(nbytes: int, chunk_bytes: int) -> List[Tuple[int, int]]:
    """(offset, size) pieces of a byte range, each at most chunk_bytes, in order."""
    if nbytes < 0 or chunk_bytes <= 0:
        raise ValueError("nbytes must be >= 0 and chunk_bytes > 0")
    return [(o, min(chunk_bytes, nbytes - o)) for o in range(0, nbytes, chunk_bytes)]


class WeightUploader:
    """Uploads QuantWeights through `n_buffers` pinned staging buffers of `chunk_bytes` each."""

    def __init__(self, device="cuda", chunk_bytes: int = 32 << 20, n_buffers: int = 2):
        if not torch.cuda.is_available():
            raise RuntimeError("cogni_ml_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self.device = torch.device(device)
        self.chunk_bytes = int(chunk_bytes)
        self.stream = torch.cuda.Stream(device=self.device)
        self._staging = [torch.empty(self.chunk_bytes, dtype=torch.uint8, pin_memory=True)
                         for _ in range(n_buffers)]
        self._free_at: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self._next = 0
        self.bytes_uploaded = 0

    def upload(self, qw: QuantWeight, row_begin: int = 0, row_end: Optional[int] = None) -> DeviceQuantWeight:
        """Enqueues the copy of rows [row_begin, row_end) and returns the device weight at once;
        its bytes are complete after `finish()` (or after the uploader's stream has been waited on)."""
        row_end = qw.out_dim if row_end is None else row_end
        rb = row_bytes(qw.type, qw.in_dim)
        src = qw.raw[row_begin * rb:row_end * rb]
        dev = torch.empty(src.size, dtype=torch.uint8, device=self.device)
        # the allocation may reuse a block whose last user is still queued on the current stream,
        # and the caching allocator must not hand it out again while the copies are in flight
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        dev.record_stream(self.stream)
        for off, size in plan_chunks(src.size, self.chunk_bytes):
            i = self._next
            self._next = (i + 1) % len(self._staging)
            if self._free_at[i] is not None:
                self._free_at[i].synchronize()          # the buffer's previous chunk has left
            stage = self._staging[i]
            np.copyto(stage.numpy()[:size], src[off:off + size])   # faults the mmap pages in
            with torch.cuda.stream(self.stream):
                dev[off:off + size].copy_(stage[:size], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self._free_at[i] = ev
        self.bytes_uploaded += src.size
        out = DeviceQuantWeight(dev, qw.type, row_end - row_begin, qw.in_dim, row_begin)
        return out

    def upload_shard(self, qw: QuantWeight, rank: int, world: int) -> DeviceQuantWeight:
        r0, r1 = shard_rows(qw.out_dim, rank, world)
        return self.upload(qw, r0, r1)

    def finish(self, weights: Sequence[DeviceQuantWeight] = ()) -> None:
        """Waits for every enqueued copy; the given weights are then marked resident."""
        self.stream.synchronize()
        for w in weights:
            w.resident = True
